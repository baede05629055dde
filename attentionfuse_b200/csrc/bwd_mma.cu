// Host side of the tcgen05 backward: support predicate, workspace, TMA descriptors, and the
// three launches (delta, dK/dV, dQ).
#include "bwd_tcgen05.cuh"

namespace af {

namespace {
int64_t align256(int64_t x) { return (x + 255) & ~(int64_t)255; }
}  // namespace

bool bwd_mma_supports(const AfBwdParams& a, const char** why) {
  const AfProblem& p = a.p;
  auto no = [&](const char* w) { if (why) *why = w; return false; };
  if (p.dtype != AF_F16 && p.dtype != AF_BF16) return no("dtype is not f16/bf16");
  if (p.D != 64 && p.D != 128) return no("head_dim is not 64 or 128");
  if (p.norm_kind != AF_NORM_SOFTMAX) return no("normalisation is not softmax");
  if (p.bias_kind == AF_BIAS_ADDITIVE) return no("additive bias");
  if (p.mask_kind == AF_MASK_WINDOW && p.window < 1) return no("window must be positive");
  if (!(p.sm_scale > 0.f)) return no("non-positive scale");
  if (p.N_q < 1 || p.N_kv < 1) return no("empty sequence");
  if (p.mask_kind == AF_MASK_CAUSAL && p.N_q != p.N_kv) return no("causal with N_q != N_kv");
  if (p.mask_kind == AF_MASK_BLOCKS && (p.block_m % 128 != 0 || p.block_n % 128 != 0))
    return no("block size is not a multiple of 128");
  if (!tc_tma_ok(p.q, p.B, p.H_q, p.N_q, p.q_stride) || !tc_tma_ok(p.k, p.B, p.H_kv, p.N_kv, p.k_stride) ||
      !tc_tma_ok(p.v, p.B, p.H_kv, p.N_kv, p.v_stride))
    return no("Q/K/V not TMA-addressable");
  if (a.d_o != nullptr) {   // full parameter block (af_query_family passes only the problem)
    if (!tc_tma_ok(a.d_o, p.B, p.H_q, p.N_q, a.do_stride)) return no("dO not TMA-addressable");
    auto rows_ok = [](const void* ptr, const int64_t* st) {
      return st[3] == 1 && ((uintptr_t)ptr & 15) == 0 && st[2] % 8 == 0 && st[1] % 8 == 0 && st[0] % 8 == 0;
    };
    if (!rows_ok(a.dq, a.dq_stride) || !rows_ok(a.dk, a.dk_stride) || !rows_ok(a.dv, a.dv_stride))
      return no("gradient rows not 16-byte aligned");
    if (p.rope && (a.workspace == nullptr || a.workspace_bytes < bwd_mma_workspace_bytes(a) ||
                   ((uintptr_t)a.workspace & 255) != 0))
      return no("RoPE backward needs workspace for the rotated Q and K");
  }
  if (p.rope && (p.rope_stride_n % 8 != 0 || ((uintptr_t)p.cos & 15) != 0 || ((uintptr_t)p.sin & 15) != 0))
    return no("cos/sin rows not 16-byte aligned");
  return true;
}

int64_t bwd_mma_workspace_bytes(const AfBwdParams& a) {
  const AfProblem& p = a.p;
  if (!p.rope) return 0;
  return align256((int64_t)p.B * p.H_q * p.N_q * p.D * 2) + align256((int64_t)p.B * p.H_kv * p.N_kv * p.D * 2);
}

int launch_bwd_mma(const AfBwdParams& a, cudaStream_t st) {
  const char* why = nullptr;
  if (!bwd_mma_supports(a, &why)) return fail(AF_ERR_UNSUPPORTED, "tensor-core backward: %s", why);
  const AfProblem& p = a.p;
  int rc = launch_bwd_delta(a, st);
  if (rc != AF_OK) return rc;

  const void* q_ptr = p.q;
  const void* k_ptr = p.k;
  int64_t qs[4] = {p.q_stride[0], p.q_stride[1], p.q_stride[2], p.q_stride[3]};
  int64_t ks[4] = {p.k_stride[0], p.k_stride[1], p.k_stride[2], p.k_stride[3]};
  if (p.rope) {
    void* q_rot = a.workspace;
    void* k_rot = static_cast<char*>(a.workspace) + align256((int64_t)p.B * p.H_q * p.N_q * p.D * 2);
    if (!a.workspace_holds_rotated && (rc = tc_launch_prepass(p, q_rot, k_rot, st)) != AF_OK) return rc;
    q_ptr = q_rot; k_ptr = k_rot;
    qs[3] = 1; qs[2] = p.D; qs[1] = (int64_t)p.N_q * p.D; qs[0] = qs[1] * p.H_q;
    ks[3] = 1; ks[2] = p.D; ks[1] = (int64_t)p.N_kv * p.D; ks[0] = ks[1] * p.H_kv;
  }

  CUtensorMap k128, v128, q64, do64, q128, do128, k64, v64;
  if ((rc = tc_make_map(&k128, p.dtype, k_ptr, p.B, p.H_kv, p.N_kv, p.D, ks, 128)) != AF_OK) return rc;
  if ((rc = tc_make_map(&v128, p.dtype, p.v, p.B, p.H_kv, p.N_kv, p.D, p.v_stride, 128)) != AF_OK) return rc;
  if ((rc = tc_make_map(&q64, p.dtype, q_ptr, p.B, p.H_q, p.N_q, p.D, qs, 64)) != AF_OK) return rc;
  if ((rc = tc_make_map(&do64, p.dtype, a.d_o, p.B, p.H_q, p.N_q, p.D, a.do_stride, 64)) != AF_OK) return rc;
  if ((rc = tc_make_map(&q128, p.dtype, q_ptr, p.B, p.H_q, p.N_q, p.D, qs, 128)) != AF_OK) return rc;
  if ((rc = tc_make_map(&do128, p.dtype, a.d_o, p.B, p.H_q, p.N_q, p.D, a.do_stride, 128)) != AF_OK) return rc;
  if ((rc = tc_make_map(&k64, p.dtype, k_ptr, p.B, p.H_kv, p.N_kv, p.D, ks, 64)) != AF_OK) return rc;
  if ((rc = tc_make_map(&v64, p.dtype, p.v, p.B, p.H_kv, p.N_kv, p.D, p.v_stride, 64)) != AF_OK) return rc;

  const bool blocks = p.mask_kind == AF_MASK_BLOCKS;
  tcb::BwdArgs dkv;
  dkv.a = a;
  dkv.tiles = (p.N_kv + 127) / 128;
  dkv.stat_per_block = blocks ? p.block_n / 128 : 1;
  dkv.steps_per_block = blocks ? p.block_m / 64 : 1;
  tcb::BwdArgs dq;
  dq.a = a;
  dq.tiles = (p.N_q + 127) / 128;
  dq.stat_per_block = blocks ? p.block_m / 128 : 1;
  dq.steps_per_block = blocks ? p.block_n / 64 : 1;
  AF_REQUIRE((int64_t)dq.tiles * p.B * p.H_q <= 0x7fffffff, "too many tiles for one launch");
  // Persistent launches: one CTA per SM walks its share of the stationary tiles, so that the loads
  // and first products of the next tile overlap the epilogue of the previous one.
  int dev = 0, sms = 0;
  AF_CUDA_OK(cudaGetDevice(&dev));
  AF_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  dkv.total_items = dkv.tiles * p.B * p.H_kv;
  dq.total_items = dq.tiles * p.B * p.H_q;
  dkv.grid_ctas = (sms > 0 && sms < dkv.total_items) ? sms : dkv.total_items;
  dq.grid_ctas = (sms > 0 && sms < dq.total_items) ? sms : dq.total_items;
  if (blocks) {
    // Block lists make the items uneven in ways the static zig-zag cannot balance (a global key
    // block is visited by every query block): one CTA per item leaves the balancing to the
    // hardware scheduler (BigBird masks at [2,16,8192,64]: 0.94 ms against 1.04 ms persistent).
    dkv.grid_ctas = dkv.total_items;
    dq.grid_ctas = dq.total_items;
  }

  if (p.D == 64) {
    if ((rc = tcb::launch_dkv_d64(p.dtype, dkv, k128, v128, q64, do64, st)) != AF_OK) return rc;
    return tcb::launch_dq_d64(p.dtype, dq, q128, do128, k64, v64, st);
  }
  if ((rc = tcb::launch_dkv_d128(p.dtype, dkv, k128, v128, q64, do64, st)) != AF_OK) return rc;
  return tcb::launch_dq_d128(p.dtype, dq, q128, do128, k64, v64, st);
}

}  // namespace af
