// Host side of the tcgen05 backward: support predicate, workspace, TMA descriptors, and the
// launches: delta, then either the two passes (dK/dV, dQ) or -- head_dim 128 with a dQ
// accumulator from the caller -- the single fused pass followed by the dQ finishing kernel.
#include <cstdlib>

#include "bwd_tcgen05.cuh"

namespace af {

namespace {
int64_t align256(int64_t x) { return (x + 255) & ~(int64_t)255; }

// dQ accumulator of the fused pass: fp32 (B, H_q, N_q, D), then 256 bytes holding the item counter.
int64_t dq_accum_floats(const AfProblem& p) { return (int64_t)p.B * p.H_q * p.N_q * p.D; }

// dq = T(scale * R^T(acc)): the fused pass leaves scale-free, still-rotated sums in `acc`.  One
// thread per pair of 8-element chunks (d, d + D/2) of one row.
template <typename T, int D, bool ROPE>
__global__ void bwd_dq_finish_kernel(const float* __restrict__ acc, const AfBwdParams a, int64_t rows) {
  constexpr int HC = D / 16;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = idx / HC;
  const int c = (int)(idx - row * HC);
  if (row >= rows) return;
  const AfProblem& p = a.p;
  const int n = (int)(row % p.N_q);
  const int64_t bh = row / p.N_q;
  const int h = (int)(bh % p.H_q), b = (int)(bh / p.H_q);
  const float4* src_lo = reinterpret_cast<const float4*>(acc + row * D + c * 8);
  const float4* src_hi = reinterpret_cast<const float4*>(acc + row * D + D / 2 + c * 8);
  const float4 l0 = src_lo[0], l1 = src_lo[1], h0 = src_hi[0], h1 = src_hi[1];
  float gl[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
  float gh[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) { gl[i] *= p.sm_scale; gh[i] *= p.sm_scale; }
  if (ROPE) {
    const T* cos_row = reinterpret_cast<const T*>(p.cos) + (int64_t)n * p.rope_stride_n;
    const T* sin_row = reinterpret_cast<const T*>(p.sin) + (int64_t)n * p.rope_stride_n;
    const uint4 cl = __ldg(reinterpret_cast<const uint4*>(cos_row + c * 8));
    const uint4 ch = __ldg(reinterpret_cast<const uint4*>(cos_row + D / 2 + c * 8));
    const uint4 sl = __ldg(reinterpret_cast<const uint4*>(sin_row + c * 8));
    const uint4 sh = __ldg(reinterpret_cast<const uint4*>(sin_row + D / 2 + c * 8));
    const uint32_t clw[4] = {cl.x, cl.y, cl.z, cl.w}, chw[4] = {ch.x, ch.y, ch.z, ch.w};
    const uint32_t slw[4] = {sl.x, sl.y, sl.z, sl.w}, shw[4] = {sh.x, sh.y, sh.z, sh.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 c1 = tc::Pack2<T>::unpack(clw[i]), c2 = tc::Pack2<T>::unpack(chw[i]);
      const float2 s1 = tc::Pack2<T>::unpack(slw[i]), s2 = tc::Pack2<T>::unpack(shw[i]);
      const float a0 = gl[2 * i], a1 = gl[2 * i + 1], b0 = gh[2 * i], b1 = gh[2 * i + 1];
      // transpose of the rotation, as in the two-pass epilogue
      gl[2 * i] = a0 * c1.x + b0 * s2.x;     gl[2 * i + 1] = a1 * c1.y + b1 * s2.y;
      gh[2 * i] = b0 * c2.x - a0 * s1.x;     gh[2 * i + 1] = b1 * c2.y - a1 * s1.y;
    }
  }
  T* dst = reinterpret_cast<T*>(a.dq) + (int64_t)b * a.dq_stride[0] + (int64_t)h * a.dq_stride[1] + (int64_t)n * a.dq_stride[2];
  uint4 vl, vh;
  vl.x = tc::Pack2<T>::run(gl[0], gl[1]); vl.y = tc::Pack2<T>::run(gl[2], gl[3]);
  vl.z = tc::Pack2<T>::run(gl[4], gl[5]); vl.w = tc::Pack2<T>::run(gl[6], gl[7]);
  vh.x = tc::Pack2<T>::run(gh[0], gh[1]); vh.y = tc::Pack2<T>::run(gh[2], gh[3]);
  vh.z = tc::Pack2<T>::run(gh[4], gh[5]); vh.w = tc::Pack2<T>::run(gh[6], gh[7]);
  *reinterpret_cast<uint4*>(dst + c * 8) = vl;
  *reinterpret_cast<uint4*>(dst + D / 2 + c * 8) = vh;
}

template <typename T>
int launch_dq_finish(const float* acc, const AfBwdParams& a, cudaStream_t st) {
  constexpr int D = 128;
  const int64_t rows = (int64_t)a.p.B * a.p.H_q * a.p.N_q;
  const unsigned blocks = (unsigned)((rows * (D / 16) + 255) / 256);
  if (a.p.rope) bwd_dq_finish_kernel<T, D, true><<<blocks, 256, 0, st>>>(acc, a, rows);
  else bwd_dq_finish_kernel<T, D, false><<<blocks, 256, 0, st>>>(acc, a, rows);
  count_launch();
  return check_cuda(cudaGetLastError(), "bwd_dq_finish launch");
}
}  // namespace

// The fused single-pass kernel exists for head_dim 128 (dQ^T is produced with M = head_dim).
int64_t bwd_mma_dq_accum_bytes(const AfBwdParams& a) {
  if (a.p.D != 128 || !bwd_mma_supports(a, nullptr)) return 0;
  return align256(dq_accum_floats(a.p) * 4) + 256;
}

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
  if (p.mask_kind == AF_MASK_BLOCKS && (p.kv_slot || p.q_slot) && !(p.kv_slot && p.q_slot && p.kv_bits && p.q_bits))
    return no("element bit matrices need both list orientations (kv_slot, q_slot, kv_bits, q_bits)");
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

  const int64_t acc_bytes = bwd_mma_dq_accum_bytes(a);
  if (acc_bytes > 0 && a.dq_accum != nullptr && a.dq_accum_bytes >= acc_bytes && ((uintptr_t)a.dq_accum & 255) == 0) {
    // ---- single fused pass: dK, dV and dQ from one recompute of S and dP ----
    tcb::BwdArgs f{};
    f.a = a;
    const bool blk = p.mask_kind == AF_MASK_BLOCKS;
    f.tiles = (p.N_kv + 127) / 128;
    f.stat_per_block = blk ? p.block_n / 128 : 1;
    f.steps_per_block = blk ? p.block_m / 64 : 1;
    const int64_t units = (int64_t)p.B * p.H_kv;
    AF_REQUIRE((int64_t)f.tiles * units <= 0x7fffffff - 1024, "too many tiles for one launch");
    f.total_items = (int)(f.tiles * units);
    int sms = 0;
    if ((rc = tc_sm_count(&sms)) != AF_OK) return rc;
    f.grid_ctas = (sms > 0 && sms < f.total_items) ? sms : f.total_items;
    // Scheduling chunk: as many (batch, kv head) units as keep their dQ accumulator rows (fp32)
    // and their Q / dO rows inside the L2 (measured at B4 H32/8 N4096: 2 units 2.30 ms, 3: 2.25,
    // 8: 2.24, all 32: 2.37 for the whole training step).
    const int64_t per_unit = (int64_t)(p.H_q / p.H_kv) * p.N_q * p.D * (4 + 2 + 2);
    int64_t chunk = (128ll << 20) / (per_unit > 0 ? per_unit : 1);
    if (const char* env = getenv("ATTNFUSE_BWD_CHUNK")) chunk = atoll(env);
    if (chunk < 1) chunk = 1;
    if (chunk > units) chunk = units;
    f.chunk_units = (int)chunk;
    f.dq_acc = static_cast<float*>(a.dq_accum);
    f.sched_counter = reinterpret_cast<int32_t*>(static_cast<char*>(a.dq_accum) + align256(dq_accum_floats(p) * 4));
    AF_CUDA_OK(cudaMemsetAsync(a.dq_accum, 0, (size_t)acc_bytes, st));
    if ((rc = tcb::launch_fused_d128(p.dtype, f, k128, v128, q64, do64, st)) != AF_OK) return rc;
    return p.dtype == AF_F16 ? launch_dq_finish<__half>(f.dq_acc, a, st) : launch_dq_finish<__nv_bfloat16>(f.dq_acc, a, st);
  }
  if ((rc = tc_make_map(&q128, p.dtype, q_ptr, p.B, p.H_q, p.N_q, p.D, qs, 128)) != AF_OK) return rc;
  if ((rc = tc_make_map(&do128, p.dtype, a.d_o, p.B, p.H_q, p.N_q, p.D, a.do_stride, 128)) != AF_OK) return rc;
  if ((rc = tc_make_map(&k64, p.dtype, k_ptr, p.B, p.H_kv, p.N_kv, p.D, ks, 64)) != AF_OK) return rc;
  if ((rc = tc_make_map(&v64, p.dtype, p.v, p.B, p.H_kv, p.N_kv, p.D, p.v_stride, 64)) != AF_OK) return rc;

  const bool blocks = p.mask_kind == AF_MASK_BLOCKS;
  tcb::BwdArgs dkv{};
  dkv.a = a;
  dkv.tiles = (p.N_kv + 127) / 128;
  dkv.stat_per_block = blocks ? p.block_n / 128 : 1;
  dkv.steps_per_block = blocks ? p.block_m / 64 : 1;
  tcb::BwdArgs dq{};
  dq.a = a;
  dq.tiles = (p.N_q + 127) / 128;
  dq.stat_per_block = blocks ? p.block_m / 128 : 1;
  dq.steps_per_block = blocks ? p.block_n / 64 : 1;
  AF_REQUIRE((int64_t)dq.tiles * p.B * p.H_q <= 0x7fffffff, "too many tiles for one launch");
  // Persistent launches: one CTA per SM walks its share of the stationary tiles, so that the loads
  // and first products of the next tile overlap the epilogue of the previous one.
  int sms = 0;
  if ((rc = tc_sm_count(&sms)) != AF_OK) return rc;
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
