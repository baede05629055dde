// extern "C" entry points: argument validation, kernel-family selection, error strings.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace af {

static thread_local char g_error[512] = "";
static std::atomic<int64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return AF_OK;
  return fail(AF_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

namespace {

int validate_problem(const AfProblem& p) {
  AF_REQUIRE(p.dtype == AF_F16 || p.dtype == AF_BF16 || p.dtype == AF_F32, "unknown dtype %d", p.dtype);
  AF_REQUIRE(p.B >= 0 && p.H_q >= 1 && p.H_kv >= 1 && p.N_q >= 0 && p.N_kv >= 0, "negative extent");
  AF_REQUIRE(p.H_q % p.H_kv == 0, "Q heads (%d) must be a multiple of KV heads (%d)", p.H_q, p.H_kv);
  AF_REQUIRE(p.D >= 1 && p.D <= 256, "head_dim %d outside [1, 256]", p.D);
  AF_REQUIRE(p.mask_kind >= AF_MASK_FULL && p.mask_kind <= AF_MASK_BLOCKS, "unknown mask_kind %d", p.mask_kind);
  AF_REQUIRE(p.bias_kind >= AF_BIAS_NONE && p.bias_kind <= AF_BIAS_ADDITIVE, "unknown bias_kind %d", p.bias_kind);
  AF_REQUIRE(p.norm_kind == AF_NORM_SOFTMAX || p.norm_kind == AF_NORM_RELU, "unknown norm_kind %d", p.norm_kind);
  AF_REQUIRE(p.q && p.k && p.v, "q/k/v must be non-NULL");
  AF_REQUIRE((int64_t)p.B * p.H_q <= 65535, "B*H_q exceeds the launch grid limit");
  AF_REQUIRE(p.q_offset >= 0, "q_offset must be non-negative (got %d)", p.q_offset);
  if (p.mask_kind == AF_MASK_WINDOW) AF_REQUIRE(p.window > 0, "window must be positive");
  if (p.mask_kind == AF_MASK_BLOCKS) {
    AF_REQUIRE(p.block_m > 0 && p.block_n > 0, "block sizes must be positive");
    AF_REQUIRE(p.kv_num && p.kv_idx, "block lists (kv_num, kv_idx) must be non-NULL");
    if (p.kv_slot || p.q_slot) AF_REQUIRE(p.kv_bits != nullptr, "bit-matrix numbers (kv_slot / q_slot) need kv_bits");
  }
  if (p.bias_kind == AF_BIAS_ALIBI) AF_REQUIRE(p.slopes != nullptr, "ALiBi needs slopes");
  if (p.bias_kind == AF_BIAS_ADDITIVE) AF_REQUIRE(p.bias != nullptr, "additive bias needs a bias tensor");
  if (p.rope) {
    AF_REQUIRE(p.cos && p.sin, "RoPE needs cos and sin tables");
    AF_REQUIRE(p.D % 2 == 0, "RoPE needs an even head_dim");
  }
  return AF_OK;
}

}  // namespace
}  // namespace af

using namespace af;

extern "C" {

int af_fwd(const AfFwdParams* params, af_stream_t stream) {
  if (params == nullptr) return fail(AF_ERR_INVALID, "params is NULL");
  const AfFwdParams& a = *params;
  int rc = validate_problem(a.p);
  if (rc != AF_OK) return rc;
  AF_REQUIRE(a.o != nullptr, "o must be non-NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const char* why = nullptr;
  const bool tc_ok = fwd_tcgen05_supports(a.p, a.o, a.o_stride, &why);
  if (a.p.family == AF_FAMILY_TCGEN05) {
    if (!tc_ok) return fail(AF_ERR_UNSUPPORTED, "tcgen05 forward: %s", why);
    return launch_fwd_tcgen05(a, st);
  }
  if (a.p.family == AF_FAMILY_AUTO && tc_ok) return launch_fwd_tcgen05(a, st);
  return launch_fwd_ffma(a, st);
}

int64_t af_fwd_workspace_bytes(const AfFwdParams* params) {
  if (params == nullptr) return 0;
  const AfFwdParams& a = *params;
  if (a.p.family == AF_FAMILY_FFMA || !fwd_tcgen05_supports(a.p, a.o, a.o_stride, nullptr)) return 0;
  return fwd_tcgen05_workspace_bytes(a.p);
}

int af_bwd(const AfBwdParams* params, af_stream_t stream) {
  if (params == nullptr) return fail(AF_ERR_INVALID, "params is NULL");
  const AfBwdParams& a = *params;
  int rc = validate_problem(a.p);
  if (rc != AF_OK) return rc;
  AF_REQUIRE(a.p.norm_kind == AF_NORM_SOFTMAX, "backward is defined for softmax normalisation only");
  AF_REQUIRE(a.p.q_offset == 0, "backward does not take a query position offset");
  AF_REQUIRE(a.o && a.d_o && a.lse && a.delta && a.dq && a.dk && a.dv, "NULL backward operand");
  if (a.p.mask_kind == AF_MASK_BLOCKS) AF_REQUIRE(a.p.q_num && a.p.q_idx, "backward needs key-major block lists");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const char* why = nullptr;
  const bool mma_ok = bwd_mma_supports(a, &why);
  if (a.p.family == AF_FAMILY_TCGEN05) {
    if (!mma_ok) return fail(AF_ERR_UNSUPPORTED, "tensor-core backward: %s", why);
    return launch_bwd_mma(a, st);
  }
  if (a.p.family == AF_FAMILY_AUTO && mma_ok) return launch_bwd_mma(a, st);
  return launch_bwd_ffma(a, st);
}

int64_t af_bwd_workspace_bytes(const AfBwdParams* params) {
  if (params == nullptr || params->p.family == AF_FAMILY_FFMA) return 0;
  return bwd_mma_workspace_bytes(*params);
}

int64_t af_bwd_dq_accum_bytes(const AfBwdParams* params) {
  if (params == nullptr || params->p.family == AF_FAMILY_FFMA) return 0;
  return bwd_mma_dq_accum_bytes(*params);
}

int af_decode_split(const AfDecodeParams* params, af_stream_t stream) {
  if (params == nullptr) return fail(AF_ERR_INVALID, "params is NULL");
  return launch_decode_split(*params, static_cast<cudaStream_t>(stream));
}

int af_decode_combine(const AfDecodeParams* params, af_stream_t stream) {
  if (params == nullptr) return fail(AF_ERR_INVALID, "params is NULL");
  return launch_decode_combine(*params, static_cast<cudaStream_t>(stream));
}

int af_decode_static(const AfDecodeParams* params, af_stream_t stream) {
  if (params == nullptr) return fail(AF_ERR_INVALID, "params is NULL");
  return launch_decode_static(*params, static_cast<cudaStream_t>(stream));
}

int af_decode_combine_gathered(const float* gathered, int32_t G, int32_t B, int32_t H_q, int32_t D, int32_t dtype,
                               void* o, const int64_t o_stride[4], af_stream_t stream) {
  return launch_decode_combine_gathered(gathered, G, B, H_q, D, dtype, o, o_stride, static_cast<cudaStream_t>(stream));
}

int64_t af_decode_exchange_bytes(int32_t world, int32_t B, int32_t H_q, int32_t D) {
  if (world < 1 || B < 1 || H_q < 1 || D < 1) return 0;
  return decode_exchange_bytes(world, B, H_q, D);
}

int af_decode_combine_push(const AfDecodeParams* params, const AfPeerExchange* exchange, af_stream_t stream) {
  if (params == nullptr) return fail(AF_ERR_INVALID, "params is NULL");
  return launch_decode_combine_push(*params, exchange, static_cast<cudaStream_t>(stream));
}

int af_decode_sharded_step(const AfDecodeParams* params, const AfPeerExchange* exchange, int32_t mode, af_stream_t stream) {
  if (params == nullptr) return fail(AF_ERR_INVALID, "params is NULL");
  return launch_decode_sharded_step(*params, exchange, mode, static_cast<cudaStream_t>(stream));
}

int af_decode_wait_merge(const AfPeerExchange* exchange, int32_t B, int32_t H_q, int32_t D, int32_t dtype, void* o,
                         const int64_t o_stride[4], af_stream_t stream) {
  return launch_decode_wait_merge(exchange, B, H_q, D, dtype, o, o_stride, static_cast<cudaStream_t>(stream));
}

int32_t af_decode_num_splits(int32_t B, int32_t H_q, int32_t H_kv, int32_t N_kv, int32_t sm_count, int32_t ragged) {
  // Bandwidth-bound groups (<= 16 query heads per KV head): one CTA per (split, batch, kv head),
  // two CTAs resident per SM, about five waves of CTAs so that the ragged tail of per-sequence
  // lengths averages out.  Keep at least 512 keys per split so the pipeline prologue amortises;
  // cap at 64.
  if (sm_count <= 0) sm_count = 148;
  if (B < 1) B = 1;
  if (H_kv < 1) H_kv = 1;
  const int group = H_q > H_kv ? H_q / H_kv : 1;
  const int64_t units = (int64_t)B * H_kv * ((group + 63) / 64);
  int64_t want;
  if (group > 16) {
    // Tensor-bound groups run on the persistent tcgen05 kernel, one CTA per SM: long items
    // amortise the per-item prologue and epilogue, so aim at one or two items per CTA, whichever
    // fills the SMs better (never one item more than a whole number of rounds).
    const int64_t s1 = sm_count / units > 0 ? sm_count / units : 1;
    const int64_t s2 = 2LL * sm_count / units > 0 ? 2LL * sm_count / units : 1;
    auto fill = [&](int64_t s) {
      const int64_t items = units * s, rounds = (items + sm_count - 1) / sm_count;
      return (double)items / (double)(rounds * sm_count);
    };
    want = fill(s2) > fill(s1) + 1e-9 ? s2 : s1;
  } else {
    const int64_t slots = 2LL * sm_count;          // CTAs resident at once
    want = (5 * slots + units - 1) / units;
    // Whole waves: with equal-length sequences every CTA takes the same time, so a last wave that
    // fills a fifth of the slots costs as much as a full one.  Among the split counts around the
    // five-wave target take the one whose last wave is fullest (B16 H32/8 L32768: 16 splits 0.318 ms
    // against 0.332 ms with 12).  Ragged lengths even out by themselves and prefer fewer, longer
    // CTAs (12 splits 0.243 ms against 0.249 ms with 16).
    const int64_t cap0 = N_kv / 512 > 1 ? N_kv / 512 : 1;
    const int64_t hi = (want * 3 / 2 < cap0 ? want * 3 / 2 : cap0) < 64 ? (want * 3 / 2 < cap0 ? want * 3 / 2 : cap0) : 64;
    const int64_t lo = want * 3 / 4 > 1 ? want * 3 / 4 : 1;
    double best = -1.0;
    int64_t pick = want;
    for (int64_t s = lo; s <= hi; ++s) {
      const int64_t ctas = units * s, waves = (ctas + slots - 1) / slots;
      const double fill = (double)ctas / (double)(waves * slots);
      const int64_t dist = s > want ? s - want : want - s, best_dist = pick > want ? pick - want : want - pick;
      if (fill > best + 1e-9 || (fill > best - 1e-9 && dist < best_dist)) { best = fill; pick = s; }
    }
    if (hi >= lo && !ragged) want = pick;
  }
  const int64_t cap = N_kv / 512 > 1 ? N_kv / 512 : 1;
  if (want > cap) want = cap;
  if (want > 64) want = 64;
  if (want < 1) want = 1;
  return (int32_t)want;
}

int32_t af_query_family(const AfProblem* p, int32_t backward) {
  if (p == nullptr) return fail(AF_ERR_INVALID, "problem is NULL");
  if (backward) {
    AfBwdParams b{};
    b.p = *p;
    return bwd_mma_supports(b, nullptr) ? AF_FAMILY_TCGEN05 : AF_FAMILY_FFMA;
  }
  int64_t os[4] = {p->q_stride[0], p->q_stride[1], p->q_stride[2], p->q_stride[3]};
  return fwd_tcgen05_supports(*p, p->q, os, nullptr) ? AF_FAMILY_TCGEN05 : AF_FAMILY_FFMA;
}

int64_t af_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char* af_last_error(void) { return g_error; }
int32_t af_abi_version(void) { return AF_ABI_VERSION; }

}  // extern "C"
