// KV-sharded decode: the exchange of per-rank partials fused into the combine kernels, over
// peer memory (NVLink / NVSwitch), instead of a library all-gather between them.
//
//   combine + push   merges this rank's split-K partials (as decode_combine_kernel does) and
//                    stores the normalised O row and its log-sum-exp straight into slot `rank`
//                    of EVERY rank's exchange buffer with plain peer stores; the last CTA to
//                    finish publishes the step number in every rank's flag word (after one
//                    system-scope fence).
//   wait + merge     spins (bounded) until all ranks' flags show the current step, then merges
//                    the `world` partials from its OWN copy of the buffer and writes O.
//
// Exchange buffer of one rank (symmetric: same layout on all ranks), two parities so that a rank
// that is one step ahead never overwrites what a slower rank still reads:
//     float    o  [2][world][rows][D]
//     float    lse[2][world][rows]
//     uint32_t flag[2][world]
// The step counter lives in local memory (`state[0]`) and is advanced by the kernels themselves,
// so a captured CUDA graph can be replayed.  No cluster-multicast load and no TMA is involved;
// loads are always from the rank's own memory.  The reference is single-GPU: no counterpart.
#include "common.cuh"

namespace af {
namespace {

// Flag store.  Ordering against the data comes from ONE system-scope fence issued before the
// loop over peers; a release store per peer would pay a full system fence each time.
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct Layout {
  int64_t o_floats, lse_floats;   // per parity
  __host__ __device__ Layout(int world, int rows, int D)
      : o_floats((int64_t)world * rows * D), lse_floats((int64_t)world * rows) {}
  __host__ __device__ int64_t o_off(int parity, int src, int rows, int D) const {
    return parity * o_floats + (int64_t)src * rows * D;
  }
  __host__ __device__ int64_t lse_off(int parity, int src, int rows) const {
    return 2 * o_floats + parity * lse_floats + (int64_t)src * rows;
  }
  __host__ __device__ int64_t flag_off_floats() const { return 2 * o_floats + 2 * lse_floats; }
};

// One warp per (batch, head) row; D / 32 floats per lane.
template <int D>
__global__ void decode_combine_push_kernel(const AfDecodeParams a, const AfPeerExchange x) {
  constexpr int VEC = D / 32;
  const int rows = a.B * a.H_q;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const uint32_t step = x.state[0] + 1;          // advanced by the last CTA below
  const int parity = step & 1;
  const Layout lay(x.world, rows, D);
  if (row < rows) {
    const int S = a.num_splits;
    float mstar = -INFINITY;
    for (int s = 0; s < S; ++s) mstar = fmaxf(mstar, a.ws_m[(int64_t)s * rows + row]);
    const float m_use = (mstar == -INFINITY) ? 0.f : mstar;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    float lsum = 0.f;
    for (int s = 0; s < S; ++s) {
      const int64_t r = (int64_t)s * rows + row;
      const float w = expf(a.ws_m[r] - m_use);
      lsum += w * a.ws_l[r];
      const float* src = a.ws_acc + r * D + lane * VEC;
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] += w * src[i];
    }
    const float inv = lsum == 0.f ? 0.f : 1.f / lsum;
    const float lse = lsum == 0.f ? -INFINITY : mstar + logf(lsum);
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] *= inv;
    for (int peer = 0; peer < x.world; ++peer) {
      float* base = reinterpret_cast<float*>(x.peer_bases[peer]);
      float* dst = base + lay.o_off(parity, x.rank, rows, D) + (int64_t)row * D + lane * VEC;
      if constexpr (VEC == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      } else {
        *reinterpret_cast<float2*>(dst) = make_float2(acc[0], acc[1]);
      }
      if (lane == 0) base[lay.lse_off(parity, x.rank, rows) + row] = lse;
    }
  }
  // Publish: the CTA barrier orders every thread's peer stores before thread 0, whose system-scope
  // fence then makes them visible before it counts the CTA in; the last CTA advances the local
  // step and raises this rank's flag on every peer.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t done = atomicAdd(&x.state[1], 1u);
    if (done == gridDim.x - 1) {
      x.state[1] = 0;
      __threadfence_system();
      for (int peer = 0; peer < x.world; ++peer) {
        uint32_t* flags = reinterpret_cast<uint32_t*>(reinterpret_cast<float*>(x.peer_bases[peer]) + lay.flag_off_floats());
        st_relaxed_sys(flags + parity * x.world + x.rank, step);
      }
      x.state[0] = step;
      __threadfence();
    }
  }
}

template <typename T>
__global__ void decode_wait_merge_kernel(const AfPeerExchange x, int rows, int H_q, int D, T* o, int64_t s0, int64_t s1,
                                         int64_t s3) {
  __shared__ int failed;
  const uint32_t step = x.state[0];               // set by the push kernel earlier on this stream
  const int parity = step & 1;
  const Layout lay(x.world, rows, D);
  const float* base = reinterpret_cast<const float*>(x.peer_bases[x.rank]);
  const uint32_t* flags = reinterpret_cast<const uint32_t*>(base + lay.flag_off_floats()) + parity * x.world;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if ((int)threadIdx.x < x.world) {
    const long long limit = x.wait_cycles > 0 ? x.wait_cycles : (1ll << 31);
    const long long t0 = clock64();
    // flags only grow; a flag at or past `step` (modulo wrap) means that rank's partial landed
    while ((int32_t)(ld_acquire_sys(flags + threadIdx.x) - step) < 0) {
      if (clock64() - t0 > limit) {
        failed = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (failed) {
    if (threadIdx.x == 0 && x.status != nullptr) atomicExch(x.status, AF_STATUS_WAIT_TIMEOUT);
    return;
  }
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  // all log-sum-exps first (independent loads), then the weighted rows
  float w[32];
  float mstar = -INFINITY;
#pragma unroll 8
  for (int r = 0; r < x.world; ++r) {
    w[r & 31] = base[lay.lse_off(parity, r, rows) + row];
    mstar = fmaxf(mstar, w[r & 31]);
  }
  const float m_use = (mstar == -INFINITY) ? 0.f : mstar;
  float wsum = 0.f;
#pragma unroll 8
  for (int r = 0; r < x.world; ++r) {
    w[r & 31] = (w[r & 31] == -INFINITY) ? 0.f : expf(w[r & 31] - m_use);
    wsum += w[r & 31];
  }
  const float inv = (mstar == -INFINITY) ? 0.f : 1.f / wsum;
  T* dst = o + (int64_t)(row / H_q) * s0 + (int64_t)(row % H_q) * s1;
  for (int d = lane; d < D; d += 32) {
    float acc = 0.f;
#pragma unroll 8
    for (int r = 0; r < x.world; ++r)
      if (w[r & 31] != 0.f) acc += w[r & 31] * base[lay.o_off(parity, r, rows, D) + (int64_t)row * D + d];
    dst[(int64_t)d * s3] = Elem<T>::from_f32(acc * inv);
  }
}

int check_exchange(const AfPeerExchange* x) {
  AF_REQUIRE(x != nullptr, "exchange is NULL");
  AF_REQUIRE(x->world >= 1 && x->world <= 32 && x->rank >= 0 && x->rank < x->world, "bad rank/world %d/%d", x->rank,
             x->world);
  AF_REQUIRE(x->peer_bases != nullptr && x->state != nullptr, "exchange pointers must be non-NULL");
  return AF_OK;
}

}  // namespace

int64_t decode_exchange_bytes(int world, int B, int H_q, int D) {
  const Layout lay(world, B * H_q, D);
  return (lay.flag_off_floats() + 2 * world) * 4;
}

int launch_decode_combine_push(const AfDecodeParams& a, const AfPeerExchange* x, cudaStream_t st) {
  int rc = check_exchange(x);
  if (rc != AF_OK) return rc;
  AF_REQUIRE(a.D == 64 || a.D == 128, "decode kernels are instantiated for D in {64,128} (got %d)", a.D);
  AF_REQUIRE(a.ws_m && a.ws_l && a.ws_acc && a.num_splits >= 1 && a.B > 0 && a.H_q > 0, "bad decode parameters");
  AF_REQUIRE(((uintptr_t)a.ws_acc & 15) == 0, "ws_acc must be 16-byte aligned");
  AF_REQUIRE(a.balanced_ctas == 0, "the two-kernel exchange takes the per-unit split grid (balanced_ctas = 0)");
  const int rows = a.B * a.H_q;
  if (a.D == 64)
    decode_combine_push_kernel<64><<<(rows + 3) / 4, 128, 0, st>>>(a, *x);
  else
    decode_combine_push_kernel<128><<<(rows + 3) / 4, 128, 0, st>>>(a, *x);
  count_launch();
  return check_cuda(cudaGetLastError(), "decode_combine_push launch");
}

int launch_decode_wait_merge(const AfPeerExchange* x, int B, int H_q, int D, int dtype, void* o, const int64_t* os,
                             cudaStream_t st) {
  int rc = check_exchange(x);
  if (rc != AF_OK) return rc;
  AF_REQUIRE(o && os && B > 0 && H_q > 0 && D > 0, "bad merge arguments");
  const int rows = B * H_q;
  const unsigned blocks = (rows + 3) / 4;
  if (dtype == AF_F16)
    decode_wait_merge_kernel<__half><<<blocks, 128, 0, st>>>(*x, rows, H_q, D, (__half*)o, os[0], os[1], os[3]);
  else if (dtype == AF_BF16)
    decode_wait_merge_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>(*x, rows, H_q, D, (__nv_bfloat16*)o, os[0], os[1], os[3]);
  else if (dtype == AF_F32)
    decode_wait_merge_kernel<float><<<blocks, 128, 0, st>>>(*x, rows, H_q, D, (float*)o, os[0], os[1], os[3]);
  else
    return fail(AF_ERR_INVALID, "unknown dtype %d", dtype);
  count_launch();
  return check_cuda(cudaGetLastError(), "decode_wait_merge launch");
}

}  // namespace af
