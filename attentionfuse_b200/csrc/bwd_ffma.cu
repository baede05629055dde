// Exact backward kernels: fp32 FFMA arithmetic, any composition, any head_dim <= 256.
//
// Same three-step structure as the reference backward (attnfuse/compiler/codegen_backward.py:
// 45-302): delta = rowsum(dO * O); a key-stationary kernel that owns one (key tile, batch,
// kv head), loops over the query heads of its group and the query tiles that can see it,
// and accumulates dK / dV without atomics; a query-stationary kernel that accumulates dQ.
// Scores are recomputed, P = exp(S - L), dS = P * (dP - delta), and dK, dQ are scaled by
// sm_scale at the end.  With RoPE the recompute uses the rotated Q', K' (rounded to the input
// dtype as in the forward) and the epilogue applies the transpose of the rotation to dQ', dK'.
#include "common.cuh"

namespace af {
namespace {

constexpr int BT = 32;   // query rows and keys per tile
constexpr int NT = 128;

template <typename T>
__device__ __forceinline__ float ld_elem(const void* base, int64_t off) {
  return Elem<T>::to_f32(reinterpret_cast<const T*>(base)[off]);
}

template <typename T, int LD>
__device__ __forceinline__ void load_tile(float* dst, const void* src, int64_t off, int64_t s_row,
                                          int64_t s_col, int row0, int row_end, int D, int DMAX) {
  for (int idx = threadIdx.x; idx < BT * DMAX; idx += NT) {
    const int r = idx / DMAX, d = idx - r * DMAX;
    float x = 0.f;
    if (row0 + r < row_end && d < D) x = ld_elem<T>(src, off + (int64_t)(row0 + r) * s_row + (int64_t)d * s_col);
    dst[r * LD + d] = x;
  }
}

template <typename T, int LD>
__device__ __forceinline__ void rope_tile(float* tile, int pos0, int pos_end, int D, const void* cos_,
                                          const void* sin_, int64_t stride_n) {
  const int half = D / 2;
  for (int idx = threadIdx.x; idx < BT * half; idx += NT) {
    const int r = idx / half, d = idx - r * half;
    const int pos = pos0 + r;
    if (pos >= pos_end) continue;
    const int64_t base = (int64_t)pos * stride_n;
    const float c1 = ld_elem<T>(cos_, base + d), s1 = ld_elem<T>(sin_, base + d);
    const float c2 = ld_elem<T>(cos_, base + d + half), s2 = ld_elem<T>(sin_, base + d + half);
    const float x1 = tile[r * LD + d], x2 = tile[r * LD + d + half];
    tile[r * LD + d] = round_through<T>(x1 * c1 - x2 * s1);
    tile[r * LD + d + half] = round_through<T>(x2 * c2 + x1 * s2);
  }
}

// Transpose of the rotation, applied to a gradient tile:  g[d] = g'[d]*cos[d] + g'[d+h]*sin[d+h],
// g[d+h] = g'[d+h]*cos[d+h] - g'[d]*sin[d].
template <typename T, int LD>
__device__ __forceinline__ void unrope_tile(float* tile, int pos0, int pos_end, int D, const void* cos_,
                                            const void* sin_, int64_t stride_n) {
  const int half = D / 2;
  for (int idx = threadIdx.x; idx < BT * half; idx += NT) {
    const int r = idx / half, d = idx - r * half;
    const int pos = pos0 + r;
    if (pos >= pos_end) continue;
    const int64_t base = (int64_t)pos * stride_n;
    const float c1 = ld_elem<T>(cos_, base + d), s1 = ld_elem<T>(sin_, base + d);
    const float c2 = ld_elem<T>(cos_, base + d + half), s2 = ld_elem<T>(sin_, base + d + half);
    const float g1 = tile[r * LD + d], g2 = tile[r * LD + d + half];
    tile[r * LD + d] = g1 * c1 + g2 * s2;
    tile[r * LD + d + half] = g2 * c2 - g1 * s1;
  }
}

template <typename T>
__global__ void bwd_delta_kernel(const AfBwdParams a) {
  const AfProblem& p = a.p;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int64_t total = (int64_t)p.B * p.H_q * p.N_q;
  if (warp >= total) return;
  const int row = warp % p.N_q, h = (warp / p.N_q) % p.H_q, b = warp / ((int64_t)p.N_q * p.H_q);
  const int64_t oo = (int64_t)b * a.o_stride[0] + (int64_t)h * a.o_stride[1] + (int64_t)row * a.o_stride[2];
  const int64_t go = (int64_t)b * a.do_stride[0] + (int64_t)h * a.do_stride[1] + (int64_t)row * a.do_stride[2];
  float s = 0.f;
  for (int d = lane; d < p.D; d += 32)
    s += ld_elem<T>(a.o, oo + (int64_t)d * a.o_stride[3]) * ld_elem<T>(a.d_o, go + (int64_t)d * a.do_stride[3]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) a.delta[warp] = s;
}

// Vector form for 2-byte element types with unit inner strides and 16-byte-aligned rows: LPR
// lanes per row, each with one 16-byte load of O and of dO (8 elements), so that the launch is
// bound by HBM bandwidth rather than by load instructions.
template <typename T, int LPR>
__global__ void bwd_delta_vec_kernel(const AfBwdParams a) {
  const AfProblem& p = a.p;
  const int64_t gthread = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r = gthread / LPR;
  const int sub = (int)(gthread % LPR);
  const int64_t total = (int64_t)p.B * p.H_q * p.N_q;
  float s = 0.f;
  if (r < total) {
    const int row = (int)(r % p.N_q), h = (int)((r / p.N_q) % p.H_q);
    const int64_t b = r / ((int64_t)p.N_q * p.H_q);
    const T* o = reinterpret_cast<const T*>(a.o) + b * a.o_stride[0] + (int64_t)h * a.o_stride[1] + (int64_t)row * a.o_stride[2] + sub * 8;
    const T* g = reinterpret_cast<const T*>(a.d_o) + b * a.do_stride[0] + (int64_t)h * a.do_stride[1] + (int64_t)row * a.do_stride[2] + sub * 8;
    const uint4 ov = *reinterpret_cast<const uint4*>(o), gv = *reinterpret_cast<const uint4*>(g);
    const T* oe = reinterpret_cast<const T*>(&ov);
    const T* ge = reinterpret_cast<const T*>(&gv);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += Elem<T>::to_f32(oe[i]) * Elem<T>::to_f32(ge[i]);
  }
#pragma unroll
  for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (sub == 0 && r < total) a.delta[r] = s;
}

// Recompute one 32x32 tile of P and dS into shared memory.  Thread (ty, tx) owns query rows
// 4*ty..4*ty+3 and keys tx, tx+16.
template <typename T, int LD>
__device__ __forceinline__ void tile_p_ds(const AfBwdParams& a, const float* sQ, const float* sK,
                                          const float* sV, const float* sDO, float* sP, float* sDS,
                                          int b, int h, int m0, int m_end, int n0, int n_end, float slope,
                                          const uint64_t* tile_bits = nullptr, int row_base = 0, int key_base = 0) {
  // tile_bits: query-major bit matrix of a partially active block whose first row / key are
  // row_base / key_base; nullptr when every element of the block is active
  const AfProblem& p = a.p;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float s[4][2], dp[4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) s[i][j] = dp[i][j] = 0.f;
  for (int d = 0; d < p.D; ++d) {
    float qv[4], gv[4], kv[2], vv[2];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      qv[i] = sQ[(ty * 4 + i) * LD + d];
      gv[i] = sDO[(ty * 4 + i) * LD + d];
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      kv[j] = sK[(tx + 16 * j) * LD + d];
      vv[j] = sV[(tx + 16 * j) * LD + d];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[i][j] = fmaf(qv[i], kv[j], s[i][j]);
        dp[i][j] = fmaf(gv[i], vv[j], dp[i][j]);
      }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + ty * 4 + i;
    float L = 0.f, dl = 0.f;
    if (row < m_end) {
      L = a.lse[(int64_t)b * a.lse_stride[0] + (int64_t)h * a.lse_stride[1] + (int64_t)row * a.lse_stride[2]];
      dl = a.delta[((int64_t)b * p.H_q + h) * p.N_q + row];
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int key = n0 + tx + 16 * j;
      float x = s[i][j] * p.sm_scale;
      if (p.bias_kind == AF_BIAS_ALIBI) {
        x += -slope * (float)abs(row - key);
      } else if (p.bias_kind == AF_BIAS_ADDITIVE) {
        if (row < p.N_q && key < p.N_kv)
          x += ld_elem<T>(p.bias, (int64_t)b * p.bias_stride[0] + (int64_t)h * p.bias_stride[1] +
                                      (int64_t)row * p.bias_stride[2] + (int64_t)key * p.bias_stride[3]);
      }
      bool keep = (row < m_end) && (key < n_end);
      if (tile_bits != nullptr && keep)
        keep = (tile_bits[(int64_t)(row - row_base) * ((p.block_n + 63) / 64) + ((key - key_base) >> 6)] >> ((key - key_base) & 63)) & 1ull;
      if (p.mask_kind == AF_MASK_CAUSAL) keep = keep && (row >= key);
      if (p.mask_kind == AF_MASK_WINDOW) keep = keep && (abs(row - key) < p.window);
      // A row with no visible key has L = -inf; its probabilities are zero.
      const float pr = (keep && L != -INFINITY) ? expf(x - L) : 0.f;
      sP[(ty * 4 + i) * (BT + 1) + tx + 16 * j] = pr;
      sDS[(ty * 4 + i) * (BT + 1) + tx + 16 * j] = pr * (dp[i][j] - dl);
    }
  }
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(NT) bwd_dkv_ffma_kernel(const AfBwdParams a, const int subs_per_block) {
  constexpr int LD = DMAX + 1;
  constexpr int NC = DMAX / 16;
  const AfProblem& p = a.p;
  extern __shared__ float smem[];
  float* sK = smem;
  float* sV = sK + BT * LD;
  float* sQ = sV + BT * LD;
  float* sDO = sQ + BT * LD;
  float* sP = sDO + BT * LD;
  float* sDS = sP + BT * (BT + 1);

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int b = blockIdx.y / p.H_kv, h_kv = blockIdx.y % p.H_kv;
  const int group = p.H_q / p.H_kv;
  const int D = p.D;

  int n0, n_end, kb = 0;
  if (p.mask_kind == AF_MASK_BLOCKS) {
    kb = blockIdx.x / subs_per_block;
    n0 = kb * p.block_n + (blockIdx.x % subs_per_block) * BT;
    n_end = min(kb * p.block_n + p.block_n, p.N_kv);
  } else {
    n0 = blockIdx.x * BT;
    n_end = min(n0 + BT, p.N_kv);
  }
  if (n0 >= n_end) return;
  n_end = min(n_end, n0 + BT);

  const int64_t k_off = (int64_t)b * p.k_stride[0] + (int64_t)h_kv * p.k_stride[1];
  const int64_t v_off = (int64_t)b * p.v_stride[0] + (int64_t)h_kv * p.v_stride[1];
  load_tile<T, LD>(sK, p.k, k_off, p.k_stride[2], p.k_stride[3], n0, n_end, D, DMAX);
  load_tile<T, LD>(sV, p.v, v_off, p.v_stride[2], p.v_stride[3], n0, n_end, D, DMAX);
  __syncthreads();
  if (p.rope) {
    rope_tile<T, LD>(sK, n0, n_end, D, p.cos, p.sin, p.rope_stride_n);
    __syncthreads();
  }

  float dk[4][NC], dv[4][NC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) dk[i][c] = dv[i][c] = 0.f;

  for (int g = 0; g < group; ++g) {
    const int h = h_kv * group + g;
    const float slope = (p.bias_kind == AF_BIAS_ALIBI) ? load_slope<T>(p.slopes, h) : 0.f;
    const int64_t q_off = (int64_t)b * p.q_stride[0] + (int64_t)h * p.q_stride[1];
    const int64_t g_off = (int64_t)b * a.do_stride[0] + (int64_t)h * a.do_stride[1];

    auto process = [&](const int m0, const int m_end, const uint64_t* tile_bits, const int row_base) {
      load_tile<T, LD>(sQ, p.q, q_off, p.q_stride[2], p.q_stride[3], m0, m_end, D, DMAX);
      load_tile<T, LD>(sDO, a.d_o, g_off, a.do_stride[2], a.do_stride[3], m0, m_end, D, DMAX);
      __syncthreads();
      if (p.rope) {
        rope_tile<T, LD>(sQ, m0, m_end, D, p.cos, p.sin, p.rope_stride_n);
        __syncthreads();
      }
      tile_p_ds<T, LD>(a, sQ, sK, sV, sDO, sP, sDS, b, h, m0, m_end, n0, n_end, slope, tile_bits, row_base, kb * p.block_n);
      __syncthreads();
      for (int m = 0; m < BT; ++m) {
        float pv[4], sv[4], gv[NC], qv[NC];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pv[i] = sP[m * (BT + 1) + ty * 4 + i];
          sv[i] = sDS[m * (BT + 1) + ty * 4 + i];
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          gv[c] = sDO[m * LD + tx + 16 * c];
          qv[c] = sQ[m * LD + tx + 16 * c];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            dv[i][c] = fmaf(pv[i], gv[c], dv[i][c]);
            dk[i][c] = fmaf(sv[i], qv[c], dk[i][c]);
          }
      }
      __syncthreads();
    };

    if (p.mask_kind == AF_MASK_BLOCKS) {
      const int n = p.q_num[(int64_t)h * p.q_num_stride_h + kb];
      const int32_t* list = p.q_idx + (int64_t)h * p.q_idx_stride_h + (int64_t)kb * p.q_idx_stride_k;
      const int32_t* slots = p.q_slot ? p.q_slot + (int64_t)h * p.q_idx_stride_h + (int64_t)kb * p.q_idx_stride_k : nullptr;
      const int bit_words = (p.block_n + 63) / 64;
      for (int slot = 0; slot < n; ++slot) {
        const int qb = list[slot];
        const int qb_end = min(qb * p.block_m + p.block_m, p.N_q);
        const int bs = slots ? slots[slot] : -1;
        const uint64_t* tile_bits = bs >= 0 ? p.kv_bits + (int64_t)bs * p.block_m * bit_words : nullptr;
        for (int m0 = qb * p.block_m; m0 < qb_end; m0 += BT) process(m0, min(m0 + BT, qb_end), tile_bits, qb * p.block_m);
      }
    } else {
      int lo = 0, hi = p.N_q;
      if (p.mask_kind == AF_MASK_CAUSAL) lo = n0;  // rows i >= key
      if (p.mask_kind == AF_MASK_WINDOW) {
        lo = max(0, n0 - p.window + 1);
        hi = min(hi, n_end + p.window - 1);
      }
      for (int m0 = lo; m0 < hi; m0 += BT) process(m0, min(m0 + BT, hi), nullptr, 0);
    }
  }

  // Epilogue: dK *= scale, undo the rotation, store.
  float* sOut = sQ;  // reuse
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) sOut[(ty * 4 + i) * LD + tx + 16 * c] = dk[i][c] * p.sm_scale;
  __syncthreads();
  if (p.rope) {
    unrope_tile<T, LD>(sOut, n0, n_end, D, p.cos, p.sin, p.rope_stride_n);
    __syncthreads();
  }
  const int64_t dk_off = (int64_t)b * a.dk_stride[0] + (int64_t)h_kv * a.dk_stride[1];
  const int64_t dv_off = (int64_t)b * a.dv_stride[0] + (int64_t)h_kv * a.dv_stride[1];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int key = n0 + ty * 4 + i;
    if (key >= n_end) continue;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int d = tx + 16 * c;
      if (d >= D) continue;
      reinterpret_cast<T*>(a.dk)[dk_off + (int64_t)key * a.dk_stride[2] + (int64_t)d * a.dk_stride[3]] =
          Elem<T>::from_f32(sOut[(ty * 4 + i) * LD + d]);
      reinterpret_cast<T*>(a.dv)[dv_off + (int64_t)key * a.dv_stride[2] + (int64_t)d * a.dv_stride[3]] =
          Elem<T>::from_f32(dv[i][c]);
    }
  }
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(NT) bwd_dq_ffma_kernel(const AfBwdParams a, const int subs_per_block) {
  constexpr int LD = DMAX + 1;
  constexpr int NC = DMAX / 16;
  const AfProblem& p = a.p;
  extern __shared__ float smem[];
  float* sK = smem;
  float* sV = sK + BT * LD;
  float* sQ = sV + BT * LD;
  float* sDO = sQ + BT * LD;
  float* sP = sDO + BT * LD;
  float* sDS = sP + BT * (BT + 1);

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int b = blockIdx.y / p.H_q, h = blockIdx.y % p.H_q;
  const int h_kv = h / (p.H_q / p.H_kv);
  const int D = p.D;

  int m0, m_end, qb = 0;
  if (p.mask_kind == AF_MASK_BLOCKS) {
    qb = blockIdx.x / subs_per_block;
    m0 = qb * p.block_m + (blockIdx.x % subs_per_block) * BT;
    m_end = min(qb * p.block_m + p.block_m, p.N_q);
  } else {
    m0 = blockIdx.x * BT;
    m_end = min(m0 + BT, p.N_q);
  }
  if (m0 >= m_end) return;
  m_end = min(m_end, m0 + BT);

  const int64_t q_off = (int64_t)b * p.q_stride[0] + (int64_t)h * p.q_stride[1];
  const int64_t g_off = (int64_t)b * a.do_stride[0] + (int64_t)h * a.do_stride[1];
  const int64_t k_off = (int64_t)b * p.k_stride[0] + (int64_t)h_kv * p.k_stride[1];
  const int64_t v_off = (int64_t)b * p.v_stride[0] + (int64_t)h_kv * p.v_stride[1];
  load_tile<T, LD>(sQ, p.q, q_off, p.q_stride[2], p.q_stride[3], m0, m_end, D, DMAX);
  load_tile<T, LD>(sDO, a.d_o, g_off, a.do_stride[2], a.do_stride[3], m0, m_end, D, DMAX);
  __syncthreads();
  if (p.rope) {
    rope_tile<T, LD>(sQ, m0, m_end, D, p.cos, p.sin, p.rope_stride_n);
    __syncthreads();
  }
  const float slope = (p.bias_kind == AF_BIAS_ALIBI) ? load_slope<T>(p.slopes, h) : 0.f;

  float dq[4][NC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) dq[i][c] = 0.f;

  auto process = [&](const int n0, const int n_end, const uint64_t* tile_bits, const int key_base) {
    load_tile<T, LD>(sK, p.k, k_off, p.k_stride[2], p.k_stride[3], n0, n_end, D, DMAX);
    load_tile<T, LD>(sV, p.v, v_off, p.v_stride[2], p.v_stride[3], n0, n_end, D, DMAX);
    __syncthreads();
    if (p.rope) {
      rope_tile<T, LD>(sK, n0, n_end, D, p.cos, p.sin, p.rope_stride_n);
      __syncthreads();
    }
    tile_p_ds<T, LD>(a, sQ, sK, sV, sDO, sP, sDS, b, h, m0, m_end, n0, n_end, slope, tile_bits, qb * p.block_m, key_base);
    __syncthreads();
    for (int n = 0; n < BT; ++n) {
      float sv[4], kv[NC];
#pragma unroll
      for (int i = 0; i < 4; ++i) sv[i] = sDS[(ty * 4 + i) * (BT + 1) + n];
#pragma unroll
      for (int c = 0; c < NC; ++c) kv[c] = sK[n * LD + tx + 16 * c];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < NC; ++c) dq[i][c] = fmaf(sv[i], kv[c], dq[i][c]);
    }
    __syncthreads();
  };

  if (p.mask_kind == AF_MASK_BLOCKS) {
    const int n = p.kv_num[(int64_t)h * p.kv_num_stride_h + qb];
    const int32_t* list = p.kv_idx + (int64_t)h * p.kv_idx_stride_h + (int64_t)qb * p.kv_idx_stride_q;
    const int32_t* slots = p.kv_slot ? p.kv_slot + (int64_t)h * p.kv_idx_stride_h + (int64_t)qb * p.kv_idx_stride_q : nullptr;
    const int bit_words = (p.block_n + 63) / 64;
    for (int slot = 0; slot < n; ++slot) {
      const int kb = list[slot];
      const int kb_end = min(kb * p.block_n + p.block_n, p.N_kv);
      const int bs = slots ? slots[slot] : -1;
      const uint64_t* tile_bits = bs >= 0 ? p.kv_bits + (int64_t)bs * p.block_m * bit_words : nullptr;
      for (int n0 = kb * p.block_n; n0 < kb_end; n0 += BT) process(n0, min(n0 + BT, kb_end), tile_bits, kb * p.block_n);
    }
  } else {
    int lo = 0, hi = p.N_kv;
    if (p.mask_kind == AF_MASK_CAUSAL) hi = min(hi, m_end);
    if (p.mask_kind == AF_MASK_WINDOW) {
      lo = max(0, m0 - p.window + 1);
      hi = min(hi, m_end + p.window - 1);
    }
    for (int n0 = lo; n0 < hi; n0 += BT) process(n0, min(n0 + BT, hi), nullptr, 0);
  }

  float* sOut = sK;  // reuse
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) sOut[(ty * 4 + i) * LD + tx + 16 * c] = dq[i][c] * p.sm_scale;
  __syncthreads();
  if (p.rope) {
    unrope_tile<T, LD>(sOut, m0, m_end, D, p.cos, p.sin, p.rope_stride_n);
    __syncthreads();
  }
  const int64_t dq_off = (int64_t)b * a.dq_stride[0] + (int64_t)h * a.dq_stride[1];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + ty * 4 + i;
    if (row >= m_end) continue;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int d = tx + 16 * c;
      if (d < D)
        reinterpret_cast<T*>(a.dq)[dq_off + (int64_t)row * a.dq_stride[2] + (int64_t)d * a.dq_stride[3]] =
            Elem<T>::from_f32(sOut[(ty * 4 + i) * LD + d]);
    }
  }
}

template <typename T, int DMAX>
int launch_one(const AfBwdParams& a, cudaStream_t st) {
  const AfProblem& p = a.p;
  const size_t smem = sizeof(float) * ((size_t)4 * BT * (DMAX + 1) + (size_t)2 * BT * (BT + 1));
  auto kdkv = bwd_dkv_ffma_kernel<T, DMAX>;
  auto kdq = bwd_dq_ffma_kernel<T, DMAX>;
  AF_CUDA_OK(cudaFuncSetAttribute(kdkv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  AF_CUDA_OK(cudaFuncSetAttribute(kdq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));

  { const int rc = launch_bwd_delta(a, st); if (rc != AF_OK) return rc; }
  int subs_n = 1, subs_m = 1, n_tiles, m_tiles;
  if (p.mask_kind == AF_MASK_BLOCKS) {
    subs_n = (p.block_n + BT - 1) / BT;
    subs_m = (p.block_m + BT - 1) / BT;
    n_tiles = ((p.N_kv + p.block_n - 1) / p.block_n) * subs_n;
    m_tiles = ((p.N_q + p.block_m - 1) / p.block_m) * subs_m;
  } else {
    n_tiles = (p.N_kv + BT - 1) / BT;
    m_tiles = (p.N_q + BT - 1) / BT;
  }
  if (n_tiles > 0 && p.B * p.H_kv > 0) {
    kdkv<<<dim3(n_tiles, p.B * p.H_kv), NT, smem, st>>>(a, subs_n);
    count_launch();
    AF_CUDA_OK(cudaGetLastError());
  }
  if (m_tiles > 0 && p.B * p.H_q > 0) {
    kdq<<<dim3(m_tiles, p.B * p.H_q), NT, smem, st>>>(a, subs_m);
    count_launch();
    AF_CUDA_OK(cudaGetLastError());
  }
  return AF_OK;
}

template <typename T>
int launch_dtype(const AfBwdParams& a, cudaStream_t st) {
  if (a.p.D <= 64) return launch_one<T, 64>(a, st);
  if (a.p.D <= 128) return launch_one<T, 128>(a, st);
  return launch_one<T, 256>(a, st);
}

}  // namespace

// delta = rowsum(dO * O), fp32 (B, H_q, N_q); shared by both backward families.
int launch_bwd_delta(const AfBwdParams& a, cudaStream_t st) {
  const int64_t rows = (int64_t)a.p.B * a.p.H_q * a.p.N_q;
  if (rows <= 0) return AF_OK;
  const AfProblem& p = a.p;
  const bool aligned = a.o_stride[3] == 1 && a.do_stride[3] == 1 && ((uintptr_t)a.o & 15) == 0 && ((uintptr_t)a.d_o & 15) == 0 &&
                       a.o_stride[0] % 8 == 0 && a.o_stride[1] % 8 == 0 && a.o_stride[2] % 8 == 0 &&
                       a.do_stride[0] % 8 == 0 && a.do_stride[1] % 8 == 0 && a.do_stride[2] % 8 == 0;
  if (aligned && p.dtype != AF_F32 && (p.D == 64 || p.D == 128 || p.D == 256)) {
    const int lpr = p.D / 8;
    const unsigned vblocks = (unsigned)((rows * lpr + 255) / 256);
#define AF_DELTA_VEC(TYPE)                                                                  \
    if (lpr == 8) bwd_delta_vec_kernel<TYPE, 8><<<vblocks, 256, 0, st>>>(a);                \
    else if (lpr == 16) bwd_delta_vec_kernel<TYPE, 16><<<vblocks, 256, 0, st>>>(a);         \
    else bwd_delta_vec_kernel<TYPE, 32><<<vblocks, 256, 0, st>>>(a);
    if (p.dtype == AF_F16) { AF_DELTA_VEC(__half) } else { AF_DELTA_VEC(__nv_bfloat16) }
#undef AF_DELTA_VEC
    count_launch();
    return check_cuda(cudaGetLastError(), "bwd_delta launch");
  }
  const unsigned blocks = (unsigned)((rows * 32 + 255) / 256);
  switch (a.p.dtype) {
    case AF_F16: bwd_delta_kernel<__half><<<blocks, 256, 0, st>>>(a); break;
    case AF_BF16: bwd_delta_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(a); break;
    case AF_F32: bwd_delta_kernel<float><<<blocks, 256, 0, st>>>(a); break;
    default: return fail(AF_ERR_INVALID, "unknown dtype %d", a.p.dtype);
  }
  count_launch();
  return check_cuda(cudaGetLastError(), "bwd_delta launch");
}

int launch_bwd_ffma(const AfBwdParams& a, cudaStream_t st) {
  switch (a.p.dtype) {
    case AF_F16: return launch_dtype<__half>(a, st);
    case AF_BF16: return launch_dtype<__nv_bfloat16>(a, st);
    case AF_F32: return launch_dtype<float>(a, st);
  }
  return fail(AF_ERR_INVALID, "unknown dtype %d", a.p.dtype);
}

}  // namespace af
