// Exact forward kernel: fp32 FFMA arithmetic for every composition and any head_dim <= 256.
//
// Serves the compositions the tcgen05 kernel does not instantiate: fp32 inputs (whose parity
// bound of 1e-4 rules out single-pass TF32), head dims other than 64/128, additive bias,
// ReLU normalisation and block lists whose block size is not a multiple of 128.  The
// arithmetic follows the reference forward kernel step by step
// (attnfuse/compiler/codegen.py:98-381): scores in fp32, scale, ALiBi / additive bias,
// causal / window / out-of-range masking with -inf, online softmax (or ReLU row sums),
// O = acc / l with l == 0 mapped to 1, L = m + log(l).
//
// Tiling: one CTA of 128 threads owns 32 query rows of one (batch, head) and walks 64-key
// tiles.  Thread (ty, tx) = (tid / 16, tid % 16) owns rows 4*ty..4*ty+3, keys tx + 16*j and
// output columns tx + 16*c, so row reductions stay inside 16-lane groups.
#include "common.cuh"

namespace af {
namespace {

constexpr int TM = 32;
constexpr int TN = 64;
constexpr int NT = 128;

template <typename T>
__device__ __forceinline__ float ld_elem(const void* base, int64_t off) {
  return Elem<T>::to_f32(reinterpret_cast<const T*>(base)[off]);
}

// Rotate-half on a tile held as fp32 in shared memory, then round through T -- the reference
// rotates in fp32 and casts back to the input dtype before the matmul
// (attnfuse/compiler/codegen.py:126-135, 332-341).
template <typename T, int LD>
__device__ __forceinline__ void rope_tile(float* tile, int rows, int pos0, int pos_end, int D,
                                          const void* cos_, const void* sin_, int64_t stride_n) {
  const int half = D / 2;
  for (int idx = threadIdx.x; idx < rows * half; idx += NT) {
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

template <typename T, int DMAX>
__global__ void __launch_bounds__(NT) fwd_ffma_kernel(const AfFwdParams a, const int subs_per_block) {
  constexpr int LD = DMAX + 1;
  constexpr int NC = DMAX / 16;
  const AfProblem& p = a.p;
  extern __shared__ float smem[];
  float* sQ = smem;
  float* sK = sQ + TM * LD;
  float* sV = sK + TN * LD;
  float* sP = sV + TN * LD;  // [TM][TN + 1]

  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int b = blockIdx.y / p.H_q, h = blockIdx.y % p.H_q;
  const int h_kv = h / (p.H_q / p.H_kv);
  const int D = p.D;

  int r0, r_end, qb = 0;
  if (p.mask_kind == AF_MASK_BLOCKS) {
    qb = blockIdx.x / subs_per_block;
    r0 = qb * p.block_m + (blockIdx.x % subs_per_block) * TM;
    r_end = min(qb * p.block_m + p.block_m, p.N_q);
  } else {
    r0 = blockIdx.x * TM;
    r_end = min(r0 + TM, p.N_q);
  }
  if (r0 >= r_end) return;

  const int64_t q_off = (int64_t)b * p.q_stride[0] + (int64_t)h * p.q_stride[1];
  const int64_t k_off = (int64_t)b * p.k_stride[0] + (int64_t)h_kv * p.k_stride[1];
  const int64_t v_off = (int64_t)b * p.v_stride[0] + (int64_t)h_kv * p.v_stride[1];

  for (int idx = tid; idx < TM * DMAX; idx += NT) {
    const int r = idx / DMAX, d = idx - r * DMAX;
    float x = 0.f;
    if (r0 + r < r_end && d < D)
      x = ld_elem<T>(p.q, q_off + (int64_t)(r0 + r) * p.q_stride[2] + (int64_t)d * p.q_stride[3]);
    sQ[r * LD + d] = x;
  }
  __syncthreads();
  if (p.rope) {
    rope_tile<T, LD>(sQ, TM, r0 + p.q_offset, r_end + p.q_offset, D, p.cos, p.sin, p.rope_stride_n);
    __syncthreads();
  }

  const float slope = (p.bias_kind == AF_BIAS_ALIBI) ? load_slope<T>(p.slopes, h) : 0.f;
  float m_i[4], l_i[4], acc[4][NC];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_i[i] = -INFINITY;
    l_i[i] = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[i][c] = 0.f;
  }

  // tile_bits: bit matrix of a partially active tile whose first key is key_base (rows = queries
  // from the block's first row), or nullptr when every element of the tile is active
  const int bit_words = (p.block_n + 63) / 64;
  auto process = [&](const int k0, const int k_end, const uint64_t* tile_bits, const int key_base) {
    for (int idx = tid; idx < TN * DMAX; idx += NT) {
      const int r = idx / DMAX, d = idx - r * DMAX;
      float kx = 0.f, vx = 0.f;
      if (k0 + r < k_end && d < D) {
        kx = ld_elem<T>(p.k, k_off + (int64_t)(k0 + r) * p.k_stride[2] + (int64_t)d * p.k_stride[3]);
        vx = ld_elem<T>(p.v, v_off + (int64_t)(k0 + r) * p.v_stride[2] + (int64_t)d * p.v_stride[3]);
      }
      sK[r * LD + d] = kx;
      sV[r * LD + d] = vx;
    }
    __syncthreads();
    if (p.rope) {
      rope_tile<T, LD>(sK, TN, k0, k_end, D, p.cos, p.sin, p.rope_stride_n);
      __syncthreads();
    }

    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    for (int d = 0; d < D; ++d) {
      float qv[4], kv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = sQ[(ty * 4 + i) * LD + d];
#pragma unroll
      for (int j = 0; j < 4; ++j) kv[j] = sK[(tx + 16 * j) * LD + d];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[i][j] = fmaf(qv[i], kv[j], s[i][j]);
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = r0 + ty * 4 + i;
      const int pos = row + p.q_offset;          // the row's position on the key axis
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = k0 + tx + 16 * j;
        float x = s[i][j] * p.sm_scale;
        if (p.bias_kind == AF_BIAS_ALIBI) {
          x += -slope * (float)abs(pos - key);
        } else if (p.bias_kind == AF_BIAS_ADDITIVE) {
          if (row < p.N_q && key < p.N_kv)
            x += ld_elem<T>(p.bias, (int64_t)b * p.bias_stride[0] + (int64_t)h * p.bias_stride[1] +
                                        (int64_t)row * p.bias_stride[2] + (int64_t)key * p.bias_stride[3]);
        }
        bool keep = key < k_end;
        if (tile_bits != nullptr && keep && row < r_end)
          keep = (tile_bits[(int64_t)(row - qb * p.block_m) * bit_words + ((key - key_base) >> 6)] >> ((key - key_base) & 63)) & 1ull;
        if (p.mask_kind == AF_MASK_CAUSAL) keep = keep && (pos >= key);
        if (p.mask_kind == AF_MASK_WINDOW) keep = keep && (abs(pos - key) < p.window);
        x = keep ? x : -INFINITY;
        s[i][j] = x;
        mx = fmaxf(mx, x);
      }
      if (p.norm_kind == AF_NORM_SOFTMAX) {
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float m_new = fmaxf(m_i[i], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = expf(m_i[i] - m_use);  // exp(-inf) = 0 on the first tile
        float rs = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float e = expf(s[i][j] - m_use);
          s[i][j] = e;
          rs += e;
        }
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
        l_i[i] = alpha * l_i[i] + rs;
        m_i[i] = m_new;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[i][c] *= alpha;
      } else {
        float rs = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float e = fmaxf(s[i][j], 0.f);
          s[i][j] = e;
          rs += e;
        }
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
        l_i[i] += rs;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) sP[(ty * 4 + i) * (TN + 1) + tx + 16 * j] = s[i][j];
    }
    __syncthreads();

    for (int n = 0; n < TN; ++n) {
      float pv[4], vv[NC];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = sP[(ty * 4 + i) * (TN + 1) + n];
#pragma unroll
      for (int c = 0; c < NC; ++c) vv[c] = sV[n * LD + tx + 16 * c];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[i][c] = fmaf(pv[i], vv[c], acc[i][c]);
    }
    __syncthreads();
  };

  if (p.mask_kind == AF_MASK_BLOCKS) {
    const int n = p.kv_num[(int64_t)h * p.kv_num_stride_h + qb];
    const int32_t* list = p.kv_idx + (int64_t)h * p.kv_idx_stride_h + (int64_t)qb * p.kv_idx_stride_q;
    const int32_t* slots = p.kv_slot ? p.kv_slot + (int64_t)h * p.kv_idx_stride_h + (int64_t)qb * p.kv_idx_stride_q : nullptr;
    for (int slot = 0; slot < n; ++slot) {
      const int kb = list[slot];
      const int kb_end = min(kb * p.block_n + p.block_n, p.N_kv);
      const int bs = slots ? slots[slot] : -1;
      const uint64_t* tile_bits = bs >= 0 ? p.kv_bits + (int64_t)bs * p.block_m * bit_words : nullptr;
      for (int k0 = kb * p.block_n; k0 < kb_end; k0 += TN) process(k0, min(k0 + TN, kb_end), tile_bits, kb * p.block_n);
    }
  } else {
    int lo = 0, hi = p.N_kv;
    if (p.mask_kind == AF_MASK_CAUSAL) hi = min(hi, r_end + p.q_offset);
    if (p.mask_kind == AF_MASK_WINDOW) {
      lo = max(0, r0 + p.q_offset - p.window + 1);
      hi = min(hi, r_end + p.q_offset + p.window - 1);
    }
    for (int k0 = lo; k0 < hi; k0 += TN) process(k0, min(k0 + TN, hi), nullptr, 0);
  }

  const int64_t o_off = (int64_t)b * a.o_stride[0] + (int64_t)h * a.o_stride[1];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = r0 + ty * 4 + i;
    if (row >= r_end) continue;
    const float safe_l = (l_i[i] == 0.f) ? 1.f : l_i[i];
    const float inv = 1.f / safe_l;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int d = tx + 16 * c;
      if (d < D)
        reinterpret_cast<T*>(a.o)[o_off + (int64_t)row * a.o_stride[2] + (int64_t)d * a.o_stride[3]] =
            Elem<T>::from_f32(acc[i][c] * inv);
    }
    if (a.lse != nullptr && tx == 0)
      a.lse[(int64_t)b * a.lse_stride[0] + (int64_t)h * a.lse_stride[1] + (int64_t)row * a.lse_stride[2]] =
          m_i[i] + logf(safe_l);
  }
}

template <typename T, int DMAX>
int launch_one(const AfFwdParams& a, cudaStream_t st) {
  const AfProblem& p = a.p;
  const size_t smem = sizeof(float) * ((size_t)(TM + 2 * TN) * (DMAX + 1) + (size_t)TM * (TN + 1));
  auto kern = fwd_ffma_kernel<T, DMAX>;
  AF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int subs = 1, row_tiles;
  if (p.mask_kind == AF_MASK_BLOCKS) {
    subs = (p.block_m + TM - 1) / TM;
    row_tiles = ((p.N_q + p.block_m - 1) / p.block_m) * subs;
  } else {
    row_tiles = (p.N_q + TM - 1) / TM;
  }
  dim3 grid(row_tiles, p.B * p.H_q);
  kern<<<grid, NT, smem, st>>>(a, subs);
  count_launch();
  return check_cuda(cudaGetLastError(), "fwd_ffma launch");
}

template <typename T>
int launch_dtype(const AfFwdParams& a, cudaStream_t st) {
  if (a.p.D <= 64) return launch_one<T, 64>(a, st);
  if (a.p.D <= 128) return launch_one<T, 128>(a, st);
  return launch_one<T, 256>(a, st);
}

}  // namespace

int launch_fwd_ffma(const AfFwdParams& a, cudaStream_t st) {
  if (a.p.N_q == 0 || a.p.B == 0 || a.p.H_q == 0) return AF_OK;
  switch (a.p.dtype) {
    case AF_F16: return launch_dtype<__half>(a, st);
    case AF_BF16: return launch_dtype<__nv_bfloat16>(a, st);
    case AF_F32: return launch_dtype<float>(a, st);
  }
  return fail(AF_ERR_INVALID, "unknown dtype %d", a.p.dtype);
}

}  // namespace af
