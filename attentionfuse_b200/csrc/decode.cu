// Split-K flash-decoding for query length 1 (GQA / MQA), plus the log-sum-exp combine.
//
// Replaces the reference's two decode kernels (attnfuse/compiler/codegen_decode.py:46-211).
// The work is bound by HBM: every K and V byte is read exactly once.  One CTA owns one
// (split, batch, kv head) and serves all query heads of the group from the same K/V tiles,
// so the cache is streamed once per group rather than once per query head.
//
//   * K/V tiles of 64 keys are streamed with 16-byte cp.async into a 3-stage ring in shared
//     memory (XOR-swizzled 16-byte chunks, so ldmatrix is bank-conflict free); rows past the
//     valid length are zero-filled by the copy itself.
//   * The query heads of the group sit on the M side of mma.sync.m16n8k16 (padded to 16 rows,
//     as the reference pads to BLOCK_H = 16).  For groups <= 16 the four warps split the 64
//     keys of a tile and merge their partial (m, l, acc) at the end; for larger groups (MQA)
//     each warp owns 16 heads and sees all keys.
//   * Partial results go to fp32 workspaces; a vectorised combine kernel merges the splits.
//
// Per-sequence valid lengths (kv_lens) are an extension: the reference only has a scalar N_KV.
#include <mutex>

#include "common.cuh"

namespace af {
namespace {

constexpr int DEC_BN = 64;       // keys per pipeline stage
constexpr int DEC_STAGES = 3;
constexpr int DEC_THREADS = 128;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <typename T> struct MmaOp;
template <> struct MmaOp<__half> {
  __device__ __forceinline__ static void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct MmaOp<__nv_bfloat16> {
  __device__ __forceinline__ static void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// Byte offset of 16-byte chunk `c` of key row `r` inside a [DEC_BN][D] tile.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
  constexpr int ROW_BYTES = D * 2;
  return (uint32_t)(r * ROW_BYTES + (((c & ~7) | ((c ^ r) & 7)) << 4));
}

// Unpack / pack two elements of T.
template <typename T> struct Pair;
template <> struct Pair<__half> {
  __device__ __forceinline__ static float2 unpack(uint32_t x) { return __half22float2(*reinterpret_cast<__half2*>(&x)); }
};
template <> struct Pair<__nv_bfloat16> {
  __device__ __forceinline__ static float2 unpack(uint32_t x) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&x)); }
};

// Rotate-half on two packed pairs: (lo, hi) are elements (d, d+1) and (d + D/2, d + D/2 + 1);
// fp32 math, one rounding to T -- the rounding point of the forward kernels.
template <typename T>
__device__ __forceinline__ void rotate_words(uint32_t& lo, uint32_t& hi, uint32_t c_lo, uint32_t c_hi, uint32_t s_lo,
                                             uint32_t s_hi) {
  const float2 x1 = Pair<T>::unpack(lo), x2 = Pair<T>::unpack(hi);
  const float2 c1 = Pair<T>::unpack(c_lo), c2 = Pair<T>::unpack(c_hi);
  const float2 s1 = Pair<T>::unpack(s_lo), s2 = Pair<T>::unpack(s_hi);
  lo = MmaOp<T>::pack(x1.x * c1.x - x2.x * s1.x, x1.y * c1.y - x2.y * s1.y);
  hi = MmaOp<T>::pack(x2.x * c2.x + x1.x * s2.x, x2.y * c2.y + x1.y * s2.y);
}

// KPW = keys of each 64-key tile one warp handles (16: warps split keys; 64: warps split heads).
// ROPE: the query row is rotated in registers at its position, every K tile in place in shared
// memory at the keys' positions, before the dot.
// System-scope flag accesses of the fused exchange (plain peer stores carry the data; one
// system-scope fence orders them before the flag).
__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Exchange buffer layout (the same as the two-kernel exchange uses): per parity
// o[world][rows][D], then lse[2][world][rows], then flag[2][world].
struct XLayout {
  int64_t o_floats, lse_floats;
  __device__ XLayout(int world, int rows, int D) : o_floats((int64_t)world * rows * D), lse_floats((int64_t)world * rows) {}
  __device__ int64_t o_off(int parity, int src, int rows, int D) const { return parity * o_floats + (int64_t)src * rows * D; }
  __device__ int64_t lse_off(int parity, int src, int rows) const { return 2 * o_floats + parity * lse_floats + (int64_t)src * rows; }
  __device__ int64_t flag_off() const { return 2 * o_floats + 2 * lse_floats; }
};

// Position of local key j on the key axis (contiguous shard, or blocks dealt round-robin).
__device__ __forceinline__ int key_pos(const AfDecodeParams& a, int j) {
  if (a.kv_pos_block <= 0) return a.kv_offset + j;
  const int blk = j / a.kv_pos_block;
  return a.kv_offset + blk * a.kv_pos_stride + (j - blk * a.kv_pos_block);
}
// Number of local keys at positions <= pos (positions grow with the local index in both layouts).
__device__ __forceinline__ int keys_upto(const AfDecodeParams& a, int pos) {
  const int rel = pos - a.kv_offset;
  if (rel < 0) return 0;
  if (a.kv_pos_block <= 0) return rel + 1;
  const int full = rel / a.kv_pos_stride, rem = rel - full * a.kv_pos_stride;
  return full * a.kv_pos_block + min(rem + 1, a.kv_pos_block);
}

// One segment of split-K work: the query heads of chunk `chunk` of KV head (b, h_kv) against the
// keys [lo, hi) of that head, written as un-normalised partials (m, l, acc) to the rows starting
// at `ws_rowc` (the row of the chunk's first head).  Ends with a CTA barrier, so that segments
// can follow one another in one CTA.
template <typename T, int D, int KPW, bool ROPE>
__device__ __forceinline__ void decode_segment(const AfDecodeParams& a, unsigned char* smem_raw, const int b, const int h_kv,
                                               const int chunk, const int lo, const int hi, const int q_pos,
                                               const int64_t ws_rowc) {
  constexpr int ROW_BYTES = D * 2;
  constexpr int CHUNKS = ROW_BYTES / 16;       // 16-byte chunks per row
  constexpr int TILE_BYTES = DEC_BN * ROW_BYTES;
  constexpr int KSTEPS = D / 16;               // k-steps of Q.K^T
  constexpr int NT_S = KPW / 8;                // score n-tiles per warp
  constexpr int NT_O = D / 8;                  // output n-tiles
  constexpr bool SPLIT_KEYS = (KPW == 16);
  unsigned char* sK = smem_raw;
  unsigned char* sV = smem_raw + DEC_STAGES * TILE_BYTES;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int group = a.H_q / a.H_kv;
  // First head (inside the group) of this warp's 16-row M tile.
  const int head0 = chunk * 64 + (SPLIT_KEYS ? 0 : warp * 16);
  const int key_w0 = SPLIT_KEYS ? warp * 16 : 0;   // first key of the tile this warp handles
  const int n_tiles = hi > lo ? (hi - lo + DEC_BN - 1) / DEC_BN : 0;
  const T* kbase = reinterpret_cast<const T*>(a.k) + (int64_t)b * a.k_stride[0] + (int64_t)h_kv * a.k_stride[1];
  const T* vbase = reinterpret_cast<const T*>(a.v) + (int64_t)b * a.v_stride[0] + (int64_t)h_kv * a.v_stride[1];

  auto issue = [&](int tile, int slot) {
    const int key0 = lo + tile * DEC_BN;
    for (int i = tid; i < DEC_BN * CHUNKS; i += DEC_THREADS) {
      const int r = i / CHUNKS, c = i - r * CHUNKS;
      const int key = key0 + r;
      const bool ok = key < hi;
      const int64_t krow = ok ? key : 0;
      const uint32_t off = tile_off<D>(r, c);
      cp_async16(smem_u32(sK + slot * TILE_BYTES + off), kbase + krow * a.k_stride[2] + c * 8, ok ? 16 : 0);
      cp_async16(smem_u32(sV + slot * TILE_BYTES + off), vbase + krow * a.v_stride[2] + c * 8, ok ? 16 : 0);
    }
  };

  // Query fragments: rows g and g+8 of the M tile; rows past the group are zero.
  uint32_t qf[KSTEPS][4];
  {
    const int hl0 = head0 + g, hl1 = head0 + g + 8;
    const bool ok0 = hl0 < group, ok1 = hl1 < group;
    const T* q0 = reinterpret_cast<const T*>(a.q) + (int64_t)b * a.q_stride[0] +
                  (int64_t)(h_kv * group + (ok0 ? hl0 : 0)) * a.q_stride[1];
    const T* q1 = reinterpret_cast<const T*>(a.q) + (int64_t)b * a.q_stride[0] +
                  (int64_t)(h_kv * group + (ok1 ? hl1 : 0)) * a.q_stride[1];
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int d = kk * 16 + 2 * t;
      qf[kk][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
      qf[kk][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
      qf[kk][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
      qf[kk][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
    }
  }

  if (ROPE) {
    // elements d (k-step kk) pair with d + D/2 (k-step kk + KSTEPS/2), same register slot
    const T* cr = reinterpret_cast<const T*>(a.cos) + (int64_t)q_pos * a.rope_stride_n;
    const T* sr = reinterpret_cast<const T*>(a.sin) + (int64_t)q_pos * a.rope_stride_n;
#pragma unroll
    for (int kk = 0; kk < KSTEPS / 2; ++kk) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int d = kk * 16 + 2 * t + (r >> 1) * 8;
        rotate_words<T>(qf[kk][r], qf[kk + KSTEPS / 2][r], *reinterpret_cast<const uint32_t*>(cr + d),
                        *reinterpret_cast<const uint32_t*>(cr + d + D / 2), *reinterpret_cast<const uint32_t*>(sr + d),
                        *reinterpret_cast<const uint32_t*>(sr + d + D / 2));
      }
    }
  }

  const float scale2 = a.sm_scale * kLog2e;
  float slope2[2] = {0.f, 0.f};
  if (a.bias_kind == AF_BIAS_ALIBI) {
    const int hl0 = head0 + g, hl1 = head0 + g + 8;
    if (hl0 < group) slope2[0] = load_slope<T>(a.slopes, h_kv * group + hl0) * kLog2e;
    if (hl1 < group) slope2[1] = load_slope<T>(a.slopes, h_kv * group + hl1) * kLog2e;
  }
  float m2[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

#pragma unroll
  for (int s = 0; s < DEC_STAGES - 1; ++s) {
    if (s < n_tiles) issue(s, s);
    cp_async_commit();
  }

  for (int tile = 0; tile < n_tiles; ++tile) {
    cp_async_wait<DEC_STAGES - 2>();
    __syncthreads();
    {
      const int nxt = tile + DEC_STAGES - 1;
      if (nxt < n_tiles) issue(nxt, nxt % DEC_STAGES);
      cp_async_commit();
    }
    const int slot = tile % DEC_STAGES;
    const uint32_t kt = smem_u32(sK + slot * TILE_BYTES);
    const uint32_t vt = smem_u32(sV + slot * TILE_BYTES);
    if (ROPE && a.rope == 1) {   // rope == 2: the cache already holds rotated keys
      // rotate the K tile in place: a thread takes pairs of 16-byte chunks (c, c + CHUNKS/2) of a row
      const int key0 = lo + tile * DEC_BN;
      for (int i = tid; i < DEC_BN * (CHUNKS / 2); i += DEC_THREADS) {
        const int r = i / (CHUNKS / 2), c = i - r * (CHUNKS / 2);
        if (key0 + r >= hi) continue;
        const int64_t tab = (int64_t)key_pos(a, key0 + r) * a.rope_stride_n + c * 8;
        const uint4 cl = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.cos) + tab));
        const uint4 ch = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.cos) + tab + D / 2));
        const uint4 sl = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.sin) + tab));
        const uint4 sh = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.sin) + tab + D / 2));
        uint4* pl = reinterpret_cast<uint4*>(sK + slot * TILE_BYTES + tile_off<D>(r, c));
        uint4* ph = reinterpret_cast<uint4*>(sK + slot * TILE_BYTES + tile_off<D>(r, c + CHUNKS / 2));
        uint4 xl = *pl, xh = *ph;
        rotate_words<T>(xl.x, xh.x, cl.x, ch.x, sl.x, sh.x);
        rotate_words<T>(xl.y, xh.y, cl.y, ch.y, sl.y, sh.y);
        rotate_words<T>(xl.z, xh.z, cl.z, ch.z, sl.z, sh.z);
        rotate_words<T>(xl.w, xh.w, cl.w, ch.w, sl.w, sh.w);
        *pl = xl; *ph = xh;
      }
      __syncthreads();
    }
    const int key_base = lo + tile * DEC_BN + key_w0;   // first key this warp sees in the tile
    if (SPLIT_KEYS && key_base >= hi) continue;         // warp-uniform: nothing valid here

    // ---- S = Q K^T ------------------------------------------------------------------
    float s[NT_S][4];
#pragma unroll
    for (int j = 0; j < NT_S; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
      for (int jp = 0; jp < NT_S / 2; ++jp) {
        // matrices: (keys 0-7, chunk 2kk) (keys 0-7, chunk 2kk+1) (keys 8-15, 2kk) (keys 8-15, 2kk+1)
        const int r = key_w0 + jp * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int c = 2 * kk + ((lane >> 3) & 1);
        uint32_t bf[4];
        ldmatrix_x4(bf, kt + tile_off<D>(r, c));
        MmaOp<T>::run(s[2 * jp], qf[kk], bf[0], bf[1]);
        MmaOp<T>::run(s[2 * jp + 1], qf[kk], bf[2], bf[3]);
      }
    }

    // ---- online softmax (base 2) ----------------------------------------------------
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NT_S; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key_base + j * 8 + 2 * t + (e & 1);
        const int row = e >> 1;
        float x = s[j][e] * scale2;
        if (a.bias_kind == AF_BIAS_ALIBI) x -= slope2[row] * (float)abs(q_pos - key_pos(a, key));
        x = key < hi ? x : -INFINITY;
        s[j][e] = x;
        mx[row] = fmaxf(mx[row], x);
      }
    }
    float alpha[2];
#pragma unroll
    for (int row = 0; row < 2; ++row) {
      mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 1));
      mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 2));
      const float m_new = fmaxf(m2[row], mx[row]);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[row] = exp2f(m2[row] - m_use);
      m2[row] = m_new;
      mx[row] = m_use;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[NT_S][2];
#pragma unroll
    for (int j = 0; j < NT_S; ++j) {
      const float p0 = exp2f(s[j][0] - mx[0]), p1 = exp2f(s[j][1] - mx[0]);
      const float p2 = exp2f(s[j][2] - mx[1]), p3 = exp2f(s[j][3] - mx[1]);
      rs[0] += p0 + p1;
      rs[1] += p2 + p3;
      pf[j][0] = MmaOp<T>::pack(p0, p1);
      pf[j][1] = MmaOp<T>::pack(p2, p3);
    }
#pragma unroll
    for (int row = 0; row < 2; ++row) {
      rs[row] += __shfl_xor_sync(0xffffffffu, rs[row], 1);
      rs[row] += __shfl_xor_sync(0xffffffffu, rs[row], 2);
      l[row] = l[row] * alpha[row] + rs[row];
    }
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }

    // ---- O += P V -------------------------------------------------------------------
#pragma unroll
    for (int ks = 0; ks < KPW / 16; ++ks) {
      const uint32_t af[4] = {pf[2 * ks][0], pf[2 * ks][1], pf[2 * ks + 1][0], pf[2 * ks + 1][1]};
#pragma unroll
      for (int dp = 0; dp < NT_O / 2; ++dp) {
        // matrices: (keys 0-7, chunk dp*2) (keys 8-15, chunk dp*2) (keys 0-7, dp*2+1) (keys 8-15, dp*2+1)
        const int r = key_w0 + ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int c = 2 * dp + (lane >> 4);
        uint32_t bf[4];
        ldmatrix_x4_trans(bf, vt + tile_off<D>(r, c));
        MmaOp<T>::run(o[2 * dp], af, bf[0], bf[1]);
        MmaOp<T>::run(o[2 * dp + 1], af, bf[2], bf[3]);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  const int64_t ws_row0 = ws_rowc - chunk * 64;   // row of the group's head 0 in the partial arrays
  if (SPLIT_KEYS) {
    // Merge the four warps' partials (each saw a quarter of the keys) through shared memory.
    float* sm_m = reinterpret_cast<float*>(smem_raw);        // [4][16]
    float* sm_l = sm_m + 64;                                 // [4][16]
    float* sm_o = sm_l + 64;                                 // [4][16][D]
    if (t == 0) {
      sm_m[warp * 16 + g] = m2[0]; sm_m[warp * 16 + g + 8] = m2[1];
      sm_l[warp * 16 + g] = l[0];  sm_l[warp * 16 + g + 8] = l[1];
    }
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      float* r0 = sm_o + ((warp * 16 + g) * D) + i * 8 + 2 * t;
      float* r1 = sm_o + ((warp * 16 + g + 8) * D) + i * 8 + 2 * t;
      r0[0] = o[i][0]; r0[1] = o[i][1];
      r1[0] = o[i][2]; r1[1] = o[i][3];
    }
    __syncthreads();
    const int rows = min(group - head0, 16);
    for (int idx = tid; idx < rows * D; idx += DEC_THREADS) {
      const int r = idx / D, d = idx - r * D;
      float mstar = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mstar = fmaxf(mstar, sm_m[w * 16 + r]);
      const float m_use = (mstar == -INFINITY) ? 0.f : mstar;
      float acc = 0.f, lsum = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float sc = exp2f(sm_m[w * 16 + r] - m_use);
        acc += sc * sm_o[(w * 16 + r) * D + d];
        lsum += sc * sm_l[w * 16 + r];
      }
      const int64_t row = ws_row0 + head0 + r;
      a.ws_acc[row * D + d] = acc;
      if (d == 0) {
        a.ws_m[row] = mstar * kLn2;
        a.ws_l[row] = lsum;
      }
    }
  } else {
#pragma unroll
    for (int row = 0; row < 2; ++row) {
      const int hl = head0 + g + 8 * row;
      if (hl >= group) continue;
      const int64_t wr = ws_row0 + hl;
      if (t == 0) {
        a.ws_m[wr] = m2[row] * kLn2;
        a.ws_l[wr] = l[row];
      }
#pragma unroll
      for (int i = 0; i < NT_O; ++i)
        *reinterpret_cast<float2*>(a.ws_acc + wr * D + i * 8 + 2 * t) =
            make_float2(o[i][2 * row], o[i][2 * row + 1]);
    }
  }
  __syncthreads();
}

enum { XMODE_NONE = 0, XMODE_PUSH = 1, XMODE_MERGE = 2, XMODE_STEP = 3 };

// Visible keys of batch entry b, [lo, lo + span), and the position of its query row.  ALiBi
// measures its distance from q_pos (the reference uses the last key,
// attnfuse/compiler/codegen_decode.py:142-145); the causal and window masks of a single row are a
// range of keys.
struct KeyRange { int lo, span, q_pos; };
__device__ __forceinline__ KeyRange key_range(const AfDecodeParams& a, int b) {
  const int len_b = a.kv_lens ? min(max(a.kv_lens[b], 0), a.N_kv) : a.N_kv;
  KeyRange r;
  r.q_pos = a.q_positions ? a.q_positions[b] : (a.q_position_p1 > 0 ? a.q_position_p1 - 1 : key_pos(a, len_b - 1));
  int k_lo = 0, k_hi = len_b;
  if (a.mask_kind == AF_MASK_CAUSAL) k_hi = min(k_hi, keys_upto(a, r.q_pos));
  if (a.mask_kind == AF_MASK_WINDOW) {
    k_lo = keys_upto(a, r.q_pos - a.window);
    k_hi = min(k_hi, keys_upto(a, r.q_pos + a.window - 1));
  }
  r.lo = k_lo;
  r.span = max(k_hi - k_lo, 0);
  return r;
}

// Balanced scheduling (balanced_ctas = C > 0): the 64-key tiles of all (batch, kv head, head
// chunk) units are laid end to end -- unit u = (b * H_kv + h_kv) * head_chunks + chunk, every unit
// at least one tile -- and CTA c takes tiles [c T / C, (c + 1) T / C): equal work per CTA whatever
// the sequence lengths, one wave, no tail.  A CTA's share may end inside a unit and start the
// next, so a unit is covered by a run of consecutive CTAs, and the partial of (unit u, CTA c)
// lives in slot u + c (unique, because both only grow along the run).
__device__ __forceinline__ int unit_tiles(const KeyRange& r) { return max(1, (r.span + DEC_BN - 1) / DEC_BN); }
__device__ __forceinline__ int64_t total_tiles(const AfDecodeParams& a, int units_per_batch) {
  int64_t T = 0;
  for (int b = 0; b < a.B; ++b) T += (int64_t)unit_tiles(key_range(a, b)) * units_per_batch;
  return T;
}
// CTA that holds tile index `tile` (0 <= tile < T): the c with  c T / C <= tile < (c + 1) T / C.
__device__ __forceinline__ int cta_of_tile(int64_t tile, int64_t T, int C) {
  int c = (int)((tile * C) / T);
  while (c + 1 < C && ((int64_t)(c + 1) * T) / C <= tile) ++c;
  while (c > 0 && ((int64_t)c * T) / C > tile) --c;
  return c;
}

// Where the partial rows of one (batch, head) row live.  Classic: split s -> row s * rows + row.
// Balanced: CTA c of the unit's run -> (unit + c) * unit_rows + head within the chunk.
struct PartialRows {
  int first, count;          // classic: splits 0 .. S-1; balanced: CTAs c_first .. c_last
  int64_t base, stride;      // row index of entry i: base + i * stride
};
__device__ __forceinline__ PartialRows partial_rows(const AfDecodeParams& a, int head_chunks, int row, int64_t T,
                                                    int64_t unit_start, int tiles_u, int unit) {
  PartialRows pr;
  const int rows = a.B * a.H_q;
  if (a.balanced_ctas <= 0) {
    pr.first = 0; pr.count = a.num_splits; pr.base = row; pr.stride = rows;
  } else {
    const int group = a.H_q / a.H_kv;
    const int unit_rows = min(group, 64);
    const int head_local = (row % a.H_q) % group % 64;
    const int c0 = cta_of_tile(unit_start, T, a.balanced_ctas), c1 = cta_of_tile(unit_start + tiles_u - 1, T, a.balanced_ctas);
    pr.first = c0; pr.count = c1 - c0 + 1;
    pr.base = (int64_t)(unit + c0) * unit_rows + head_local; pr.stride = unit_rows;
  }
  return pr;
}

// Merge the partials of one row (one warp, D / 32 floats per lane): normalised values, log-sum-exp.
template <int D>
__device__ __forceinline__ void merge_partials(const AfDecodeParams& a, const PartialRows& pr, int lane, float (&acc)[D / 32],
                                               float& lse) {
  constexpr int VEC = D / 32;
  float mstar = -INFINITY;
  for (int i = 0; i < pr.count; ++i) mstar = fmaxf(mstar, a.ws_m[pr.base + i * pr.stride]);
  const float m_use = (mstar == -INFINITY) ? 0.f : mstar;
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
  float lsum = 0.f;
  for (int i = 0; i < pr.count; ++i) {
    const int64_t r = pr.base + i * pr.stride;
    const float w = expf(a.ws_m[r] - m_use);
    lsum += w * a.ws_l[r];
    const float* src = a.ws_acc + r * D + lane * VEC;
    if constexpr (VEC == 4) {
      const float4 v = *reinterpret_cast<const float4*>(src);
      acc[0] += w * v.x; acc[1] += w * v.y; acc[2] += w * v.z; acc[3] += w * v.w;
    } else {
      const float2 v = *reinterpret_cast<const float2*>(src);
      acc[0] += w * v.x; acc[1] += w * v.y;
    }
  }
  const float inv = lsum == 0.f ? 0.f : 1.f / lsum;
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] *= inv;
  lse = lsum == 0.f ? -INFINITY : mstar + logf(lsum);
}

// XMODE (fused KV-sharded step, one launch): XMODE_PUSH -- after its partials are written, a CTA
// takes a ticket of the (batch, kv head[, head chunk]) unit it worked on; the unit's last CTA
// merges the unit's partials and stores the normalised rows and their log-sum-exps into slot
// `rank` of every rank's exchange buffer (plain peer stores), and the CTA that completes the last
// unit raises this rank's flag on every rank.  XMODE_MERGE -- once all of its own work is done,
// such a CTA waits (bounded) for all ranks' flags and merges its units' rows from this rank's own
// buffer into O.  Every CTA of the launch must be resident at once (checked by the host), because
// the waiting CTAs keep their slots.
template <typename T, int D, int KPW, bool ROPE, bool FUSED = false>
__global__ void __launch_bounds__(DEC_THREADS) decode_split_kernel(const AfDecodeParams a, const int head_chunks,
                                                                   const AfPeerExchange x = AfPeerExchange{},
                                                                   const int xmode = XMODE_NONE) {
  constexpr int VEC = D / 32;
  constexpr int MAX_MINE = 64;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int s_last, s_failed, s_mine[FUSED ? MAX_MINE : 1];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = a.H_q / a.H_kv;
  const int units_per_batch = a.H_kv * head_chunks;
  const int n_units = a.B * units_per_batch;
  const int rows = a.B * a.H_q;
  const bool balanced = a.balanced_ctas > 0;
  const bool do_split = !FUSED || (xmode & XMODE_PUSH);
  // fused step: the step number this launch produces (push) or consumes (merge only); read before
  // any CTA can complete the launch's last unit, which is what advances it
  uint32_t xstep = 0;
  if (FUSED) xstep = x.state[0] + ((xmode & XMODE_PUSH) ? 1u : 0u);
  const int parity = xstep & 1;
  int n_mine = 0;                                   // units whose rows this CTA merges at the end
  if (FUSED) {
    if (tid == 0) s_failed = 0;
    __syncthreads();
  }

  // After the partials of `unit` are written: ticket, and for the unit's last CTA the merge of its
  // partials with the push to every rank.  `expected` = CTAs that work on the unit.
  auto after_unit = [&](const int unit, const int expected, const bool designated, const int64_t unit_start,
                        const int tiles_u, const int64_t T_all) {
    bool last = designated;                                            // merge-only launch: no ticket
    if (xmode & XMODE_PUSH) {
      __threadfence();                                                 // this CTA's partials, device-wide
      __syncthreads();
      if (tid == 0) {
        uint32_t* tickets = x.state + 2;
        const uint32_t got = atomicAdd(&tickets[unit], 1u);
        s_last = (got == (uint32_t)expected - 1u);
        if (s_last) tickets[unit] = 0u;                                // ready for the next step
      }
      __syncthreads();
      last = s_last != 0;
      if (last) {
        __threadfence();                                               // the other CTAs' partials
        const int chunk = unit % head_chunks, h_kv = (unit / head_chunks) % a.H_kv, b = unit / units_per_batch;
        const int unit_rows = min(group - chunk * 64, 64);
        const int row0 = b * a.H_q + h_kv * group + chunk * 64;
        const XLayout lay(x.world, rows, D);
        for (int r = warp; r < unit_rows; r += DEC_THREADS / 32) {
          const int row = row0 + r;
          const PartialRows pr = partial_rows(a, head_chunks, row, T_all, unit_start, tiles_u, unit);
          float acc[VEC], lse;
          merge_partials<D>(a, pr, lane, acc, lse);
          for (int peer = 0; peer < x.world; ++peer) {
            float* base = reinterpret_cast<float*>(x.peer_bases[peer]);
            float* dst = base + lay.o_off(parity, x.rank, rows, D) + (int64_t)row * D + lane * VEC;
            if constexpr (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            else *reinterpret_cast<float2*>(dst) = make_float2(acc[0], acc[1]);
            if (lane == 0) base[lay.lse_off(parity, x.rank, rows) + row] = lse;
          }
        }
        __syncthreads();
        if (tid == 0) {
          __threadfence_system();                                      // the unit's peer stores before the count
          const uint32_t done = atomicAdd(&x.state[1], 1u);
          if (done == (uint32_t)n_units - 1u) {
            x.state[1] = 0u;
            __threadfence_system();
            for (int peer = 0; peer < x.world; ++peer) {
              uint32_t* flags = reinterpret_cast<uint32_t*>(reinterpret_cast<float*>(x.peer_bases[peer]) + lay.flag_off());
              st_relaxed_sys_u32(flags + parity * x.world + x.rank, xstep);
            }
            x.state[0] = xstep;
            __threadfence();
          }
        }
      }
    }
    if (last && (xmode & XMODE_MERGE)) {
      if (n_mine < MAX_MINE) {
        if (tid == 0) s_mine[n_mine] = unit;
      } else if (tid == 0) {
        s_failed = 1;                                                  // more units than the list holds
      }
      ++n_mine;
    }
  };

  if (!balanced) {
    const int split = blockIdx.x, unit = blockIdx.y;
    const int chunk = unit % head_chunks, h_kv = (unit / head_chunks) % a.H_kv, b = unit / units_per_batch;
    const KeyRange kr = key_range(a, b);
    int split_len = (kr.span + a.num_splits - 1) / a.num_splits;
    split_len = ((split_len + DEC_BN - 1) / DEC_BN) * DEC_BN;
    const int lo = kr.lo + split * split_len;
    const int hi = min(lo + split_len, kr.lo + kr.span);
    if (do_split)
      decode_segment<T, D, KPW, ROPE>(a, smem_raw, b, h_kv, chunk, lo, hi, kr.q_pos,
                                      ((int64_t)split * a.B + b) * a.H_q + (int64_t)h_kv * group + chunk * 64);
    if (FUSED) after_unit(unit, a.num_splits, split == 0, 0, 0, 0);
  } else {
    const int C = (int)gridDim.x, c = (int)blockIdx.x;
    const int64_t T_all = total_tiles(a, units_per_batch);
    const int64_t t_lo = ((int64_t)c * T_all) / C, t_hi = ((int64_t)(c + 1) * T_all) / C;
    const int unit_rows_max = min(group, 64);
    int64_t base = 0;
    for (int b = 0; b < a.B && base < t_hi; ++b) {
      const KeyRange kr = key_range(a, b);
      const int tiles_u = unit_tiles(kr);
      const int64_t b_end = base + (int64_t)tiles_u * units_per_batch;
      if (b_end > t_lo) {
        const int uu_first = (int)(max(t_lo - base, (int64_t)0) / tiles_u);
        for (int uu = uu_first; uu < units_per_batch; ++uu) {
          const int64_t unit_start = base + (int64_t)uu * tiles_u;
          if (unit_start >= t_hi) break;
          const int s = (int)(max(t_lo, unit_start) - unit_start), e = (int)(min(t_hi, unit_start + tiles_u) - unit_start);
          // More CTAs than tiles: a CTA with an empty share that falls strictly inside a unit still
          // belongs to the unit's run of CTAs (it writes an empty partial and takes its ticket);
          // one that falls on a unit boundary belongs to no run.
          if (e <= s && !(t_lo == t_hi && s > 0)) continue;
          const int unit = b * units_per_batch + uu;
          const int chunk = uu % head_chunks, h_kv = uu / head_chunks;
          const int lo = kr.lo + s * DEC_BN, hi = min(kr.lo + e * DEC_BN, kr.lo + kr.span);
          if (do_split)
            decode_segment<T, D, KPW, ROPE>(a, smem_raw, b, h_kv, chunk, lo, hi, kr.q_pos, (int64_t)(unit + c) * unit_rows_max);
          if (FUSED) {
            const int c0 = cta_of_tile(unit_start, T_all, C), c1 = cta_of_tile(unit_start + tiles_u - 1, T_all, C);
            after_unit(unit, c1 - c0 + 1, c == c1, unit_start, tiles_u, T_all);
          }
        }
      }
      base = b_end;
    }
  }

  if (FUSED && (xmode & XMODE_MERGE) && n_mine > 0) {
    const XLayout lay(x.world, rows, D);
    const float* base = reinterpret_cast<const float*>(x.peer_bases[x.rank]);
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(base + lay.flag_off()) + parity * x.world;
    __syncthreads();
    if (tid < x.world) {
      const long long limit = x.wait_cycles > 0 ? x.wait_cycles : (1ll << 31);
      const long long t0 = clock64();
      // flags only grow; a flag at or past the step (modulo wrap) means that rank's rows landed
      while ((int32_t)(ld_acquire_sys_u32(flags + tid) - xstep) < 0) {
        if (clock64() - t0 > limit) { s_failed = 1; break; }
      }
    }
    __syncthreads();
    if (s_failed) {
      if (tid == 0 && x.status != nullptr) atomicExch(x.status, AF_STATUS_WAIT_TIMEOUT);
    } else {
      for (int m = 0; m < min(n_mine, MAX_MINE); ++m) {
        const int unit = s_mine[m];
        const int chunk = unit % head_chunks, h_kv = (unit / head_chunks) % a.H_kv, b = unit / units_per_batch;
        const int unit_rows = min(group - chunk * 64, 64);
        const int row0 = b * a.H_q + h_kv * group + chunk * 64;
        for (int r = warp; r < unit_rows; r += DEC_THREADS / 32) {
          const int row = row0 + r;
          float w[32];
          float mstar = -INFINITY;
#pragma unroll 8
          for (int rk = 0; rk < x.world; ++rk) {
            w[rk & 31] = base[lay.lse_off(parity, rk, rows) + row];
            mstar = fmaxf(mstar, w[rk & 31]);
          }
          const float m_use = (mstar == -INFINITY) ? 0.f : mstar;
          float wsum = 0.f;
#pragma unroll 8
          for (int rk = 0; rk < x.world; ++rk) {
            w[rk & 31] = (w[rk & 31] == -INFINITY) ? 0.f : expf(w[rk & 31] - m_use);
            wsum += w[rk & 31];
          }
          const float inv = (mstar == -INFINITY) ? 0.f : 1.f / wsum;
          T* dst = reinterpret_cast<T*>(a.o) + (int64_t)(row / a.H_q) * a.o_stride[0] + (int64_t)(row % a.H_q) * a.o_stride[1];
          for (int dd = lane; dd < D; dd += 32) {
            float acc = 0.f;
#pragma unroll 8
            for (int rk = 0; rk < x.world; ++rk)
              if (w[rk & 31] != 0.f) acc += w[rk & 31] * base[lay.o_off(parity, rk, rows, D) + (int64_t)row * D + dd];
            dst[(int64_t)dd * a.o_stride[3]] = Elem<T>::from_f32(acc * inv);
          }
        }
      }
    }
  }
}

// Merge the per-split partials of one (batch, head) row: one warp per row, float4 lanes.
// Reference: attnfuse/compiler/codegen_decode.py:172-211.
template <typename T, int D>
__global__ void decode_combine_kernel(const AfDecodeParams a, const int head_chunks) {
  constexpr int VEC = D / 32;   // floats per lane: 2 (D=64) or 4 (D=128)
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int rows = a.B * a.H_q;
  if (row >= rows) return;
  const int b = row / a.H_q, h = row % a.H_q;
  int64_t T_all = 0, unit_start = 0;
  int tiles_u = 0, unit = 0;
  if (a.balanced_ctas > 0) {
    // the row's unit and its place in the tile sequence (the same walk the split kernel does)
    const int group = a.H_q / a.H_kv, units_per_batch = a.H_kv * head_chunks;
    const int uu = (h / group) * head_chunks + (h % group) / 64;
    unit = b * units_per_batch + uu;
    for (int bb = 0; bb < a.B; ++bb) {
      const int tb = unit_tiles(key_range(a, bb));
      if (bb < b) unit_start += (int64_t)tb * units_per_batch;
      if (bb == b) { tiles_u = tb; unit_start += (int64_t)uu * tb; }
      T_all += (int64_t)tb * units_per_batch;
    }
  }
  const PartialRows pr = partial_rows(a, head_chunks, row, T_all, unit_start, tiles_u, unit);
  float acc[VEC], lse;
  merge_partials<D>(a, pr, lane, acc, lse);
  if (a.o != nullptr) {
    T* dst = reinterpret_cast<T*>(a.o) + (int64_t)b * a.o_stride[0] + (int64_t)h * a.o_stride[1];
#pragma unroll
    for (int i = 0; i < VEC; ++i) dst[(int64_t)(lane * VEC + i) * a.o_stride[3]] = Elem<T>::from_f32(acc[i]);
  }
  if (a.partial != nullptr) {
    float* dst = a.partial + (int64_t)row * (D + 1);
#pragma unroll
    for (int i = 0; i < VEC; ++i) dst[lane * VEC + i] = acc[i];
    if (lane == 0) dst[D] = lse;
  }
}

// Merge G per-rank partials laid out [G][rows][D+1] (normalised O, then LSE).
template <typename T>
__global__ void decode_combine_gathered_kernel(const float* __restrict__ gathered, int G, int rows, int H_q,
                                               int D, T* o, int64_t s0, int64_t s1, int64_t s3) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int64_t stride_g = (int64_t)rows * (D + 1);
  float mstar = -INFINITY;
  for (int r = 0; r < G; ++r) mstar = fmaxf(mstar, gathered[r * stride_g + (int64_t)row * (D + 1) + D]);
  const float m_use = (mstar == -INFINITY) ? 0.f : mstar;
  float wsum = 0.f;
  for (int r = 0; r < G; ++r) wsum += expf(gathered[r * stride_g + (int64_t)row * (D + 1) + D] - m_use);
  const float inv = (mstar == -INFINITY) ? 0.f : 1.f / wsum;
  T* dst = o + (int64_t)(row / H_q) * s0 + (int64_t)(row % H_q) * s1;
  for (int d = lane; d < D; d += 32) {
    float acc = 0.f;
    for (int r = 0; r < G; ++r) {
      const float* src = gathered + r * stride_g + (int64_t)row * (D + 1);
      const float lse = src[D];
      if (lse != -INFINITY) acc += expf(lse - m_use) * src[d];
    }
    dst[(int64_t)d * s3] = Elem<T>::from_f32(acc * inv);
  }
}

template <typename T, int D>
int launch_split_impl(const AfDecodeParams& a, cudaStream_t st) {
  const int group = a.H_q / a.H_kv;
  const int head_chunks = (group + 63) / 64;
  const size_t smem = (size_t)2 * DEC_STAGES * DEC_BN * D * 2;
  const dim3 grid = a.balanced_ctas > 0 ? dim3(a.balanced_ctas, 1) : dim3(a.num_splits, a.B * a.H_kv * head_chunks);
#define AF_DECODE_LAUNCH(KPW, ROPE)                                                                        \
  do {                                                                                                    \
    auto kern = decode_split_kernel<T, D, KPW, ROPE>;                                                     \
    AF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));       \
    kern<<<grid, DEC_THREADS, smem, st>>>(a, head_chunks, AfPeerExchange{}, (int)XMODE_NONE);             \
  } while (0)
  if (group <= 16) {
    if (a.rope) AF_DECODE_LAUNCH(16, true); else AF_DECODE_LAUNCH(16, false);
  } else {
    if (a.rope) AF_DECODE_LAUNCH(64, true); else AF_DECODE_LAUNCH(64, false);
  }
#undef AF_DECODE_LAUNCH
  count_launch();
  return check_cuda(cudaGetLastError(), "decode_split launch");
}

template <typename T, int D>
int launch_combine_impl(const AfDecodeParams& a, cudaStream_t st) {
  const int rows = a.B * a.H_q;
  decode_combine_kernel<T, D><<<(rows + 3) / 4, 128, 0, st>>>(a, (a.H_q / a.H_kv + 63) / 64);
  count_launch();
  return check_cuda(cudaGetLastError(), "decode_combine launch");
}

int validate_decode(const AfDecodeParams& a) {
  AF_REQUIRE(a.dtype == AF_F16 || a.dtype == AF_BF16, "decode kernels take f16/bf16 (got dtype %d)", a.dtype);
  AF_REQUIRE(a.D == 64 || a.D == 128, "decode kernels are instantiated for D in {64,128} (got %d)", a.D);
  AF_REQUIRE(a.B > 0 && a.H_kv > 0 && a.H_q > 0 && a.H_q % a.H_kv == 0, "bad head/batch counts");
  AF_REQUIRE(a.num_splits >= 1 || a.balanced_ctas > 0, "num_splits must be >= 1");
  AF_REQUIRE(a.balanced_ctas >= 0 && a.balanced_ctas <= 65535, "balanced_ctas outside [0, 65535]");
  AF_REQUIRE((int64_t)a.B * a.H_kv * ((a.H_q / a.H_kv + 63) / 64) <= 65535, "B*H_kv too large for one launch");
  AF_REQUIRE(a.ws_m && a.ws_l && a.ws_acc, "decode workspaces must be non-NULL");
  // the combine reads ws_acc rows as float4 (D = 128) / float2 (D = 64); the tensor-core split
  // epilogue stores float4
  AF_REQUIRE(((uintptr_t)a.ws_acc & 15) == 0, "ws_acc must be 16-byte aligned");
  AF_REQUIRE(((uintptr_t)a.ws_m & 3) == 0 && ((uintptr_t)a.ws_l & 3) == 0, "ws_m / ws_l must be 4-byte aligned");
  return AF_OK;
}

}  // namespace

// ---------------------------------------------------------------------------------------
// Decode without any allocation: the split-K partials live in a fixed array in device memory
// that is part of the library image, so a caller that may not (or cannot) call cudaMalloc --
// a serving loop that has handed all device memory to its own pool, code running inside a
// region where the allocator must not be touched, a plugin host that only passes input and
// output buffers -- can still decode.  Every GPU that loads the library holds the array
// (AF_DECODE_STATIC_SCRATCH_BYTES) until the process exits.
// ---------------------------------------------------------------------------------------
constexpr size_t kStaticScratchFloats = AF_DECODE_STATIC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_decode_static_scratch[kStaticScratchFloats];

// Device address of the array on the current device.  In host code the symbol's name is only a
// stand-in, so the address is looked up once per device with cudaGetSymbolAddress (the device
// must be current) and cached.
static int static_scratch_address(float** out) {
  static std::mutex mu;
  static float* cached[64] = {};
  int dev = 0;
  AF_CUDA_OK(cudaGetDevice(&dev));
  AF_REQUIRE(dev >= 0 && dev < 64, "device index %d outside the cache of scratch addresses", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    AF_CUDA_OK(cudaGetSymbolAddress(&ptr, g_decode_static_scratch));
    AF_REQUIRE(ptr != nullptr, "cudaGetSymbolAddress returned a null scratch address");
    cached[dev] = static_cast<float*>(ptr);
  }
  *out = cached[dev];
  return AF_OK;
}

int launch_decode_static(const AfDecodeParams& in, cudaStream_t st) {
  AfDecodeParams a = in;
  a.balanced_ctas = 0;   // the built-in scratch is laid out for the per-unit split grid
  if (a.num_splits <= 0) {
    int dev = 0, sms = 0;
    AF_CUDA_OK(cudaGetDevice(&dev));
    AF_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    a.num_splits = af_decode_num_splits(a.B, a.H_q, a.H_kv, a.N_kv, sms, a.kv_lens != nullptr);
  }
  AF_REQUIRE(a.B > 0 && a.H_q > 0 && a.D > 0, "bad sizes");
  AF_REQUIRE(a.o || a.partial, "combine needs o or partial");
  const size_t rows = (size_t)a.num_splits * a.B * a.H_q;
  // m and l each take rows rounded up to 4 floats, so that acc starts on a 16-byte boundary
  const size_t rows_pad = (rows + 3) & ~(size_t)3;
  const size_t need = 2 * rows_pad + rows * (size_t)a.D;
  if (need > kStaticScratchFloats)
    return fail(AF_ERR_WORKSPACE,
                "af_decode_static: the partials of num_splits*B*H_q rows need %zu floats, which exceeds the built-in scratch of %zu floats "
                "(%d bytes); use af_decode_split/af_decode_combine with caller workspaces",
                need, (size_t)kStaticScratchFloats, (int)AF_DECODE_STATIC_SCRATCH_BYTES);
  float* base = nullptr;
  int rc = static_scratch_address(&base);
  if (rc != AF_OK) return rc;
  // Layout: m[rows_pad], l[rows_pad], acc[rows][D].  The split kernel writes every row of all three
  // (empty splits write m = -inf, l = 0, acc = 0), so nothing left by an earlier call is read
  // and nothing needs clearing.
  a.ws_m = base;
  a.ws_l = base + rows_pad;
  a.ws_acc = base + 2 * rows_pad;
  if ((rc = validate_decode(a)) != AF_OK) return rc;   // nothing is launched on a bad parameter block
  if ((rc = launch_decode_split(a, st)) != AF_OK) return rc;
  return launch_decode_combine(a, st);
}

int launch_decode_split(const AfDecodeParams& a, cudaStream_t st) {
  int rc = validate_decode(a);
  if (rc != AF_OK) return rc;
  AF_REQUIRE(a.q && a.k && a.v, "q/k/v must be non-NULL");
  AF_REQUIRE(a.q_stride[3] == 1 && a.k_stride[3] == 1 && a.v_stride[3] == 1, "decode needs unit inner strides");
  AF_REQUIRE(a.k_stride[2] % 8 == 0 && a.v_stride[2] % 8 == 0 && a.k_stride[1] % 8 == 0 && a.v_stride[1] % 8 == 0 &&
                 a.k_stride[0] % 8 == 0 && a.v_stride[0] % 8 == 0,
             "decode needs 16-byte aligned K/V rows");
  AF_REQUIRE(((uintptr_t)a.k % 16) == 0 && ((uintptr_t)a.v % 16) == 0 && ((uintptr_t)a.q % 4) == 0,
             "decode needs 16-byte aligned K/V base pointers");
  AF_REQUIRE(a.q_stride[1] % 2 == 0 && a.q_stride[0] % 2 == 0, "decode needs 4-byte aligned Q rows");
  AF_REQUIRE(a.bias_kind == AF_BIAS_NONE || (a.bias_kind == AF_BIAS_ALIBI && a.slopes), "bad bias_kind for decode");
  AF_REQUIRE(a.mask_kind == AF_MASK_FULL || a.mask_kind == AF_MASK_CAUSAL || (a.mask_kind == AF_MASK_WINDOW && a.window > 0),
             "decode takes full, causal or window masks (mask_kind %d, window %d)", a.mask_kind, a.window);
  if (a.rope) {
    AF_REQUIRE(a.rope == 1 || a.rope == 2, "decode rope is 0, 1 (rotate query and keys) or 2 (query only), got %d", a.rope);
    AF_REQUIRE(a.cos && a.sin, "RoPE decode needs cos and sin tables");
    AF_REQUIRE(a.rope_stride_n % 8 == 0 && ((uintptr_t)a.cos & 15) == 0 && ((uintptr_t)a.sin & 15) == 0,
               "cos/sin rows must be 16-byte aligned");
  }
  // more than 16 query heads per KV head: tensor-bound on mma.sync, so the tcgen05 kernel takes it
  if (a.balanced_ctas == 0 && decode_tc_supports(a)) return launch_decode_split_tc(a, st);
  if (a.dtype == AF_F16) return a.D == 64 ? launch_split_impl<__half, 64>(a, st) : launch_split_impl<__half, 128>(a, st);
  return a.D == 64 ? launch_split_impl<__nv_bfloat16, 64>(a, st) : launch_split_impl<__nv_bfloat16, 128>(a, st);
}

// The KV-sharded step as ONE launch: split-K over this rank's keys, the per-unit merge with the
// push to every rank's exchange buffer, and (mode bit 2) the bounded wait for the other ranks with
// the final merge.  Mode 1 and mode 2 as separate launches run the two halves on their own, which
// is how several "ranks" are exercised on one GPU (all pushes first, then the merges): kernels
// that wait for one another must never be separate launches on one device.
template <typename T, int D>
int launch_sharded_impl(const AfDecodeParams& a, const AfPeerExchange& x, int mode, cudaStream_t st) {
  const int group = a.H_q / a.H_kv;
  const int head_chunks = (group + 63) / 64;
  const size_t smem = (size_t)2 * DEC_STAGES * DEC_BN * D * 2;
  const dim3 grid = a.balanced_ctas > 0 ? dim3(a.balanced_ctas, 1) : dim3(a.num_splits, a.B * a.H_kv * head_chunks);
#define AF_SHARDED_LAUNCH(KPW, ROPE)                                                                      \
  do {                                                                                                    \
    auto kern = decode_split_kernel<T, D, KPW, ROPE, true>;                                               \
    AF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));       \
    if (mode & XMODE_MERGE) {                                                                             \
      /* waiting CTAs keep their slots: every CTA of the launch has to be resident at once */             \
      int per_sm = 0, sms = 0;                                                                            \
      AF_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, DEC_THREADS, smem));        \
      { const int rc_sm = tc_sm_count(&sms); if (rc_sm != AF_OK) return rc_sm; }                          \
      if ((int64_t)grid.x * grid.y > (int64_t)per_sm * sms)                                               \
        return fail(AF_ERR_INVALID, "fused sharded step: %lld CTAs exceed the %lld that are resident at once; "  \
                    "lower num_splits", (long long)grid.x * grid.y, (long long)per_sm * sms);             \
    }                                                                                                     \
    kern<<<grid, DEC_THREADS, smem, st>>>(a, head_chunks, x, mode);                                       \
  } while (0)
  if (group <= 16) {
    if (a.rope) AF_SHARDED_LAUNCH(16, true); else AF_SHARDED_LAUNCH(16, false);
  } else {
    if (a.rope) AF_SHARDED_LAUNCH(64, true); else AF_SHARDED_LAUNCH(64, false);
  }
#undef AF_SHARDED_LAUNCH
  count_launch();
  return check_cuda(cudaGetLastError(), "decode_sharded_step launch");
}

int launch_decode_sharded_step(const AfDecodeParams& a, const AfPeerExchange* x, int mode, cudaStream_t st) {
  int rc = validate_decode(a);
  if (rc != AF_OK) return rc;
  AF_REQUIRE(x != nullptr && x->world >= 1 && x->world <= 32 && x->rank >= 0 && x->rank < x->world, "bad exchange");
  AF_REQUIRE(x->peer_bases != nullptr && x->state != nullptr, "exchange pointers must be non-NULL");
  AF_REQUIRE(mode >= XMODE_PUSH && mode <= XMODE_STEP, "mode must be 1 (push), 2 (merge) or 3 (whole step)");
  AF_REQUIRE(a.q && a.k && a.v, "q/k/v must be non-NULL");
  AF_REQUIRE(!(mode & XMODE_MERGE) || a.o != nullptr, "the merge writes o");
  AF_REQUIRE(a.q_stride[3] == 1 && a.k_stride[3] == 1 && a.v_stride[3] == 1, "decode needs unit inner strides");
  AF_REQUIRE(a.k_stride[2] % 8 == 0 && a.v_stride[2] % 8 == 0 && a.k_stride[1] % 8 == 0 && a.v_stride[1] % 8 == 0 &&
                 a.k_stride[0] % 8 == 0 && a.v_stride[0] % 8 == 0 && ((uintptr_t)a.k % 16) == 0 && ((uintptr_t)a.v % 16) == 0,
             "decode needs 16-byte aligned K/V rows");
  AF_REQUIRE(((uintptr_t)a.q % 4) == 0 && a.q_stride[1] % 2 == 0 && a.q_stride[0] % 2 == 0, "decode needs 4-byte aligned Q rows");
  AF_REQUIRE(a.bias_kind == AF_BIAS_NONE || (a.bias_kind == AF_BIAS_ALIBI && a.slopes), "bad bias_kind for decode");
  AF_REQUIRE(a.mask_kind == AF_MASK_FULL || a.mask_kind == AF_MASK_CAUSAL || (a.mask_kind == AF_MASK_WINDOW && a.window > 0),
             "decode takes full, causal or window masks");
  if (a.rope) AF_REQUIRE(a.cos && a.sin && a.rope_stride_n % 8 == 0, "RoPE decode needs 16-byte aligned cos / sin tables");
  if (a.dtype == AF_F16) return a.D == 64 ? launch_sharded_impl<__half, 64>(a, *x, mode, st) : launch_sharded_impl<__half, 128>(a, *x, mode, st);
  return a.D == 64 ? launch_sharded_impl<__nv_bfloat16, 64>(a, *x, mode, st) : launch_sharded_impl<__nv_bfloat16, 128>(a, *x, mode, st);
}

int launch_decode_combine(const AfDecodeParams& a, cudaStream_t st) {
  int rc = validate_decode(a);
  if (rc != AF_OK) return rc;
  AF_REQUIRE(a.o || a.partial, "combine needs o or partial");
  if (a.dtype == AF_F16) return a.D == 64 ? launch_combine_impl<__half, 64>(a, st) : launch_combine_impl<__half, 128>(a, st);
  return a.D == 64 ? launch_combine_impl<__nv_bfloat16, 64>(a, st) : launch_combine_impl<__nv_bfloat16, 128>(a, st);
}

int launch_decode_combine_gathered(const float* gathered, int G, int B, int H_q, int D, int dtype, void* o,
                                   const int64_t* os, cudaStream_t st) {
  AF_REQUIRE(gathered && o && os, "NULL argument");
  AF_REQUIRE(G >= 1 && B >= 1 && H_q >= 1 && D >= 1, "bad sizes");
  const int rows = B * H_q;
  const unsigned blocks = (rows + 3) / 4;
  if (dtype == AF_F16)
    decode_combine_gathered_kernel<__half><<<blocks, 128, 0, st>>>(gathered, G, rows, H_q, D, (__half*)o, os[0], os[1], os[3]);
  else if (dtype == AF_BF16)
    decode_combine_gathered_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>(gathered, G, rows, H_q, D, (__nv_bfloat16*)o, os[0], os[1], os[3]);
  else if (dtype == AF_F32)
    decode_combine_gathered_kernel<float><<<blocks, 128, 0, st>>>(gathered, G, rows, H_q, D, (float*)o, os[0], os[1], os[3]);
  else
    return fail(AF_ERR_INVALID, "unknown dtype %d", dtype);
  count_launch();
  return check_cuda(cudaGetLastError(), "decode_combine_gathered launch");
}

}  // namespace af
