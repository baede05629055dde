// Forward attention on the 5th-generation tensor cores (tcgen05 + TMEM) with TMA staging.
//
// Replaces the reference forward kernel (attnfuse/compiler/codegen.py:67-381) and its
// block-sparse sibling (attnfuse/compiler/codegen_blocksparse.py:34-171) for f16/bf16 inputs
// with head_dim 64 or 128 and softmax normalisation.
//
// A work item is 128 query rows of one (batch, query head) against its 128-key tiles.  The kernel
// is persistent: one CTA per SM takes items in a zig-zag over the heaviest-first item list, and
// the barrier phases run on per-CTA running counts, so the loads and the first S product of the
// next item are under way while the previous item's output is still being written.  Roles:
//
//   producer warp   TMA loads: the Q tile once, then K and V tiles into a STAGES-deep ring of
//                   128-byte-swizzled shared-memory tiles (no cluster multicast anywhere).
//   rotation warp   (RoPE only) one warp rotates each K tile in place in shared memory as it
//                   lands -- fp32 math, rounded back to the input dtype exactly as the reference
//                   does before its dot (codegen.py:332-341) -- then hand it to the MMA warp.
//                   The Q tile is rotated once by the softmax group (codegen.py:126-135).
//   MMA warps       one thread issues  S = Q K^T  (tcgen05.mma, operands from shared memory,
//                   fp32 accumulator in TMEM, two S buffers), a thread of another warp issues
//                   O += P V  (P read from TMEM, V from shared memory, N-major); both commit to
//                   mbarriers.
//   softmax group   256 threads, two per query row (TMEM lane = row, so row max / row sum need
//                   no shuffles); each thread owns 64 of a tile's 128 key columns and runs an
//                   online softmax of its own over them -- own reference maximum, own row sum,
//                   own accumulator O_h in TMEM -- so the two warps that share a scheduler never
//                   synchronise inside the tile loop.  Per tile: tcgen05.ld the S columns, apply
//                   scale, ALiBi, causal / window / length masks, exponentials in base 2, write
//                   P as f16/bf16 over the thread's own S columns with tcgen05.st.  O_h is
//                   rescaled only when the maximum grew by more than 2^6 since the value the
//                   accumulator is expressed in (the result is mathematically unchanged: P, l and
//                   O share that reference), and in the steady state no separate pass for the tile
//                   maximum runs at all.  The two halves of a row are merged once per item.
//
// Every mbarrier wait is bounded; on a timeout the CTA raises a status word, drains and
// frees its TMEM.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace af {
namespace tc {

using namespace ptx;

enum { ROPE_NONE = 0, ROPE_FUSED = 1 };   // a pre-pass rotation runs the ROPE_NONE kernels
enum { EMASK_NONE = 0, EMASK_CAUSAL = 1, EMASK_WINDOW = 2, EMASK_BITS = 3 };  // element-level mask of the instantiation
// (EMASK_BITS: block lists in which some tiles carry a bit matrix of their active elements)

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int PANEL_BYTES = 128 * 128;   // 128 rows x 64 elements x 2 bytes
// The reference maximum of a softmax stream moves only when a tile maximum exceeds it by more than
// kRescaleThreshold (log2 units).  A tile processed without looking at its maximum first is accepted
// when the sum over the thread's 64 columns stays below kRowSumBound: every term is then below the
// bound too, far inside the f16 range, and a rejected tile has a term above kRowSumBound / 64 = 2^7 >
// 2^kRescaleThreshold, so the classic pass that follows is certain to move the reference and the
// next tile is accepted again.
constexpr float kRescaleThreshold = 6.f;
constexpr float kRowSumBound = 8192.f;

template <int D> struct Cfg {
  static constexpr int PANELS = D / 64;
  static constexpr int TILE_BYTES = PANELS * PANEL_BYTES;     // one Q, K or V tile
  // K tiles are consumed early (S runs up to two tiles ahead of the softmax group), V tiles late
  // (after the tile's softmax), so a V slot freed by P.V of tile j is not needed before tile j+2
  // has gone through the softmax group: two V stages suffice at head dim 128, and the tile they
  // leave free stages the output rows for a TMA store.
  static constexpr int STAGES = (D == 128) ? 3 : 4;            // K ring
  static constexpr int STAGES_V = (D == 128) ? 2 : 4;          // V ring
  // 8 regions [half][row quadrant] of 32 rows; a row of a region holds D/2 elements and sits on
  // the 128-byte pitch of the swizzle whether it fills it (D = 128) or not (D = 64)
  static constexpr int O_STAGE_BYTES = 8 * 32 * 128;
  static constexpr int SMEM_BYTES = TILE_BYTES * (1 + STAGES + STAGES_V) + O_STAGE_BYTES + 1024 /*align*/ +
                                    1536 /*barriers, exchange*/;
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_S0 = 0, COL_S1 = 128, COL_O0 = 256, COL_O1 = 256 + D;   // one O per half of the key columns
};

// Warp roles.  The softmax group has two threads per query row: warps 0-3 take key columns
// 0..63 of a tile, warps 4-7 columns 64..127 (warp w and w+4 own the same 32 TMEM lanes).
constexpr int SOFTMAX_THREADS = 256;
constexpr int HALF_COLS = BN / 2;
enum { WARP_PRODUCER = 8, WARP_QK = 9, WARP_PV = 10, WARP_ROTATE = 11 };

struct Barriers {
  uint64_t q_full, q_ready, q_empty;
  uint64_t k_full[4], k_ready[4], k_empty[4];
  uint64_t v_full[4], v_empty[4];
  uint64_t s_full[2][2], p_full[2][2], pv_done[2][2];   // [S buffer][half of the key columns]; head dim 128 uses [.][0] of s_full / pv_done
  uint64_t o_free;
  uint32_t tmem_base;
  int abort_flag;
  uint32_t pair_flag[2][8];   // hand-shake counts of the softmax warps, two slots by parity of the count
  float xchg[SOFTMAX_THREADS];   // reference maximum / row sum exchange between the two halves of a row
};

// Division of a non-negative int by a divisor fixed per launch (round-up multiplier method): the
// item decode runs once per item in every role and a hardware-emulated division costs about as
// much as a tenth of a key tile.
struct FastDiv {
  uint32_t mul, shr;   // shr == 0: divisor 1
  __host__ static FastDiv make(uint32_t d) {
    FastDiv f{0u, 0u};
    if (d <= 1) return f;
    uint32_t l = 0;
    while ((1ull << l) < d) ++l;
    f.mul = (uint32_t)(((1ull << 32) * ((1ull << l) - d)) / d + 1);
    f.shr = l;
    return f;
  }
  __device__ __forceinline__ int div(int n) const {
    if (shr == 0) return n;
    const uint32_t q = __umulhi((uint32_t)n, mul);
    return (int)(((((uint32_t)n - q) >> 1) + q) >> (shr - 1));
  }
};

static_assert(sizeof(Barriers) <= 1536, "Cfg::SMEM_BYTES reserves 1536 bytes for the barriers and the exchange");

struct TcArgs {
  AfFwdParams a;
  int num_m_blocks;
  int kv_tiles_per_block;   // block_n / 128 for block lists
  int q_tiles_per_block;    // block_m / 128
  int total_items;          // num_m_blocks * B * H_q query tiles (split mode: num_splits * B * H)
  int grid_ctas;            // CTAs to launch: one per SM (persistent) or one per item
  FastDiv div_hq, div_group;           // by H_q, by H_q / H_kv
  // Item order.  The units -- (batch, head) pairs, heads of a KV group adjacent -- are taken in
  // chunks whose K and V fit the L2 together; inside a chunk the items run row of query tiles by
  // row (all units of the chunk, then the next row), so a key tile fetched from DRAM is still in
  // the L2 when the chunk's other query tiles ask for it.  One chunk = all units is the plain
  // row-major order.  Odd chunks run their rows in reverse, so that the item weights of a causal
  // problem fall and rise continuously across chunk boundaries (the zig-zag deal evens out
  // monotonic stretches, not steps).
  int unit_chunk, items_per_chunk;     // units per chunk (divides the unit count); rows * unit_chunk
  FastDiv div_ipc, div_chunk;          // by items_per_chunk, by unit_chunk
  // Split-K decode mode (num_splits > 0): the "query rows" of an item are the query heads of one
  // KV group (N_q = group size, one pseudo-head per KV head), the keys of a sequence are dealt out
  // to num_splits items, and the epilogue writes un-normalised partials (m, l, acc) for the
  // combine kernel instead of O.  Row index of the partials: (split * B + b) * H_total + head.
  int num_splits;
  const int32_t* kv_lens;   // optional per-batch valid key count
  float* ws_m;
  float* ws_l;
  float* ws_acc;
};

// Which key tiles a query tile visits.
struct TileWalk {
  int n_tiles;
  int first_tile;            // dense / causal / window: lowest tile index
  int step;                  // +1, or -1 when the tiles are walked from the diagonal down
  const int32_t* list;       // block lists: active key blocks of this query block
  const int32_t* slots;      // block lists: bit-matrix number of each listed block (-1: fully active), or null
  int per_block;
  __device__ __forceinline__ int key0(int j) const {
    if (list != nullptr) return (list[j / per_block] * per_block + (j % per_block)) * BN;
    return (first_tile + (step > 0 ? j : n_tiles - 1 - j)) * BN;
  }
};

__device__ __forceinline__ TileWalk make_walk(const AfProblem& p, const TcArgs& args, int m_blk, int h) {
  TileWalk w;
  w.list = nullptr;
  w.slots = nullptr;
  w.per_block = 1;
  w.first_tile = 0;
  // Causal + ALiBi: the bias grows towards the diagonal by slope * 128 per tile, so walking up
  // would raise the row maximum (and rescale the accumulator) at every tile; walking down from
  // the diagonal sets the reference in the first tile and every later tile stays below it.
  w.step = (p.mask_kind == AF_MASK_CAUSAL && p.bias_kind == AF_BIAS_ALIBI) ? -1 : 1;
  const int m0 = m_blk * BM + p.q_offset;                 // first / one-past-last position of the tile
  const int m_end = min(m_blk * BM + BM, p.N_q) + p.q_offset;
  if (p.mask_kind == AF_MASK_BLOCKS) {
    const int qb = m_blk / args.q_tiles_per_block;
    w.per_block = args.kv_tiles_per_block;
    w.list = p.kv_idx + (int64_t)h * p.kv_idx_stride_h + (int64_t)qb * p.kv_idx_stride_q;
    if (p.kv_slot != nullptr) w.slots = p.kv_slot + (int64_t)h * p.kv_idx_stride_h + (int64_t)qb * p.kv_idx_stride_q;
    w.n_tiles = p.kv_num[(int64_t)h * p.kv_num_stride_h + qb] * w.per_block;
  } else if (p.mask_kind == AF_MASK_CAUSAL) {
    w.n_tiles = (min(m_end, p.N_kv) + BN - 1) / BN;
  } else if (p.mask_kind == AF_MASK_WINDOW) {
    const int lo = max(0, m0 - p.window + 1);
    const int hi = min(p.N_kv, m_end + p.window - 1);
    w.first_tile = lo / BN;
    w.n_tiles = hi > lo ? (hi + BN - 1) / BN - w.first_tile : 0;
  } else {
    w.n_tiles = (p.N_kv + BN - 1) / BN;
  }
  if (w.n_tiles < 0) w.n_tiles = 0;
  return w;
}

// Item number -> (row index in visiting order, unit); see TcArgs::unit_chunk.
__device__ __forceinline__ void split_item(const TcArgs& args, int w, int n_rows, int& row_idx, int& unit) {
  const int c = args.div_ipc.div(w);
  const int r = w - c * args.items_per_chunk;
  row_idx = args.div_chunk.div(r);
  unit = c * args.unit_chunk + (r - row_idx * args.unit_chunk);
  if (c & 1) row_idx = n_rows - 1 - row_idx;
}

// One work item = one 128-row query tile of one (batch, query head).
struct Item {
  int m0, b, h, h_kv;
  int split, n_kv;           // split mode: which share of the keys; valid keys of the batch entry
  TileWalk walk;
};

// Items are numbered heaviest first (causal: the last query tiles).  A CTA takes item
// r*G + c in even rounds r and r*G + (G-1-c) in odd rounds (c = blockIdx.x, G = gridDim.x): with
// item weights that fall monotonically the zig-zag evens out the key tiles per CTA to within a
// fraction of a percent.  With G = number of items every CTA runs exactly one item.
template <int EMASK, bool SPLIT>
__device__ __forceinline__ bool get_item(const TcArgs& args, int round, Item& it) {
  const int G = (int)gridDim.x, c = (int)blockIdx.x;
  const int64_t w64 = (int64_t)round * G + ((round & 1) ? G - 1 - c : c);
  if (w64 >= args.total_items) return false;
  const int w = (int)w64;
  const AfProblem& p = args.a.p;
  int w_over_bh, bh;   // row of query tiles in visiting order (split mode: the split), (batch, head) unit
  split_item(args, w, SPLIT ? args.num_splits : args.num_m_blocks, w_over_bh, bh);
  it.b = args.div_hq.div(bh);
  it.h = bh - it.b * p.H_q;
  it.h_kv = args.div_group.div(it.h);
  it.split = 0;
  it.n_kv = p.N_kv;
  if (SPLIT) {
    // split-K decode: one query tile per (batch, pseudo-head); the 128-key tiles of the valid
    // length are dealt out evenly to the splits
    it.split = w_over_bh;
    it.m0 = 0;
    TileWalk& wk = it.walk;
    wk.list = nullptr; wk.slots = nullptr; wk.per_block = 1; wk.step = 1;
    it.n_kv = args.kv_lens ? min(max(args.kv_lens[it.b], 0), p.N_kv) : p.N_kv;
    const int tiles = (it.n_kv + BN - 1) / BN;
    wk.first_tile = (int)((int64_t)it.split * tiles / args.num_splits);
    wk.n_tiles = (int)((int64_t)(it.split + 1) * tiles / args.num_splits) - wk.first_tile;
    return true;
  }
  const int m_blk = (EMASK == EMASK_CAUSAL) ? (args.num_m_blocks - 1 - w_over_bh) : w_over_bh;
  it.m0 = m_blk * BM;
  it.walk = make_walk(p, args, m_blk, it.h);
  return true;
}

// Position of a role in the CTA's sequence of key tiles (items without key tiles are skipped):
// gg = running tile count, qi = running count of items with tiles, j = tile within the item.
struct TileCursor {
  Item it;
  int round, j, gg, qi;
};
__device__ __forceinline__ void cursor_init(TileCursor& c) {
  c.round = -1; c.j = 0; c.gg = -1; c.qi = -1;
  c.it.walk.n_tiles = 0;
}
template <int EMASK, bool SPLIT>
__device__ __forceinline__ bool cursor_next(const TcArgs& args, TileCursor& c) {
  if (c.j + 1 < c.it.walk.n_tiles) { ++c.j; ++c.gg; return true; }
  for (;;) {
    ++c.round;
    if (!get_item<EMASK, SPLIT>(args, c.round, c.it)) return false;
    if (c.it.walk.n_tiles > 0) { c.j = 0; ++c.gg; ++c.qi; return true; }
  }
}

template <typename T> struct Pack2;
template <> struct Pack2<__half> {
  __device__ __forceinline__ static uint32_t run(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ __forceinline__ static float2 unpack(uint32_t x) {
    return __half22float2(*reinterpret_cast<__half2*>(&x));
  }
};
template <> struct Pack2<__nv_bfloat16> {
  __device__ __forceinline__ static uint32_t run(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ __forceinline__ static float2 unpack(uint32_t x) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&x));
  }
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Rotate-half on row `r` of a 128-row tile stored as 64-element panels with the 128-byte TMA
// swizzle (16-byte chunk c of row r lives at chunk c ^ (r & 7)).  Element d pairs with
// d + D/2: the same chunk of the second panel for D = 128, chunk c + 4 of the same panel for
// D = 64.  fp32 math, one rounding to T.
template <typename T, int D>
__device__ __forceinline__ void rope_row(uint32_t tile, int r, const T* cos_row, const T* sin_row) {
  constexpr int HC = D / 16;  // 16-byte chunks per half row
  const uint32_t row_base = tile + r * 128;
#pragma unroll
  for (int c = 0; c < HC; ++c) {
    const uint32_t a_lo = row_base + ((c ^ (r & 7)) << 4);
    const uint32_t a_hi = (D == 128) ? a_lo + PANEL_BYTES : row_base + (((c + HC) ^ (r & 7)) << 4);
    const uint4 xl = lds128(a_lo), xh = lds128(a_hi);
    const uint4 cl = __ldg(reinterpret_cast<const uint4*>(cos_row + c * 8));
    const uint4 ch = __ldg(reinterpret_cast<const uint4*>(cos_row + D / 2 + c * 8));
    const uint4 sl = __ldg(reinterpret_cast<const uint4*>(sin_row + c * 8));
    const uint4 sh = __ldg(reinterpret_cast<const uint4*>(sin_row + D / 2 + c * 8));
    const uint32_t xlw[4] = {xl.x, xl.y, xl.z, xl.w}, xhw[4] = {xh.x, xh.y, xh.z, xh.w};
    const uint32_t clw[4] = {cl.x, cl.y, cl.z, cl.w}, chw[4] = {ch.x, ch.y, ch.z, ch.w};
    const uint32_t slw[4] = {sl.x, sl.y, sl.z, sl.w}, shw[4] = {sh.x, sh.y, sh.z, sh.w};
    uint32_t ol[4], oh[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x1 = Pack2<T>::unpack(xlw[i]), x2 = Pack2<T>::unpack(xhw[i]);
      const float2 c1 = Pack2<T>::unpack(clw[i]), c2 = Pack2<T>::unpack(chw[i]);
      const float2 s1 = Pack2<T>::unpack(slw[i]), s2 = Pack2<T>::unpack(shw[i]);
      ol[i] = Pack2<T>::run(x1.x * c1.x - x2.x * s1.x, x1.y * c1.y - x2.y * s1.y);
      oh[i] = Pack2<T>::run(x2.x * c2.x + x1.x * s2.x, x2.y * c2.y + x1.y * s2.y);
    }
    sts128(a_lo, make_uint4(ol[0], ol[1], ol[2], ol[3]));
    sts128(a_hi, make_uint4(oh[0], oh[1], oh[2], oh[3]));
  }
}


__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Hand-shake between the two warps that share 32 query rows (warp w and w ^ 4).  Each warp
// publishes its hand-shake count with a release store and polls the partner's word with acquire
// loads; whatever both wrote to shared memory before is visible afterwards.  The words alternate
// between two slots by the parity of the count, so a warp that runs ahead to its next hand-shake
// cannot overwrite a word its partner has not read yet.  The wait is bounded like the mbarrier
// waits (a hardware named barrier would hang if the partner left after a time-out).  It orders
// shared-memory traffic only: the two warps never touch each other's TMEM columns.
__device__ __forceinline__ bool pair_sync(Barriers* bars, int warp, int lane, uint32_t& count,
                                          volatile int* abort_flag) {
  ++count;
  __syncwarp();
  uint32_t* mine = &bars->pair_flag[count & 1][warp];
  const uint32_t* theirs = &bars->pair_flag[count & 1][warp ^ 4];
  if (lane == 0)
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(mine)), "r"(count) : "memory");
  const long long t0 = clock64();
  uint32_t v, spins = 0;
  for (;;) {
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(theirs)) : "memory");
    if (v == count) break;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  __syncwarp();
  return true;
}

// Maximum of NC fp32 bit patterns, four independent chains.
template <int NC>
__device__ __forceinline__ float row_max(const uint32_t (&xr)[NC]) {
  float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int c = 0; c < NC; c += 4) {
#pragma unroll
    for (int u = 0; u < 4; ++u) mx4[u] = fmaxf(mx4[u], __uint_as_float(xr[c + u]));
  }
  return fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
}

// P = 2^y packed to T and the row sum of the unrounded values, with
//   EXP_SCALE      y = x * scale2 + shift
//   EXP_AFFINE     y = x * scale2 + slope_c * c + shift     (ALiBi folded in, c = column index)
//   EXP_PRESCALED  y = x + shift                            (scores already scaled and biased)
enum { EXP_SCALE = 0, EXP_AFFINE = 1, EXP_PRESCALED = 2 };
// Packed fp32 pairs (sm_100: fma / add on two fp32 values in one 64-bit register pair, one issue
// slot): the scale-and-shift and the row sum of the exponent pass take half the instructions.
__device__ __forceinline__ uint64_t f32x2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f32x2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f32x2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f32x2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

template <typename T, int KIND, int NC>
__device__ __forceinline__ void exp_pass(const uint32_t (&xr)[NC], uint32_t (&pk)[NC / 2], float scale2, float shift,
                                         float slope_c, float& rsum) {
  if (KIND == EXP_AFFINE) {
    float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < NC; c += 4) {
      float e[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float x = __uint_as_float(xr[c + u]);
        e[u] = ex2_approx(fmaf(x, scale2, fmaf(slope_c, (float)(c + u), shift)));
        rs4[u] += e[u];
      }
      pk[c >> 1] = Pack2<T>::run(e[0], e[1]);
      pk[(c >> 1) + 1] = Pack2<T>::run(e[2], e[3]);
    }
    rsum = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
    return;
  }
  const uint64_t sc2 = f32x2_pack(scale2, scale2), sh2 = f32x2_pack(shift, shift);
  uint64_t rs2[2] = {f32x2_pack(0.f, 0.f), f32x2_pack(0.f, 0.f)};
#pragma unroll
  for (int c = 0; c < NC; c += 4) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint64_t x2 = f32x2_pack(__uint_as_float(xr[c + 2 * u]), __uint_as_float(xr[c + 2 * u + 1]));
      const uint64_t y2 = (KIND == EXP_PRESCALED) ? f32x2_add(x2, sh2) : f32x2_fma(x2, sc2, sh2);
      float y0, y1;
      f32x2_unpack(y2, y0, y1);
      const float e0 = ex2_approx(y0), e1 = ex2_approx(y1);
      rs2[u] = f32x2_add(rs2[u], f32x2_pack(e0, e1));
      pk[(c >> 1) + u] = Pack2<T>::run(e0, e1);
    }
  }
  float a0, a1, b0, b1;
  f32x2_unpack(rs2[0], a0, a1);
  f32x2_unpack(rs2[1], b0, b1);
  rsum = (a0 + a1) + (b0 + b1);
}

// One instantiation per composition: element type, head_dim, RoPE mode, element-level mask and
// ALiBi are compile-time, so the per-element code of the softmax group carries no run-time
// branches on the composition.
template <typename T, int D, int ROPE, int EMASK, bool ALIBI, bool SPLIT>
__global__ void __launch_bounds__(ROPE == ROPE_FUSED ? 384 : 352, 1)
fwd_tcgen05_kernel(const TcArgs args, const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                   const __grid_constant__ CUtensorMap tmap_o) {
  using C = Cfg<D>;
  constexpr int STAGES = C::STAGES, STAGES_V = C::STAGES_V;
  constexpr bool ROT_K = (ROPE == ROPE_FUSED);
  constexpr int AB_FMT = (Elem<T>::code == AF_BF16) ? 1 : 0;
  // Head dim 64: one S product per half of the key columns, each with barriers of its own, so the
  // two softmax streams of a row never wait for each other (the operands are small enough that
  // reading Q twice per tile does not load the shared-memory port; at head dim 128 it does, and
  // the whole-tile product is faster there).
  constexpr bool SPLIT_S = (D == 64);
  constexpr int S_PARTS = SPLIT_S ? 2 : 1;
  constexpr uint32_t IDESC_QK = umma_idesc_f16(AB_FMT, BM, SPLIT_S ? HALF_COLS : BN, 0, 0);
  constexpr uint32_t IDESC_PV = umma_idesc_f16(AB_FMT, BM, D, 0, 1);

  const AfFwdParams& a = args.a;
  const AfProblem& p = a.p;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base;
  const uint32_t sK0 = sQ + C::TILE_BYTES;
  const uint32_t sV0 = sK0 + STAGES * C::TILE_BYTES;
  const uint32_t sO = sV0 + STAGES_V * C::TILE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(smem + C::TILE_BYTES * (1 + STAGES + STAGES_V) + C::O_STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // Every role walks the same item sequence (get_item) and keeps two running counts: `g`, key
  // tiles processed so far by this CTA (ring stage g % STAGES, S buffer g & 1, barrier phases
  // derived from g), and `qi`, items with at least one key tile (phases of the Q / O hand-overs).
  // The pipeline therefore runs across item boundaries: the first S product of the next item is
  // issued while the softmax group still writes the previous item's output.
  if (tid == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_ready, 128);
    mbar_init(&bars->q_empty, 1);
    mbar_init(&bars->o_free, SOFTMAX_THREADS);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_ready[s], 32);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      for (int hh = 0; hh < 2; ++hh) {
        mbar_init(&bars->s_full[t][hh], 1);
        mbar_init(&bars->p_full[t][hh], SOFTMAX_THREADS / 2);
        mbar_init(&bars->pv_done[t][hh], 1);
      }
    }
    bars->abort_flag = 0;
    for (int i = 0; i < 16; ++i) (&bars->pair_flag[0][0])[i] = 0u;
    mbar_fence_init();
  }
  if (warp == WARP_PRODUCER) {
    tmem_alloc(&bars->tmem_base, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;

  if (warp == WARP_PRODUCER) {
    // ============================== TMA producer ==============================
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      tma_prefetch_desc(&tmap_o);
      // Two cursors over the same tile sequence: K runs one tile ahead of V, so that a wait for
      // a V slot (free only after the P.V product two tiles back) never holds up a K load.
      // split-K decode reads every cache tile exactly once: nothing to keep there
      const uint64_t stream = l2_policy_evict_first(), keep = SPLIT ? stream : l2_policy_evict_last();
      TileCursor ck, cv;
      cursor_init(ck);
      cursor_init(cv);
      auto load_k = [&]() -> bool {
        if (ck.j == 0) {
          // the single Q buffer is free once the last S product of the previous item has run
          if (ck.qi > 0 && !mbar_wait(&bars->q_empty, (ck.qi - 1) & 1, abort_flag)) return false;
          mbar_arrive_expect_tx(&bars->q_full, C::TILE_BYTES);
#pragma unroll
          for (int pn = 0; pn < C::PANELS; ++pn)
            tma_load_4d_hint(smem + pn * PANEL_BYTES, &tmap_q, &bars->q_full, pn * 64, ck.it.m0, ck.it.h, ck.it.b, stream);
        }
        const int s = ck.gg % STAGES;
        const uint32_t par = ((ck.gg / STAGES) & 1) ^ 1;   // parity of the previous use of the slot
        unsigned char* dk = smem + C::TILE_BYTES * (1 + s);
        if (ck.gg >= STAGES && !mbar_wait(&bars->k_empty[s], par, abort_flag)) return false;
        mbar_arrive_expect_tx(&bars->k_full[s], C::TILE_BYTES);
        const int key0 = ck.it.walk.key0(ck.j);
#pragma unroll
        for (int pn = 0; pn < C::PANELS; ++pn)
          tma_load_4d_hint(dk + pn * PANEL_BYTES, &tmap_k, &bars->k_full[s], pn * 64, key0, ck.it.h_kv, ck.it.b, keep);
        return true;
      };
      auto load_v = [&]() -> bool {
        const int s = cv.gg % STAGES_V;
        const uint32_t par = ((cv.gg / STAGES_V) & 1) ^ 1;
        unsigned char* dv = smem + C::TILE_BYTES * (1 + STAGES + s);
        if (cv.gg >= STAGES_V && !mbar_wait(&bars->v_empty[s], par, abort_flag)) return false;
        mbar_arrive_expect_tx(&bars->v_full[s], C::TILE_BYTES);
        const int key0 = cv.it.walk.key0(cv.j);
#pragma unroll
        for (int pn = 0; pn < C::PANELS; ++pn)
          tma_load_4d_hint(dv + pn * PANEL_BYTES, &tmap_v, &bars->v_full[s], pn * 64, key0, cv.it.h_kv, cv.it.b, keep);
        return true;
      };
      bool more_k = cursor_next<EMASK, SPLIT>(args, ck);
      bool more_v = cursor_next<EMASK, SPLIT>(args, cv);
      // K runs one tile ahead of V (a wait for a V slot never holds up a K load) -- except across
      // an item boundary: the first K load of an item starts with a wait for the Q buffers (the
      // previous item's last S product), so every V tile of the previous item goes out before it.
      while (more_k || more_v) {
        const bool at_boundary = more_k && ck.j == 0 && ck.qi > 0 && more_v && cv.gg < ck.gg;
        if (more_k && !at_boundary && (!more_v || ck.gg <= cv.gg + 1)) {
          if (!load_k()) break;
          more_k = cursor_next<EMASK, SPLIT>(args, ck);
        } else {
          if (!load_v()) break;
          more_v = cursor_next<EMASK, SPLIT>(args, cv);
        }
      }
    }
  } else if (warp == WARP_QK) {
    // ============================== MMA issuer 1: S = Q K^T ==============================
    // The two products are issued by two threads.  A tcgen05.mma issue blocks while the pipe's
    // short queue is full, so a single issuing thread leaves the pipe idle during its own barrier
    // waits and commits (measured: about 800 of 2000 cycles per key tile).
    if (lane == 0) {
      const uint64_t desc_q0 = umma_desc_sw128(sQ, 16, 1024);
      const uint64_t desc_k0 = umma_desc_sw128(sK0, 16, 1024);
      Item it;
      int g = 0, qi = 0;
      bool ok = true;
      for (int round = 0; ok && get_item<EMASK, SPLIT>(args, round, it); ++round) {
        const int n_tiles = it.walk.n_tiles;
        if (n_tiles == 0) continue;
        ok = mbar_wait(ROPE != ROPE_NONE ? &bars->q_ready : &bars->q_full, qi & 1, abort_flag);
        for (int j = 0; ok && j < n_tiles; ++j) {
          const int gg = g + j;                       // the CTA's running key-tile count
          const int s = gg % STAGES, t = gg & 1;
          if (!mbar_wait(ROT_K ? &bars->k_ready[s] : &bars->k_full[s], (gg / STAGES) & 1, abort_flag)) { ok = false; break; }
          // Descriptors are built once; a k-step, a ring stage or a half only moves the
          // start-address field (address >> 4), so the issuing thread spends one add per operand.
          const uint64_t kdesc = desc_k0 + (uint64_t)((s * C::TILE_BYTES) >> 4);
          for (int hh = 0; hh < S_PARTS && ok; ++hh) {
            // S buffer t (the half's columns of it) still holds P of tile gg-2 until its P.V product has run
            if (gg >= 2 && !mbar_wait(&bars->pv_done[t][hh], ((gg >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem + (t ? C::COL_S1 : C::COL_S0) + hh * HALF_COLS;
            const uint64_t kh = kdesc + (uint64_t)((hh * HALF_COLS * 128) >> 4);   // keys 64 hh .. : rows of the K tile
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint64_t off = (uint64_t)(((kk >> 2) * PANEL_BYTES + (kk & 3) * 32) >> 4);
              umma_ss(d_tmem, desc_q0 + off, kh + off, IDESC_QK, kk > 0 ? 1u : 0u);
            }
            umma_commit(&bars->s_full[t][hh]);
          }
          if (!ok) break;
          umma_commit(&bars->k_empty[s]);
          // the item's last S product: the Q buffer may be refilled when it has run
          if (j + 1 == n_tiles) umma_commit(&bars->q_empty);
        }
        g += n_tiles;
        ++qi;
      }
    }
  } else if (warp == WARP_PV) {
    // ============================== MMA issuer 2: O += P V ==============================
    if (lane == 0) {
      const uint64_t desc_v0 = umma_desc_sw128(sV0, PANEL_BYTES, 1024);
      Item it;
      int g = 0, qi = 0;
      bool ok = true;
      for (int round = 0; ok && get_item<EMASK, SPLIT>(args, round, it); ++round) {
        const int n_tiles = it.walk.n_tiles;
        if (n_tiles == 0) continue;
        for (int j = 0; j < n_tiles; ++j) {
          const int gg = g + j;
          const int s = gg % STAGES_V, t = gg & 1;
          if (!mbar_wait(&bars->v_full[s], (gg / STAGES_V) & 1, abort_flag)) { ok = false; break; }
          // the first P.V product of an item overwrites O: the previous item's rows must be read out
          if (j == 0 && qi > 0 && !mbar_wait(&bars->o_free, (qi - 1) & 1, abort_flag)) { ok = false; break; }
          const uint64_t vdesc = desc_v0 + (uint64_t)((s * C::TILE_BYTES) >> 4);
          // The halves of the key columns are independent softmax streams with accumulators of
          // their own: O_h += P_h V[64h .. 64h+64), issued as soon as that half's P is there.
          // P_h sits in the first 32 columns of the half's own 64 S columns.
          for (int hh = 0; hh < 2 && ok; ++hh) {
            if (!mbar_wait(&bars->p_full[t][hh], (gg >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t p_tmem = tmem + (t ? C::COL_S1 : C::COL_S0) + hh * HALF_COLS;
            const uint32_t o_tmem = tmem + (hh ? C::COL_O1 : C::COL_O0);
#pragma unroll
            for (int kk = 0; kk < HALF_COLS / 16; ++kk) {
              // V tile is N-major: 16 keys = two 8-row groups (SBO 1024 B); the second 64 columns
              // of D live one panel further (LBO).  16 keys further = 2048 bytes.
              umma_ts(o_tmem, p_tmem + kk * 8, vdesc + (uint64_t)(((hh * 4 + kk) * 2048) >> 4), IDESC_PV,
                      (j > 0 || kk > 0) ? 1u : 0u);
            }
            if (SPLIT_S) umma_commit(&bars->pv_done[t][hh]);
          }
          if (!ok) break;
          umma_commit(&bars->v_empty[s]);
          if (!SPLIT_S) umma_commit(&bars->pv_done[t][0]);
        }
        g += n_tiles;
        ++qi;
      }
    }
  } else if (warp < SOFTMAX_THREADS / 32) {
    // ============================== softmax / epilogue ==============================
    // Two threads per query row: this thread owns row `rtid` of the item and the key columns
    // [half * 64, half * 64 + 64) of every tile.  The two halves are independent online-softmax
    // streams over disjoint key sets -- own reference maximum, own row sum, own accumulator O_h in
    // TMEM -- that never synchronise inside the tile loop, so the two warps of a scheduler drift
    // out of phase and one warp's exponentials (MUFU) overlap the other's loads, stores and waits.
    // They are merged once per item in the epilogue.
    const int half = warp >> 2, rtid = tid & (BM - 1);
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const float scale2 = p.sm_scale * kLog2e;     // > 0 (checked on the host)
    Item it;
    int g = 0, qi = 0;
    uint32_t pair_count = 0;
    bool alive = true;
    for (int round = 0; alive && get_item<EMASK, SPLIT>(args, round, it); ++round) {
      const TileWalk& walk = it.walk;
      const int n_tiles = walk.n_tiles;
      const int m0 = it.m0, b = it.b, h = it.h;
      const int row = m0 + rtid;
      if (ROPE != ROPE_NONE && n_tiles > 0 && half == 0) {
        if (mbar_wait(&bars->q_full, qi & 1, abort_flag)) {
          if (row < p.N_q)
            rope_row<T, D>(sQ, rtid, reinterpret_cast<const T*>(p.cos) + (int64_t)(row + p.q_offset) * p.rope_stride_n,
                           reinterpret_cast<const T*>(p.sin) + (int64_t)(row + p.q_offset) * p.rope_stride_n);
          fence_proxy_async_smem();
          mbar_arrive(&bars->q_ready);
        }
      }
      const float slope2 = ALIBI ? load_slope<T>(p.slopes, h) * kLog2e : 0.f;
      float m_ref = -INFINITY, l_part = 0.f;        // m_ref in log2 units of the scaled score
      bool ref_ok = false;   // warp-uniform: every row of the warp has a finite reference (it never becomes -inf again)

      for (int j = 0; j < n_tiles; ++j) {
        const int gg = g + j;                       // the CTA's running key-tile count
        const int t = gg & 1;
        const int key0 = walk.key0(j);
        if (!mbar_wait(&bars->s_full[t][SPLIT_S ? half : 0], (gg >> 1) & 1, abort_flag)) { alive = false; break; }
        tc_fence_after_sync();
        const uint32_t s_tmem = tmem + lane_base + (t ? C::COL_S1 : C::COL_S0);
        const uint32_t o_tmem = tmem + lane_base + (half ? C::COL_O1 : C::COL_O0);
        uint32_t xr[HALF_COLS];   // fp32 bit patterns of this thread's raw scores
        tmem_ld32(s_tmem + half * HALF_COLS, &xr[0]);
        tmem_ld32(s_tmem + half * HALF_COLS + 32, &xr[32]);
        tmem_wait_ld();

        // Tile-level decision: only edge / diagonal tiles pay for element masking.
        const int n_kv = SPLIT ? it.n_kv : p.N_kv;
        bool need_mask = key0 + BN > n_kv;
        const int pos0 = m0 + p.q_offset;           // position of the tile's first row on the key axis
        if (EMASK == EMASK_CAUSAL) need_mask = need_mask || (key0 + BN - 1 > pos0);
        if (EMASK == EMASK_WINDOW)
          need_mask = need_mask || (pos0 + BM - 1 - key0 >= p.window) || (key0 + BN - 1 - pos0 >= p.window);
        const int col0 = key0 + half * HALF_COLS;   // key index of this thread's column 0
        const int rel = row + p.q_offset - col0;    // column c is kept iff ...
        uint64_t tile_bits = ~0ull;                 // EMASK_BITS: this thread's 64 columns of the tile's bit matrix
        if (EMASK == EMASK_BITS && walk.slots != nullptr) {
          const int bs = walk.slots[j / walk.per_block];
          if (bs >= 0) {
            const int words = p.block_n >> 6;
            tile_bits = p.kv_bits[((int64_t)bs * p.block_m + (m0 % p.block_m) + rtid) * words + (j % walk.per_block) * 2 + half];
            need_mask = true;
          }
        }
        if (need_mask) {
          const int kmax = n_kv - col0;             // ... c < kmax
#pragma unroll
          for (int c = 0; c < HALF_COLS; ++c) {
            bool keep = c < kmax;
            if (EMASK == EMASK_CAUSAL) keep = keep && (c <= rel);
            if (EMASK == EMASK_WINDOW) keep = keep && (c - rel < p.window) && (rel - c < p.window);
            if (EMASK == EMASK_BITS) keep = keep && ((tile_bits >> c) & 1ull);
            xr[c] = keep ? xr[c] : 0xff800000u;     // -inf
          }
        }
        // ALiBi: the bias -slope |rel - c| is affine in the column, slope_c * c + bias0, wherever the
        // sign of rel - c is the same for all of the thread's visible columns: always under a
        // causal mask (visible columns have c <= rel), otherwise for threads whose row lies on
        // one side of their 64 columns.  Then the bias rides along in the exponent pass as one
        // more FMA; a warp with a row inside its columns takes the classic order below.
        float slope_c = 0.f, bias0 = 0.f;
        bool affine = true;
        if (ALIBI) {
          const bool below = (EMASK == EMASK_CAUSAL) || rel >= HALF_COLS - 1;
          affine = (EMASK == EMASK_CAUSAL) || __all_sync(0xffffffffu, below || rel <= 0);
          slope_c = below ? slope2 : -slope2;
          bias0 = -slope_c * (float)rel;
        }
        // Usual case: this half of the row already has a reference maximum and the tile does not
        // exceed it by much.  Then P is formed against the standing reference right away, without
        // a pass for the tile maximum; the row sum verifies the assumption for free (all terms are
        // non-negative, an overflow gives +inf; see kRowSumBound).  Otherwise -- first tile of an
        // item, no visible key so far, or a sum past the bound -- the classic order runs: maximum
        // first, reference update, accumulator rescale, then P.
        float alpha = 1.f, rsum = 0.f;
        uint32_t pk[HALF_COLS / 2];
        bool fast = ref_ok && affine;
        if (fast) {
          exp_pass<T, ALIBI ? EXP_AFFINE : EXP_SCALE>(xr, pk, scale2, bias0 - m_ref, slope_c, rsum);
          fast = __all_sync(0xffffffffu, rsum <= kRowSumBound);
        }
        if (!fast) {
          if (ALIBI) {
            const float relf = (float)rel;
#pragma unroll
            for (int c = 0; c < HALF_COLS; ++c)
              xr[c] = __float_as_uint(fmaf(__uint_as_float(xr[c]), scale2, -slope2 * fabsf(relf - (float)c)));
          }
          float mx = row_max(xr);
          if (!ALIBI) mx *= scale2;                   // the maximum commutes with the positive scale
          const bool bump = mx > m_ref + kRescaleThreshold;   // also true for the first finite max
          const float m_next = bump ? mx : m_ref;
          alpha = bump ? ex2_approx(m_ref - m_next) : 1.f;
          m_ref = m_next;
          ref_ok = __all_sync(0xffffffffu, m_ref != -INFINITY);
          const float neg_m = (m_next == -INFINITY) ? 0.f : -m_next;
          if (j > 0 && __any_sync(0xffffffffu, bump)) {
            // The accumulator is expressed relative to the old reference: rescale it in TMEM once
            // the previous P.V product has landed.
            if (!mbar_wait(&bars->pv_done[(gg - 1) & 1][SPLIT_S ? half : 0], ((gg - 1) >> 1) & 1, abort_flag)) { alive = false; break; }
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t o[32];
              tmem_ld32(o_tmem + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(o_tmem + c * 32, o);
            }
            tmem_wait_st();
          }
          exp_pass<T, ALIBI ? EXP_PRESCALED : EXP_SCALE>(xr, pk, scale2, neg_m, 0.f, rsum);
        }
        l_part = l_part * alpha + rsum;
        if (SPLIT && key0 + BN > n_kv) {
          // Split-K decode: cache rows past the valid length hold whatever the allocation held
          // (TMA zero-fills only past the tensor's extent) and 0 * NaN would poison O, so the
          // softmax threads clear those V rows of the stage before they release P.
          const int s = gg % STAGES_V;
          if (!mbar_wait(&bars->v_full[s], (gg / STAGES_V) & 1, abort_flag)) { alive = false; break; }
          // each half clears the rows its own P.V product reads (keys [64 half, 64 half + 64))
          const int first = max(n_kv - key0, half * HALF_COLS), last = (half + 1) * HALF_COLS;
          const uint32_t v_tile = sV0 + s * C::TILE_BYTES;
          for (int idx = rtid; idx < (last - first) * C::PANELS * 8; idx += BM) {
            const int r = first + idx / (C::PANELS * 8), rem = idx % (C::PANELS * 8);
            sts128(v_tile + (rem >> 3) * PANEL_BYTES + r * 128 + ((rem & 7) << 4), make_uint4(0u, 0u, 0u, 0u));
          }
          fence_proxy_async_smem();
        }
        tmem_st32(s_tmem + half * HALF_COLS, pk);   // P_h over the first half of the thread's own S columns
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&bars->p_full[t][half]);
      }

      // Epilogue.  The two halves of a row meet and each merges its half of the output columns
      // from both accumulators,
      //   O = (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) / (l_0 2^(m_0 - m) + l_1 2^(m_1 - m)),  m = max(m_0, m_1);
      // L = m + log(l).  The exchange runs while the last P.V product is still in flight: half 1
      // hands (m_1, l_1) to half 0, which returns the two accumulator weights c_h = 2^(m_h - m) / l
      // through the same words (two hand-shakes; the next item's words are written only after
      // this item's have been read).
      if (!alive) break;
      if (!SPLIT && lane == 0) bulk_wait_read_all();   // previous item's staged rows: long gone by now
      float c0 = 0.f, c1 = 0.f, m_all = 0.f, l_sum = 0.f;
      if (half == 1) {
        bars->xchg[rtid] = m_ref;
        bars->xchg[BM + rtid] = l_part;
      }
      if (!pair_sync(bars, warp, lane, pair_count, abort_flag)) { alive = false; break; }
      if (half == 0) {
        const float m_other = bars->xchg[rtid], l_other = bars->xchg[BM + rtid];
        m_all = fmaxf(m_ref, m_other);
        const float w_mine = (m_ref == -INFINITY) ? 0.f : ex2_approx(m_ref - m_all);
        const float w_other = (m_other == -INFINITY) ? 0.f : ex2_approx(m_other - m_all);
        l_sum = l_part * w_mine + l_other * w_other;
        // split-K decode keeps the partial un-normalised for the combine kernel
        const float inv = SPLIT ? 1.f : 1.f / ((l_sum == 0.f) ? 1.f : l_sum);
        c0 = w_mine * inv;
        c1 = w_other * inv;
        bars->xchg[rtid] = c0;
        bars->xchg[BM + rtid] = c1;
      }
      if (!pair_sync(bars, warp, lane, pair_count, abort_flag)) { alive = false; break; }
      if (half == 1) {
        c0 = bars->xchg[rtid];
        c1 = bars->xchg[BM + rtid];
      }
      if (n_tiles > 0) {
        const int gl = g + n_tiles - 1;
        if (!mbar_wait(&bars->pv_done[gl & 1][0], (gl >> 1) & 1, abort_flag) ||
            (SPLIT_S && !mbar_wait(&bars->pv_done[gl & 1][1], (gl >> 1) & 1, abort_flag))) { alive = false; break; }
        tc_fence_after_sync();
      }
      float o[D / 2];
      if (n_tiles > 0) {
        uint32_t o0[D / 2], o1[D / 2];
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tmem_ld32(tmem + lane_base + C::COL_O0 + half * (D / 2) + c * 32, &o0[c * 32]);
          tmem_ld32(tmem + lane_base + C::COL_O1 + half * (D / 2) + c * 32, &o1[c * 32]);
        }
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(&bars->o_free);
#pragma unroll
        for (int i = 0; i < D / 2; ++i) o[i] = __uint_as_float(o0[i]) * c0 + __uint_as_float(o1[i]) * c1;
      } else {
#pragma unroll
        for (int i = 0; i < D / 2; ++i) o[i] = 0.f;
      }
      if (SPLIT) {
        // split-K decode: un-normalised partial of this (split, batch, head) for the combine kernel
        // The fp32 rows go through the warp's staging region too, 32 columns at a time, and leave
        // as whole 128-byte lines (four rows per store instruction) instead of 32 lines per
        // instruction: rows of the partials are D floats apart and consecutive in the workspace.
        const int64_t wr0 = ((int64_t)it.split * p.B + b) * ((int64_t)p.H_q * p.N_q) + (int64_t)h * p.N_q + m0 + (warp & 3) * 32;
        const uint32_t stage = sO + (uint32_t)((half * 4 + (warp & 3)) * 32 * 128);
        const int rows_valid = min(32, p.N_q - (m0 + (warp & 3) * 32));   // rows of this warp that exist
#pragma unroll
        for (int part = 0; part < D / 64; ++part) {                       // 32 of the thread's D/2 columns per pass
          __syncwarp();
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8)
            sts128(stage + (uint32_t)(lane * 128 + ((c8 ^ (lane & 7)) << 4)),
                   make_uint4(__float_as_uint(o[part * 32 + c8 * 4]), __float_as_uint(o[part * 32 + c8 * 4 + 1]),
                              __float_as_uint(o[part * 32 + c8 * 4 + 2]), __float_as_uint(o[part * 32 + c8 * 4 + 3])));
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + (lane >> 3), c8 = lane & 7;
            if (r < rows_valid) {
              const uint4 v = lds128(stage + (uint32_t)(r * 128 + ((c8 ^ (r & 7)) << 4)));
              *reinterpret_cast<uint4*>(args.ws_acc + (wr0 + r) * D + half * (D / 2) + part * 32 + c8 * 4) = v;
            }
          }
        }
        if (half == 0 && row < p.N_q) {
          const int64_t wr = wr0 + lane;
          args.ws_m[wr] = m_all * kLn2;      // -inf when the split saw no key
          args.ws_l[wr] = l_sum;
        }
      } else {
        // The rows go out through shared memory: a thread owns one row, so direct stores touch 32
        // different 128-byte lines per instruction (measured: 3300 cycles per item).  Each warp
        // stages its 32 rows of D bytes in the 128-byte swizzle of the output tensor map --
        // conflict-free 16-byte stores -- and one lane sends them with a TMA store, which also
        // drops the rows past N_q.  The staging region is the warp's own; before it is written
        // again the previous store must have read it.
        const uint32_t stage = sO + (uint32_t)((half * 4 + (warp & 3)) * 32 * 128);
        __syncwarp();   // lane 0 has seen the previous store off (below, before the exchange)
#pragma unroll
        for (int q8 = 0; q8 < D / 16; ++q8) {
          uint4 v;
          v.x = Pack2<T>::run(o[q8 * 8 + 0], o[q8 * 8 + 1]);
          v.y = Pack2<T>::run(o[q8 * 8 + 2], o[q8 * 8 + 3]);
          v.z = Pack2<T>::run(o[q8 * 8 + 4], o[q8 * 8 + 5]);
          v.w = Pack2<T>::run(o[q8 * 8 + 6], o[q8 * 8 + 7]);
          sts128(stage + (uint32_t)(lane * 128 + ((q8 ^ (lane & 7)) << 4)), v);
        }
        fence_proxy_async_smem();
        __syncwarp();
        const int row0 = m0 + (warp & 3) * 32;
        if (lane == 0 && row0 < p.N_q) {
          tma_store_4d_hint(&tmap_o, stage, half * (D / 2), row0, h, b, l2_policy_evict_first());
          bulk_commit_group();
        }
        if (a.lse != nullptr && half == 0 && row < p.N_q)
          a.lse[(int64_t)b * a.lse_stride[0] + (int64_t)h * a.lse_stride[1] + (int64_t)row * a.lse_stride[2]] =
              m_all * kLn2 + logf((l_sum == 0.f) ? 1.f : l_sum);
      }
      if (n_tiles > 0) {
        g += n_tiles;
        ++qi;
      }
    }
    if (lane == 0) bulk_wait_all();   // the staged rows must have left shared memory before the CTA exits
  } else if (ROT_K && warp == WARP_ROTATE) {
    // ============================== K rotation warp ==============================
    // One warp; each thread rotates four key rows of the tile.
    const int r0 = lane;
    Item it;
    int g = 0;
    bool ok = true;
    for (int round = 0; ok && get_item<EMASK, SPLIT>(args, round, it); ++round) {
      const int n_tiles = it.walk.n_tiles;
      for (int j = 0; j < n_tiles; ++j) {
        const int gg = g + j;
        const int s = gg % STAGES;
        if (!mbar_wait(&bars->k_full[s], (gg / STAGES) & 1, abort_flag)) { ok = false; break; }
        const int key0 = it.walk.key0(j);
#pragma unroll 1
        for (int r = r0; r < BN; r += 32) {
          const int pos = key0 + r;
          if (pos < p.N_kv)
            rope_row<T, D>(sK0 + s * C::TILE_BYTES, r,
                           reinterpret_cast<const T*>(p.cos) + (int64_t)pos * p.rope_stride_n,
                           reinterpret_cast<const T*>(p.sin) + (int64_t)pos * p.rope_stride_n);
        }
        fence_proxy_async_smem();
        mbar_arrive(&bars->k_ready[s]);
      }
      g += n_tiles;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, AF_STATUS_WAIT_TIMEOUT);
  if (warp == WARP_PRODUCER) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------
// Launch of one instantiation (tensor maps are encoded by the host file)
// ---------------------------------------------------------------------------------------
template <typename T, int D, int ROPE, int EMASK, bool ALIBI, bool SPLIT = false>
int launch_instance(const TcArgs& args, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                    const CUtensorMap& mo, cudaStream_t st) {
  auto kern = fwd_tcgen05_kernel<T, D, ROPE, EMASK, ALIBI, SPLIT>;
  constexpr int smem = Cfg<D>::SMEM_BYTES;
  static bool configured = false;   // benign race: the attribute call is idempotent
  if (!configured) {
    AF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  kern<<<(unsigned)args.grid_ctas, ROPE == ROPE_FUSED ? 384 : 352, smem, st>>>(args, mq, mk, mv, mo);
  count_launch();
  return check_cuda(cudaGetLastError(), "fwd_tcgen05 launch");
}

// Composition -> instantiation table for one (dtype, head_dim, RoPE mode); defined in the
// per-(D, RoPE) translation units so that they compile in parallel.
template <typename T, int D, int ROPE>
int launch_composition(const TcArgs& args, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                       const CUtensorMap& mo, cudaStream_t st) {
  const AfProblem& p = args.a.p;
  if (args.num_splits > 0) {   // split-K decode: dense, no bias, no rotation (one extra instantiation)
    if constexpr (ROPE == ROPE_NONE) return launch_instance<T, D, ROPE_NONE, EMASK_NONE, false, true>(args, mq, mk, mv, mo, st);
    else return fail(AF_ERR_UNSUPPORTED, "split-K decode takes no rotation");
  }
  int em = p.mask_kind == AF_MASK_CAUSAL ? EMASK_CAUSAL : p.mask_kind == AF_MASK_WINDOW ? EMASK_WINDOW : EMASK_NONE;
  if (p.mask_kind == AF_MASK_BLOCKS && p.kv_slot != nullptr) em = EMASK_BITS;
  const bool alibi = p.bias_kind == AF_BIAS_ALIBI;
  if (em == EMASK_BITS) {
    // block lists never come with rotation (the block-sparse call has no cos / sin)
    if constexpr (ROPE == ROPE_NONE) {
      return alibi ? launch_instance<T, D, ROPE_NONE, EMASK_BITS, true>(args, mq, mk, mv, mo, st)
                   : launch_instance<T, D, ROPE_NONE, EMASK_BITS, false>(args, mq, mk, mv, mo, st);
    } else {
      return fail(AF_ERR_UNSUPPORTED, "block lists with element bit matrices take no rotation");
    }
  }
  switch (em * 2 + (alibi ? 1 : 0)) {
    case 0: return launch_instance<T, D, ROPE, EMASK_NONE, false>(args, mq, mk, mv, mo, st);
    case 1: return launch_instance<T, D, ROPE, EMASK_NONE, true>(args, mq, mk, mv, mo, st);
    case 2: return launch_instance<T, D, ROPE, EMASK_CAUSAL, false>(args, mq, mk, mv, mo, st);
    case 3: return launch_instance<T, D, ROPE, EMASK_CAUSAL, true>(args, mq, mk, mv, mo, st);
    case 4: return launch_instance<T, D, ROPE, EMASK_WINDOW, false>(args, mq, mk, mv, mo, st);
    default: return launch_instance<T, D, ROPE, EMASK_WINDOW, true>(args, mq, mk, mv, mo, st);
  }
}

// Entry points of the instantiation units: dtype is AF_F16 / AF_BF16.
int launch_d64_norope(int dtype, const TcArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);
int launch_d64_fused(int dtype, const TcArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);
int launch_d128_norope(int dtype, const TcArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);
int launch_d128_fused(int dtype, const TcArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);
int launch_pair_d128(int dtype, const TcArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);

#define AF_DEFINE_TC_UNIT(NAME, DIM, ROPE_MODE)                                                              \
  int NAME(int dtype, const TcArgs& args, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, \
           const CUtensorMap& mo, cudaStream_t st) {                                                         \
    if (dtype == AF_F16) return launch_composition<__half, DIM, ROPE_MODE>(args, mq, mk, mv, mo, st);        \
    return launch_composition<__nv_bfloat16, DIM, ROPE_MODE>(args, mq, mk, mv, mo, st);                      \
  }

}  // namespace tc
}  // namespace af
