// Backward attention on tcgen05 + TMEM: dK/dV (key-stationary) and dQ (query-stationary).
//
// Replaces the reference backward kernels (attnfuse/compiler/codegen_backward.py:75-302 and the
// block-sparse pair, attnfuse/compiler/codegen_blocksparse_bwd.py:29-233) for f16/bf16 inputs with
// head_dim 64 or 128.  Same two-pass structure as the reference -- no atomics, dK/dV of a GQA
// group are summed inside the CTA that owns the key tile -- with the recompute on tensor cores:
//
//   MODE_DKV  one CTA owns 128 keys of one (batch, kv head): K_j, V_j stay in shared memory,
//             64-row tiles of Q_i and dO_i stream through a TMA ring, for every query head of
//             the group.  Scores are computed TRANSPOSED, S^T = K_j Q_i^T and dP^T = V_j dO_i^T
//             (TMEM lane = key), so that P^T and dS^T, written back to TMEM as f16/bf16, are
//             directly the A operands of  dV_j += P^T dO_i  and  dK_j += dS^T Q_i.
//   MODE_DQ   one CTA owns 128 query rows of one (batch, query head): Q_i, dO_i stay, 64-key
//             tiles of K_j, V_j stream;  S = Q_i K_j^T, dP = dO_i V_j^T (TMEM lane = query row),
//             dS goes back to TMEM and feeds  dQ_i += dS K_j.
//
// P = exp2(S*scale*log2e - L*log2e) with L the log-sum-exp saved by the forward;
// dS = P * (dP - delta), delta = rowsum(dO * O); dK and dQ are multiplied by the scale at the
// end (codegen_backward.py:161-191).  With RoPE the operands are the pre-rotated Q', K' and the
// epilogue applies the transpose of the rotation to dQ', dK' while they are still fp32.
// S^T/dP^T (or S/dP) are double-buffered in TMEM so that the products of step i+1 run while the
// 128 element-wise threads work on step i; the products and the accumulations are issued by two
// different threads.  All waits are bounded.
//
//   MODE_FUSED  (head_dim 128) the key-stationary pass also produces dQ, so that S and dP are
//             computed once: 5 products per step instead of 7 over the two passes.  dS^T goes to
//             shared memory (128 keys x 64 queries, query-contiguous, 128-byte swizzle) instead
//             of TMEM and is read twice from there: as the K-major A operand of dK_j += dS^T Q_i
//             and as the N-major B operand of  dQ_i^T = K_j^T dS^T  (A = the stationary K tile
//             read M-major).  dQ_i^T (TMEM lane = d, column = query) is not kept: the element-wise
//             threads read it back and add it to an fp32 (B, H_q, N_q, D) accumulator in global
//             memory with red.global.add.f32 (32 lanes = 32 consecutive d = one 128-byte line);
//             a small kernel afterwards applies the scale and the transpose of the rotation and
//             rounds to the output type.  TMEM: S^T/P^T double-buffered, dP^T single (free again
//             as soon as the element-wise threads have loaded it), dQ^T single, dV, dK = 512
//             columns.  Summation order of dQ over key tiles depends on scheduling, so dQ is
//             reproducible only to fp32 rounding; the two-pass kernels remain the deterministic
//             option.  Work items are handed out dynamically (one atomic counter, published to
//             the roles through a 4-deep shared-memory ring) in an order that keeps the dQ
//             accumulator rows of the (batch, kv head) units in flight inside the L2.
#pragma once
#include <type_traits>

#include "fwd_tcgen05.cuh"

namespace af {
namespace tcb {

using namespace ptx;
using tc::Pack2;
using tc::ex2_approx;

enum { MODE_DKV = 0, MODE_DQ = 1, MODE_FUSED = 2 };
enum { EMASK_NONE = 0, EMASK_CAUSAL = 1, EMASK_WINDOW = 2, EMASK_BITS = 3 };   // element-level mask of the instantiation
// (EMASK_BITS: block lists in which some blocks carry a bit matrix of their active elements)

constexpr int BS = 128;   // rows of the stationary operands (TMEM lanes)
constexpr int BT = 64;    // rows of a streamed tile (columns of S per step)

template <int D, int MODE = MODE_DKV> struct BCfg {
  static constexpr bool FUSED = MODE == MODE_FUSED;
  static constexpr int PANELS = D / 64;
  static constexpr int STAT_PANEL = BS * 128;               // bytes of a 128-row, 64-element panel
  static constexpr int STRM_PANEL = BT * 128;
  static constexpr int STAT_TILE = PANELS * STAT_PANEL;
  static constexpr int STRM_TILE = PANELS * STRM_PANEL;
  static constexpr int STAGES = FUSED ? 3 : 4;
  static constexpr int STATS_BYTES = 2 * BT * 4;            // L*log2e and delta of a streamed tile
  static constexpr int DS_TILE = BS * BT * 2;               // dS^T of one step (fused mode): 128 keys x 64 queries
  static constexpr int DS_BYTES = FUSED ? 2 * DS_TILE : 0;  // two buffers, right after the stationary tiles
  static constexpr int SMEM_BYTES = 2 * STAT_TILE + DS_BYTES + STAGES * (2 * STRM_TILE + STATS_BYTES) + 1024 + 512;
  static constexpr int TMEM_COLS = 512;
  // two-pass: X0 Y0 X1 Y1; fused: X0 X1 Y Z (Y = dP^T, single; Z = dQ^T, single)
  static constexpr int COL_X0 = 0, COL_Y0 = FUSED ? 128 : 64, COL_X1 = FUSED ? 64 : 128, COL_Y1 = FUSED ? 128 : 192;
  static constexpr int COL_Z = 192, COL_ACC1 = 256, COL_ACC2 = 256 + D;
  // MODE_DQ has one accumulator only: dS gets columns of its own (two buffers of 32), so the next
  // S / dP product does not have to wait until dQ += dS K has consumed the previous dS.
  static constexpr int COL_DS0 = 384, COL_DS1 = 416;
};

struct BBarriers {
  uint64_t stat_full, stat_empty, acc_free;
  uint64_t strm_full[4], strm_empty[4];
  uint64_t xy_full[2], p_full[2], acc_done[2];
  uint64_t y_free, z_free;                      // fused mode: dP^T loaded / dQ^T loaded by the element-wise threads
  uint64_t sched_full[4], sched_empty[4];       // fused mode: ring of dynamically fetched item numbers
  int32_t sched_item[4];
  uint32_t tmem_base;
  int abort_flag;
};

struct BwdArgs {
  AfBwdParams a;
  int tiles;            // stationary tiles along the sequence
  int steps_per_block;  // block lists: streamed 64-row steps per listed block
  int stat_per_block;   // block lists: stationary 128-row tiles per block
  int total_items;      // tiles * B * heads: stationary tiles to process
  int grid_ctas;        // one persistent CTA per SM (or one per item when there are fewer)
  // fused mode
  float* dq_acc;        // fp32 (B, H_q, N_q, D) accumulator, zeroed before the launch
  int32_t* sched_counter;   // zeroed before the launch
  int chunk_units;      // (batch, kv head) units per scheduling chunk
};

// The streamed steps one stationary tile visits for one head.
struct StepWalk {
  int cnt, first;
  const int32_t* list;
  const int32_t* slots;      // bit-matrix number of each listed block (-1: fully active), or null
  int per, block;
  __device__ __forceinline__ int row0(int s) const {
    if (list != nullptr) return list[s / per] * block + (s % per) * BT;
    return (first + s) * BT;
  }
};

template <int MODE>
__device__ __forceinline__ StepWalk make_steps(const AfProblem& p, const BwdArgs& args, int tile, int h) {
  StepWalk w;
  w.list = nullptr; w.slots = nullptr; w.per = 1; w.block = BT; w.first = 0;
  const int t0 = tile * BS;
  if (p.mask_kind == AF_MASK_BLOCKS) {
    const int blk = tile / args.stat_per_block;
    w.per = args.steps_per_block;
    if (MODE != MODE_DQ) {
      w.block = p.block_m;
      w.list = p.q_idx + (int64_t)h * p.q_idx_stride_h + (int64_t)blk * p.q_idx_stride_k;
      if (p.q_slot != nullptr) w.slots = p.q_slot + (int64_t)h * p.q_idx_stride_h + (int64_t)blk * p.q_idx_stride_k;
      w.cnt = p.q_num[(int64_t)h * p.q_num_stride_h + blk] * w.per;
    } else {
      w.block = p.block_n;
      w.list = p.kv_idx + (int64_t)h * p.kv_idx_stride_h + (int64_t)blk * p.kv_idx_stride_q;
      if (p.kv_slot != nullptr) w.slots = p.kv_slot + (int64_t)h * p.kv_idx_stride_h + (int64_t)blk * p.kv_idx_stride_q;
      w.cnt = p.kv_num[(int64_t)h * p.kv_num_stride_h + blk] * w.per;
    }
  } else if (p.mask_kind == AF_MASK_WINDOW) {
    // rows of the streamed operand within |i - j| < window of the stationary tile [t0, t0 + BS)
    const int n_strm = (MODE != MODE_DQ) ? p.N_q : p.N_kv;
    const int lo = max(0, t0 - p.window + 1), hi = min(n_strm, t0 + BS + p.window - 1);
    w.first = lo / BT;
    w.cnt = hi > lo ? (hi + BT - 1) / BT - w.first : 0;
  } else if (MODE != MODE_DQ) {
    const int total = (p.N_q + BT - 1) / BT;
    w.first = (p.mask_kind == AF_MASK_CAUSAL) ? t0 / BT : 0;     // query rows >= first key of the tile
    w.cnt = total - w.first;
  } else {
    const int hi = (p.mask_kind == AF_MASK_CAUSAL) ? min(min(t0 + BS, p.N_q), p.N_kv) : p.N_kv;
    w.cnt = (hi + BT - 1) / BT;
  }
  if (w.cnt < 0) w.cnt = 0;
  return w;
}

// One work item = one stationary 128-row tile of one (batch, head).  Items are numbered heaviest
// first and taken in a zig-zag by the persistent CTAs (item r*G + c in even rounds r, r*G + G-1-c
// in odd rounds), exactly as in the forward kernel.
struct BItem {
  int tile, b, hx, h_kv, t0, total_steps;
};

template <int MODE, int EMASK>
__device__ __forceinline__ void decode_bitem(const AfProblem& p, const BwdArgs& args, int w, BItem& bi) {
  const int grp = p.H_q / p.H_kv;
  const int heads = (MODE != MODE_DQ) ? p.H_kv : p.H_q;
  const int bh_count = p.B * heads;
  int bh;
  if (MODE == MODE_FUSED) {
    // Chunks of `chunk_units` (batch, kv head) units, tile-major (heaviest key tiles first) inside
    // a chunk: the dQ accumulator rows and the Q / dO tiles of the units in flight stay in the L2,
    // and the dynamic hand-out keeps the SMs busy to the end of each chunk.
    const int per_chunk = args.chunk_units * args.tiles;
    const int chunk = w / per_chunk, idx = w - chunk * per_chunk;
    const int units_here = min(args.chunk_units, bh_count - chunk * args.chunk_units);
    bi.tile = idx / units_here;
    bh = chunk * args.chunk_units + idx % units_here;
  } else {
    // heaviest tiles first: causal dK/dV work shrinks with the key tile index, dQ work grows with
    // the query tile index
    bi.tile = (MODE == MODE_DQ && EMASK == EMASK_CAUSAL) ? (args.tiles - 1 - w / bh_count) : (w / bh_count);
    bh = w % bh_count;
  }
  bi.b = bh / heads;
  bi.hx = bh % heads;                                    // kv head (DKV, fused) or query head (DQ)
  bi.h_kv = (MODE != MODE_DQ) ? bi.hx : bi.hx / grp;
  bi.t0 = bi.tile * BS;
  const int heads_per_item = (MODE != MODE_DQ) ? grp : 1;
  bi.total_steps = 0;                                    // all heads of the group in DKV mode
  for (int g = 0; g < heads_per_item; ++g)
    bi.total_steps += make_steps<MODE>(p, args, bi.tile, (MODE != MODE_DQ) ? bi.h_kv * grp + g : bi.hx).cnt;
}

// Item number k of this CTA.  Two-pass modes: static zig-zag.  Fused mode: the producer warp draws
// the numbers from a global counter and publishes them through a 4-deep ring; every other role
// (two issuing threads, 128 element-wise threads) reads slot k % 4 and releases it.
// Returns 1 (item), 0 (no more items) or -1 (aborted wait).
template <int MODE, int EMASK, bool IS_PRODUCER>
__device__ __forceinline__ int next_bitem(const AfProblem& p, const BwdArgs& args, BBarriers* bars, int k, int lane,
                                          volatile int* abort_flag, BItem& bi) {
  int w;
  if (MODE == MODE_FUSED) {
    const int slot = k & 3;
    if (IS_PRODUCER) {
      // all 32 lanes of the producer warp call this; lane 0 draws and publishes
      int drawn = 0;
      if (lane == 0) {
        if (k >= 4 && !mbar_wait(&bars->sched_empty[slot], ((k >> 2) - 1) & 1, abort_flag)) drawn = -1;
        else {
          drawn = atomicAdd(args.sched_counter, 1);
          bars->sched_item[slot] = drawn;
          mbar_arrive(&bars->sched_full[slot]);     // release: the store above is visible to waiters
        }
      }
      w = __shfl_sync(0xffffffffu, drawn, 0);
      if (w < 0) return -1;
    } else {
      if (!mbar_wait(&bars->sched_full[slot], (k >> 2) & 1, abort_flag)) return -1;
      w = bars->sched_item[slot];
      mbar_arrive(&bars->sched_empty[slot]);
    }
    if (w >= args.total_items) return 0;
  } else {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const int64_t w64 = (int64_t)k * G + ((k & 1) ? G - 1 - c : c);
    if (w64 >= args.total_items) return 0;
    w = (int)w64;
  }
  decode_bitem<MODE, EMASK>(p, args, w, bi);
  return 1;
}

template <typename T, int D, int MODE, int EMASK, bool ALIBI, bool ROPE>
__global__ void __launch_bounds__(224, 1)
bwd_tcgen05_kernel(const BwdArgs args, const __grid_constant__ CUtensorMap map_a1,
                   const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b1,
                   const __grid_constant__ CUtensorMap map_b2) {
  using C = BCfg<D, MODE>;
  constexpr bool FUSED = MODE == MODE_FUSED;
  constexpr bool KVS = MODE != MODE_DQ;          // key-stationary: MODE_DKV and MODE_FUSED
  static_assert(!FUSED || D == 128, "the fused pass computes dQ^T with M = head_dim = 128");
  constexpr int STAGES = C::STAGES;
  constexpr int AB_FMT = (Elem<T>::code == AF_BF16) ? 1 : 0;
  constexpr uint32_t IDESC_XY = umma_idesc_f16(AB_FMT, BS, BT, 0, 0);
  constexpr uint32_t IDESC_ACC = umma_idesc_f16(AB_FMT, BS, D, 0, 1);
  constexpr uint32_t IDESC_DQT = umma_idesc_f16(AB_FMT, D, BT, 1, 1);   // dQ^T = K^T dS^T: A M-major, B N-major
  constexpr int STAGE_BYTES = 2 * C::STRM_TILE + C::STATS_BYTES;
  constexpr int STAGE0_OFF = 2 * C::STAT_TILE + C::DS_BYTES;

  const AfBwdParams& a = args.a;
  const AfProblem& p = a.p;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sA1 = smem_base, sA2 = smem_base + C::STAT_TILE;
  const uint32_t sDS0 = smem_base + 2 * C::STAT_TILE;           // fused mode: two dS^T buffers (1024-byte aligned)
  const uint32_t sStage0 = smem_base + STAGE0_OFF;
  BBarriers* bars = reinterpret_cast<BBarriers*>(smem + STAGE0_OFF + STAGES * STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = p.H_q / p.H_kv;
  const int n_heads = KVS ? group : 1;

  if (tid == 0) {
    mbar_init(&bars->stat_full, 1);
    mbar_init(&bars->stat_empty, FUSED ? 2 : 1);   // fused: both issuing threads read the stationary K tile
    mbar_init(&bars->acc_free, 128);
    mbar_init(&bars->y_free, 128);
    mbar_init(&bars->z_free, 128);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&bars->strm_full[s], 1);
      mbar_init(&bars->strm_empty[s], 1);
      mbar_init(&bars->sched_full[s], 1);
      mbar_init(&bars->sched_empty[s], 130);       // two issuing threads + 128 element-wise threads
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bars->xy_full[t], 1);
      mbar_init(&bars->p_full[t], 128);
      mbar_init(&bars->acc_done[t], 1);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(&bars->tmem_base, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;

  // Every role walks the same item sequence.  `it0` counts the steps of the items before the
  // current one: ring stages, X/Y buffers and barrier phases run on the running count, so that the
  // loads and the first products of the next item overlap the previous item's epilogue; `qi`
  // counts the items with at least one step (phases of the stationary-tile and accumulator
  // hand-overs).
  if (warp == 4) {
    // ============================== producer (TMA + per-step statistics) ==============================
    if (lane == 0) {
      tma_prefetch_desc(&map_a1); tma_prefetch_desc(&map_a2); tma_prefetch_desc(&map_b1); tma_prefetch_desc(&map_b2);
    }
    // L2 hints: the stationary tiles are read once per item, the streamed rows once per stationary
    // tile of their unit
    const uint64_t pol_once = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();
    BItem bi;
    int it0 = 0, qi = 0;
    bool ok = true;
    for (int k = 0; ok && next_bitem<MODE, EMASK, true>(p, args, bars, k, lane, abort_flag, bi) > 0; ++k) {
      if (bi.total_steps == 0) continue;
      const int tile = bi.tile, b = bi.b, hx = bi.hx, h_kv = bi.h_kv, t0 = bi.t0;
      // the stationary tiles are free once the last product of the previous item that reads them has run
      if (qi > 0 && !mbar_wait(&bars->stat_empty, (qi - 1) & 1, abort_flag)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&bars->stat_full, 2 * C::STAT_TILE);
        const int ha = KVS ? h_kv : hx;
#pragma unroll
        for (int pn = 0; pn < C::PANELS; ++pn) {
          tma_load_4d_hint(smem + pn * C::STAT_PANEL, &map_a1, &bars->stat_full, pn * 64, t0, ha, b, pol_once);
          tma_load_4d_hint(smem + C::STAT_TILE + pn * C::STAT_PANEL, &map_a2, &bars->stat_full, pn * 64, t0, ha, b, pol_once);
        }
      }
      int it = it0;                                                   // running step count
      for (int g = 0; g < n_heads && ok; ++g) {
        const int h = KVS ? h_kv * group + g : hx;
        const int hb = KVS ? h : h_kv;                                // head of the streamed tensors
        const StepWalk w = make_steps<MODE>(p, args, tile, h);
        for (int s = 0; s < w.cnt; ++s, ++it) {
          const int st = it % STAGES;
          if (it >= STAGES && !mbar_wait(&bars->strm_empty[st], ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
          const int r0 = w.row0(s);
          unsigned char* stage = smem + STAGE0_OFF + st * STAGE_BYTES;
          // The TMA loads go out first; the statistics of the streamed rows (two global loads per
          // lane) are fetched while they fly, and the warp's arrival completes the stage.
          if (lane == 0) {
            mbar_expect_tx(&bars->strm_full[st], 2 * C::STRM_TILE);
#pragma unroll
            for (int pn = 0; pn < C::PANELS; ++pn) {
              tma_load_4d_hint(stage + pn * C::STRM_PANEL, &map_b1, &bars->strm_full[st], pn * 64, r0, hb, b, pol_keep);
              tma_load_4d_hint(stage + C::STRM_TILE + pn * C::STRM_PANEL, &map_b2, &bars->strm_full[st], pn * 64, r0, hb, b, pol_keep);
            }
          }
          if (KVS) {
            // L*log2e and delta of the 64 streamed query rows; rows past N_q get (+inf, 0) so that
            // their probabilities are exactly zero.
            float* stats = reinterpret_cast<float*>(stage + 2 * C::STRM_TILE);
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2) {
              const int q = r0 + lane + 32 * k2;
              float l2 = INFINITY, dl = 0.f;
              if (q < p.N_q) {
                const float l = a.lse[(int64_t)b * a.lse_stride[0] + (int64_t)h * a.lse_stride[1] + (int64_t)q * a.lse_stride[2]];
                l2 = (l == -INFINITY) ? INFINITY : l * kLog2e;
                dl = a.delta[((int64_t)b * p.H_q + h) * p.N_q + q];
              }
              stats[lane + 32 * k2] = l2;
              stats[BT + lane + 32 * k2] = dl;
            }
            __syncwarp();
          }
          if (lane == 0) mbar_arrive(&bars->strm_full[st]);
        }
      }
      it0 += bi.total_steps;
      ++qi;
    }
  } else if (warp == 5) {
    // ============================== MMA issuer 1: S / dP products ==============================
    // Two issuing threads feed the tensor pipe: a tcgen05.mma issue blocks while the pipe's short
    // queue is full, so one thread issuing both kinds leaves the pipe idle during its own barrier
    // waits and commits (measured: 1800 - 2100 cycles per step for 1000 - 1300 cycles of MMA).
    if (lane == 0) {
      const uint64_t desc_a1 = umma_desc_sw128(sA1, 16, 1024), desc_a2 = umma_desc_sw128(sA2, 16, 1024);
      const uint64_t desc_b1k = umma_desc_sw128(sStage0, 16, 1024);              // streamed tile, K-major
      BItem bi;
      int it0 = 0, qi = 0;
      bool ok = true;
      for (int k = 0; ok && next_bitem<MODE, EMASK, false>(p, args, bars, k, lane, abort_flag, bi) > 0; ++k) {
      if (bi.total_steps == 0) continue;
      ok = mbar_wait(&bars->stat_full, qi & 1, abort_flag);
      for (int it = it0; ok && it < it0 + bi.total_steps; ++it) {     // `it`: running step count
        const int st = it % STAGES, t = it & 1;
        if (!mbar_wait(&bars->strm_full[st], (it / STAGES) & 1, abort_flag)) { ok = false; break; }
        // X/Y[t] were last used by step it-2.  Key-stationary modes: P^T (and dS^T) overwrite X/Y,
        // so the accumulate MMAs of that step must have run.  MODE_DQ: the element-wise group must
        // have read them (its arrival on p_full).
        if (it >= 2) {
          uint64_t* free_bar = KVS ? &bars->acc_done[t] : &bars->p_full[t];
          if (!mbar_wait(free_bar, ((it >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
        }
        tc_fence_after_sync();
        // Descriptors are built once; k-steps and ring stages only move the start-address field.
        const uint64_t b1 = desc_b1k + (uint64_t)((st * STAGE_BYTES) >> 4), b2 = b1 + (uint64_t)(C::STRM_TILE >> 4);
        const uint32_t xt = tmem + (t ? C::COL_X1 : C::COL_X0), yt = tmem + (t ? C::COL_Y1 : C::COL_Y0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_ss(xt, desc_a1 + (uint64_t)(((kk >> 2) * C::STAT_PANEL + (kk & 3) * 32) >> 4),
                  b1 + (uint64_t)(((kk >> 2) * C::STRM_PANEL + (kk & 3) * 32) >> 4), IDESC_XY, kk > 0 ? 1u : 0u);
        if (FUSED && it >= 1) {
          // the single dP^T buffer: the element-wise threads have loaded the previous step's values
          if (!mbar_wait(&bars->y_free, (it - 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_ss(yt, desc_a2 + (uint64_t)(((kk >> 2) * C::STAT_PANEL + (kk & 3) * 32) >> 4),
                  b2 + (uint64_t)(((kk >> 2) * C::STRM_PANEL + (kk & 3) * 32) >> 4), IDESC_XY, kk > 0 ? 1u : 0u);
        umma_commit(&bars->xy_full[t]);
      }
      if (ok) umma_commit(&bars->stat_empty);   // the item's last products: the stationary tiles may be refilled
      it0 += bi.total_steps;
      ++qi;
      }
    }
  } else if (warp == 6) {
    // ============================== MMA issuer 2: gradient accumulation ==============================
    if (lane == 0) {
      const uint64_t desc_b1n = umma_desc_sw128(sStage0, C::STRM_PANEL, 1024);   // streamed tile, N-major
      // fused mode: dS^T (128 keys x 64 queries, query-contiguous) as K-major A and as N-major B;
      // the stationary K tile (128 keys x D) as M-major A (M = d: 64-element panels LBO apart)
      const uint64_t desc_ds_k = umma_desc_sw128(sDS0, 16, 1024);
      const uint64_t desc_ds_n = umma_desc_sw128(sDS0, C::DS_TILE, 1024);
      const uint64_t desc_k_m = umma_desc_sw128(sA1, C::STAT_PANEL, 1024);
      BItem bi;
      int it0 = 0, qi = 0;
      bool ok = true;
      for (int k = 0; ok && next_bitem<MODE, EMASK, false>(p, args, bars, k, lane, abort_flag, bi) > 0; ++k) {
      if (bi.total_steps == 0) continue;
      for (int it = it0; it < it0 + bi.total_steps; ++it) {            // `it`: running step count
        const int st = it % STAGES, t = it & 1;
        const bool first = it == it0;                                  // overwrites the accumulators
        if (!mbar_wait(&bars->strm_full[st], (it / STAGES) & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&bars->p_full[t], (it >> 1) & 1, abort_flag)) { ok = false; break; }
        // the previous item's epilogue must have read the accumulators out
        if (first && qi > 0 && !mbar_wait(&bars->acc_free, (qi - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint64_t b1 = desc_b1n + (uint64_t)((st * STAGE_BYTES) >> 4), b2 = b1 + (uint64_t)(C::STRM_TILE >> 4);
        const uint32_t xt = tmem + (t ? C::COL_X1 : C::COL_X0), yt = tmem + (t ? C::COL_Y1 : C::COL_Y0);
        // streamed tiles as N-major B operands: 16 rows per k-step (2048 B), panels LBO apart
        if (FUSED) {
          const uint64_t ds_k = desc_ds_k + (uint64_t)((t * C::DS_TILE) >> 4);
          const uint64_t ds_n = desc_ds_n + (uint64_t)((t * C::DS_TILE) >> 4);
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk)      // dV += P^T dO
            umma_ts(tmem + C::COL_ACC1, xt + kk * 8, b2 + (uint64_t)((kk * 2048) >> 4), IDESC_ACC,
                    (!first || kk > 0) ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk)      // dK += dS^T Q, dS^T from shared memory
            umma_ss(tmem + C::COL_ACC2, ds_k + (uint64_t)((kk * 32) >> 4), b1 + (uint64_t)((kk * 2048) >> 4), IDESC_ACC,
                    (!first || kk > 0) ? 1u : 0u);
          // the single dQ^T buffer: the element-wise threads have loaded the previous step's tile
          if (it >= 1) {
            if (!mbar_wait(&bars->z_free, (it - 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
          }
#pragma unroll
          for (int kk = 0; kk < BS / 16; ++kk)      // dQ^T = K^T dS^T over the 128 keys
            umma_ss(tmem + C::COL_Z, desc_k_m + (uint64_t)((kk * 2048) >> 4), ds_n + (uint64_t)((kk * 2048) >> 4),
                    IDESC_DQT, kk > 0 ? 1u : 0u);
        } else if (MODE == MODE_DKV) {
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk)      // dV += P^T dO
            umma_ts(tmem + C::COL_ACC1, xt + kk * 8, b2 + (uint64_t)((kk * 2048) >> 4), IDESC_ACC,
                    (!first || kk > 0) ? 1u : 0u);
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk)      // dK += dS^T Q
            umma_ts(tmem + C::COL_ACC2, yt + kk * 8, b1 + (uint64_t)((kk * 2048) >> 4), IDESC_ACC,
                    (!first || kk > 0) ? 1u : 0u);
        } else {
          const uint32_t dst = tmem + (t ? C::COL_DS1 : C::COL_DS0);
#pragma unroll
          for (int kk = 0; kk < BT / 16; ++kk)      // dQ += dS K
            umma_ts(tmem + C::COL_ACC1, dst + kk * 8, b1 + (uint64_t)((kk * 2048) >> 4), IDESC_ACC,
                    (!first || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bars->strm_empty[st]);
        umma_commit(&bars->acc_done[t]);
      }
      if (FUSED && ok) umma_commit(&bars->stat_empty);   // dQ^T reads the stationary K tile too
      it0 += bi.total_steps;
      ++qi;
      }
    }
  } else if (warp < 4) {
    // ============================== element-wise group / epilogue ==============================
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float scale2 = p.sm_scale * kLog2e;
    BItem bi;
    int it0 = 0;
    bool alive = true;
    // Fused mode: read the dQ^T tile of step `k` (TMEM lane = d = tid, column = query) and add it to
    // the fp32 accumulator rows; a warp's 32 lanes cover 32 consecutive d of one query row.
    auto drain_dq = [&](int k, float* acc_rows, int n_valid) -> bool {
      if (!mbar_wait(&bars->acc_done[k & 1], (k >> 1) & 1, abort_flag)) return false;
      tc_fence_after_sync();
      uint32_t zr[BT];
      tmem_ld32(tmem + lane_base + C::COL_Z, &zr[0]);
      tmem_ld32(tmem + lane_base + C::COL_Z + 32, &zr[32]);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(&bars->z_free);
      if (n_valid >= BT) {
#pragma unroll
        for (int c = 0; c < BT; ++c) atomicAdd(acc_rows + c * D, __uint_as_float(zr[c]));
      } else {
#pragma unroll
        for (int c = 0; c < BT; ++c)
          if (c < n_valid) atomicAdd(acc_rows + c * D, __uint_as_float(zr[c]));
      }
      return true;
    };
    float* pend_rows = nullptr;                      // fused: accumulator rows of the step not yet drained
    int pend_valid = 0, pend_it = -1;
    for (int kitem = 0; alive; ++kitem) {
    const int got = next_bitem<MODE, EMASK, false>(p, args, bars, kitem, lane, abort_flag, bi);
    if (got <= 0) break;
    const int tile = bi.tile, b = bi.b, hx = bi.hx, h_kv = bi.h_kv, t0 = bi.t0, total_steps = bi.total_steps;
    const int srow = t0 + tid;                       // key (DKV) or query row (DQ) of this thread
    float l2_row = INFINITY, dl_row = 0.f;           // DQ mode: statistics of this thread's query row
    if (MODE == MODE_DQ && srow < p.N_q) {
      const float l = a.lse[(int64_t)b * a.lse_stride[0] + (int64_t)hx * a.lse_stride[1] + (int64_t)srow * a.lse_stride[2]];
      l2_row = (l == -INFINITY) ? INFINITY : l * kLog2e;
      dl_row = a.delta[((int64_t)b * p.H_q + hx) * p.N_q + srow];
    }
    int it = it0;                                    // running step count
    for (int g = 0; g < n_heads && alive; ++g) {
      const int h = KVS ? h_kv * group + g : hx;
      const StepWalk w = make_steps<MODE>(p, args, tile, h);
      const float slope2 = ALIBI ? load_slope<T>(p.slopes, h) * kLog2e : 0.f;
      for (int s = 0; s < w.cnt; ++s, ++it) {
        const int st = it % STAGES, t = it & 1;
        const int r0 = w.row0(s);
        if (KVS && !mbar_wait(&bars->strm_full[st], (it / STAGES) & 1, abort_flag)) { alive = false; break; }
        if (!mbar_wait(&bars->xy_full[t], (it >> 1) & 1, abort_flag)) { alive = false; break; }
        tc_fence_after_sync();
        const uint32_t xt = tmem + lane_base + (t ? C::COL_X1 : C::COL_X0);
        const uint32_t yt = tmem + lane_base + (t ? C::COL_Y1 : C::COL_Y0);
        uint32_t xr[BT], yr[BT];
        tmem_ld32(xt, &xr[0]); tmem_ld32(xt + 32, &xr[32]);
        tmem_ld32(yt, &yr[0]); tmem_ld32(yt + 32, &yr[32]);
        tmem_wait_ld();
        if (FUSED) {
          // dP^T is in registers: the next step's dP^T product may overwrite the buffer
          tc_fence_before_sync();
          mbar_arrive(&bars->y_free);
        }
        const float* stats = reinterpret_cast<const float*>(smem + STAGE0_OFF + st * STAGE_BYTES + 2 * C::STRM_TILE);

        // Tile-level: does any element of this 128 x 64 tile need masking?
        //   key-stationary: lane = key srow, column c = query r0 + c;  DQ: lane = query srow, column c = key r0 + c.
        const int col_limit = (KVS ? p.N_q : p.N_kv) - r0;     // columns c < col_limit exist
        bool need_mask = col_limit < BT;
        if (EMASK == EMASK_CAUSAL)
          need_mask = need_mask || (KVS ? (r0 < t0 + BS - 1) : (r0 + BT - 1 > t0));
        if (EMASK == EMASK_WINDOW)
          need_mask = need_mask || (r0 + BT - 1 - t0 >= p.window) || (t0 + BS - 1 - r0 >= p.window);
        const int rel = srow - r0;   // key-stationary: query c kept iff c >= rel;  DQ: key c kept iff c <= rel
        uint64_t tile_bits = ~0ull;  // EMASK_BITS: this lane's 64 columns of the block's bit matrix
        if (EMASK == EMASK_BITS && w.slots != nullptr) {
          const int bs = w.slots[s / w.per];
          if (bs >= 0) {
            // key-stationary: rows of q_bits are keys, bits are queries; DQ: rows of kv_bits are queries
            const int stat_block = KVS ? p.block_n : p.block_m;
            const uint64_t* bits = KVS ? p.q_bits : p.kv_bits;
            tile_bits = bits[((int64_t)bs * stat_block + (t0 % stat_block) + tid) * (w.block >> 6) + (s % w.per)];
            need_mask = true;
          }
        }

        uint32_t pk[BT / 2], dk[BT / 2];
        const float relf = (float)rel;
        // The masking decision is taken once per tile: the element loop exists in a masked and an
        // unmasked copy, and the per-column statistics come in float4 shared-memory loads.
        auto element_pass = [&](auto masked_tag) {
          constexpr bool MASKED = decltype(masked_tag)::value;
#pragma unroll
          for (int c = 0; c < BT; c += 4) {
            float l2v[4], dlv[4];
            if (KVS) {
              const float4 a4 = *reinterpret_cast<const float4*>(stats + c);
              const float4 b4 = *reinterpret_cast<const float4*>(stats + BT + c);
              l2v[0] = a4.x; l2v[1] = a4.y; l2v[2] = a4.z; l2v[3] = a4.w;
              dlv[0] = b4.x; dlv[1] = b4.y; dlv[2] = b4.z; dlv[3] = b4.w;
            } else {
#pragma unroll
              for (int u = 0; u < 4; ++u) { l2v[u] = l2_row; dlv[u] = dl_row; }
            }
            float pe[4], de[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int cc = c + u;
              float e = fmaf(__uint_as_float(xr[cc]), scale2, -l2v[u]);
              if (ALIBI) e -= slope2 * fabsf(relf - (float)cc);
              float pr = ex2_approx(e);
              if (MASKED) {
                bool keep = cc < col_limit;
                if (EMASK == EMASK_CAUSAL) keep = keep && (KVS ? (cc >= rel) : (cc <= rel));
                if (EMASK == EMASK_WINDOW) keep = keep && (cc - rel < p.window) && (rel - cc < p.window);
                if (EMASK == EMASK_BITS) keep = keep && ((tile_bits >> cc) & 1ull);
                pr = keep ? pr : 0.f;
              }
              pe[u] = pr;
              de[u] = pr * (__uint_as_float(yr[cc]) - dlv[u]);
            }
            pk[c >> 1] = Pack2<T>::run(pe[0], pe[1]);
            pk[(c >> 1) + 1] = Pack2<T>::run(pe[2], pe[3]);
            dk[c >> 1] = Pack2<T>::run(de[0], de[1]);
            dk[(c >> 1) + 1] = Pack2<T>::run(de[2], de[3]);
          }
        };
        if (need_mask) element_pass(std::true_type{});
        else element_pass(std::false_type{});
        if (FUSED) {
          tmem_st32(xt, pk);
          // dS^T row of this key: 64 queries = 128 bytes = eight 16-byte chunks, chunk c stored at
          // c ^ (row & 7) (the 128-byte swizzle both MMA descriptors expect).  Buffer t was last read
          // by the products of step it-2, which ran before this step's S^T was issued.
          const uint32_t row_addr = sDS0 + t * C::DS_TILE + tid * 128;
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8)
            tc::sts128(row_addr + ((c8 ^ (tid & 7)) << 4),
                       make_uint4(dk[c8 * 4], dk[c8 * 4 + 1], dk[c8 * 4 + 2], dk[c8 * 4 + 3]));
          fence_proxy_async_smem();
        } else if (MODE == MODE_DKV) {
          tmem_st32(xt, pk);
          tmem_st32(yt, dk);
        } else {
          // dS buffer t was last read by the accumulate MMAs of step it-2
          if (it >= 2 && !mbar_wait(&bars->acc_done[t], ((it >> 1) - 1) & 1, abort_flag)) { alive = false; break; }
          tmem_st32(tmem + lane_base + (t ? C::COL_DS1 : C::COL_DS0), dk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&bars->p_full[t]);
        if (FUSED) {
          // the previous step's dQ^T tile is complete (or about to be): add it to the accumulator
          if (pend_it >= 0 && !drain_dq(pend_it, pend_rows, pend_valid)) { alive = false; break; }
          pend_it = it;
          pend_rows = args.dq_acc + (((int64_t)b * p.H_q + h) * p.N_q + r0) * D + tid;
          pend_valid = min(BT, p.N_q - r0);
        }
      }
    }

    // ---------------- epilogue ----------------
    if (alive && total_steps > 0) {
      const int last = it0 + total_steps - 1;
      alive = mbar_wait(&bars->acc_done[last & 1], (last >> 1) & 1, abort_flag);
      tc_fence_after_sync();
    }
    if (FUSED && alive && pend_it >= 0) {
      // the item's last dQ^T tile first: the next item's first step needs the buffer
      alive = drain_dq(pend_it, pend_rows, pend_valid);
      pend_it = -1;
    }
    if (alive) {
      const int n_rows = KVS ? p.N_kv : p.N_q;
      const bool store = srow < n_rows;
      // gradient of the stationary operand that carries the scale (dK or dQ), with the rotation undone
      {
        const uint32_t acc = tmem + lane_base + (KVS ? C::COL_ACC2 : C::COL_ACC1);
        T* dst = KVS
                     ? reinterpret_cast<T*>(a.dk) + (int64_t)b * a.dk_stride[0] + (int64_t)h_kv * a.dk_stride[1] + (int64_t)srow * a.dk_stride[2]
                     : reinterpret_cast<T*>(a.dq) + (int64_t)b * a.dq_stride[0] + (int64_t)hx * a.dq_stride[1] + (int64_t)srow * a.dq_stride[2];
        const T* cos_row = ROPE ? reinterpret_cast<const T*>(p.cos) + (int64_t)srow * p.rope_stride_n : nullptr;
        const T* sin_row = ROPE ? reinterpret_cast<const T*>(p.sin) + (int64_t)srow * p.rope_stride_n : nullptr;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          // columns [32c, 32c+32) and their partners [32c + D/2, ...)
          uint32_t lo[32], hi[32];
          if (total_steps > 0) {
            tmem_ld32(acc + c * 32, lo);
            tmem_ld32(acc + D / 2 + c * 32, hi);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) lo[i] = hi[i] = 0u;
          }
          if (store) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              float gl[8], gh[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                gl[i] = __uint_as_float(lo[q4 * 8 + i]) * p.sm_scale;
                gh[i] = __uint_as_float(hi[q4 * 8 + i]) * p.sm_scale;
              }
              if (ROPE) {
                const int d0 = c * 32 + q4 * 8;
                const uint4 cl = __ldg(reinterpret_cast<const uint4*>(cos_row + d0));
                const uint4 ch = __ldg(reinterpret_cast<const uint4*>(cos_row + D / 2 + d0));
                const uint4 sl = __ldg(reinterpret_cast<const uint4*>(sin_row + d0));
                const uint4 sh = __ldg(reinterpret_cast<const uint4*>(sin_row + D / 2 + d0));
                const uint32_t clw[4] = {cl.x, cl.y, cl.z, cl.w}, chw[4] = {ch.x, ch.y, ch.z, ch.w};
                const uint32_t slw[4] = {sl.x, sl.y, sl.z, sl.w}, shw[4] = {sh.x, sh.y, sh.z, sh.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 c1 = Pack2<T>::unpack(clw[i]), c2 = Pack2<T>::unpack(chw[i]);
                  const float2 s1 = Pack2<T>::unpack(slw[i]), s2 = Pack2<T>::unpack(shw[i]);
                  const float a0 = gl[2 * i], a1 = gl[2 * i + 1], b0 = gh[2 * i], b1 = gh[2 * i + 1];
                  // transpose of the rotation: g[d] = g'[d] cos[d] + g'[d+h] sin[d+h]; g[d+h] = g'[d+h] cos[d+h] - g'[d] sin[d]
                  gl[2 * i] = a0 * c1.x + b0 * s2.x;     gl[2 * i + 1] = a1 * c1.y + b1 * s2.y;
                  gh[2 * i] = b0 * c2.x - a0 * s1.x;     gh[2 * i + 1] = b1 * c2.y - a1 * s1.y;
                }
              }
              uint4 vl, vh;
              vl.x = Pack2<T>::run(gl[0], gl[1]); vl.y = Pack2<T>::run(gl[2], gl[3]);
              vl.z = Pack2<T>::run(gl[4], gl[5]); vl.w = Pack2<T>::run(gl[6], gl[7]);
              vh.x = Pack2<T>::run(gh[0], gh[1]); vh.y = Pack2<T>::run(gh[2], gh[3]);
              vh.z = Pack2<T>::run(gh[4], gh[5]); vh.w = Pack2<T>::run(gh[6], gh[7]);
              *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = vl;
              *reinterpret_cast<uint4*>(dst + D / 2 + c * 32 + q4 * 8) = vh;
            }
          }
        }
      }
      if (KVS) {
        T* dst = reinterpret_cast<T*>(a.dv) + (int64_t)b * a.dv_stride[0] + (int64_t)h_kv * a.dv_stride[1] + (int64_t)srow * a.dv_stride[2];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          if (total_steps > 0) {
            tmem_ld32(tmem + lane_base + C::COL_ACC1 + c * 32, o);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0u;
          }
          if (store) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 v;
              v.x = Pack2<T>::run(__uint_as_float(o[q4 * 8 + 0]), __uint_as_float(o[q4 * 8 + 1]));
              v.y = Pack2<T>::run(__uint_as_float(o[q4 * 8 + 2]), __uint_as_float(o[q4 * 8 + 3]));
              v.z = Pack2<T>::run(__uint_as_float(o[q4 * 8 + 4]), __uint_as_float(o[q4 * 8 + 5]));
              v.w = Pack2<T>::run(__uint_as_float(o[q4 * 8 + 6]), __uint_as_float(o[q4 * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = v;
            }
          }
        }
      }
    }
    if (alive && total_steps > 0) {
      // accumulators read out: the next item's first accumulation may overwrite them
      tc_fence_before_sync();
      mbar_arrive(&bars->acc_free);
      it0 += total_steps;
    }
    }  // items
  }

  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag && p.status != nullptr) atomicExch(p.status, AF_STATUS_WAIT_TIMEOUT);
  if (warp == 4) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

template <typename T, int D, int MODE, int EMASK, bool ALIBI, bool ROPE>
int launch_instance(const BwdArgs& args, const CUtensorMap& a1, const CUtensorMap& a2, const CUtensorMap& b1,
                    const CUtensorMap& b2, cudaStream_t st) {
  auto kern = bwd_tcgen05_kernel<T, D, MODE, EMASK, ALIBI, ROPE>;
  constexpr int smem = BCfg<D, MODE>::SMEM_BYTES;
  static bool configured = false;
  if (!configured) {
    AF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  if (args.total_items <= 0) return AF_OK;
  kern<<<(unsigned)args.grid_ctas, 224, smem, st>>>(args, a1, a2, b1, b2);
  count_launch();
  return check_cuda(cudaGetLastError(), "bwd_tcgen05 launch");
}

template <typename T, int D, int MODE>
int launch_composition(const BwdArgs& args, const CUtensorMap& a1, const CUtensorMap& a2, const CUtensorMap& b1,
                       const CUtensorMap& b2, cudaStream_t st) {
  const AfProblem& p = args.a.p;
  const int key = (p.mask_kind == AF_MASK_CAUSAL ? 4 : p.mask_kind == AF_MASK_WINDOW ? 8 : 0) +
                  (p.bias_kind == AF_BIAS_ALIBI ? 2 : 0) + (p.rope ? 1 : 0);
  if (p.mask_kind == AF_MASK_BLOCKS && p.kv_slot != nullptr && p.q_slot != nullptr) {
    // block lists with element bit matrices (never with rotation: the block-sparse call has none)
    if (p.rope) return fail(AF_ERR_UNSUPPORTED, "block lists with element bit matrices take no rotation");
    return p.bias_kind == AF_BIAS_ALIBI ? launch_instance<T, D, MODE, EMASK_BITS, true, false>(args, a1, a2, b1, b2, st)
                                        : launch_instance<T, D, MODE, EMASK_BITS, false, false>(args, a1, a2, b1, b2, st);
  }
  switch (key) {
    case 8: return launch_instance<T, D, MODE, EMASK_WINDOW, false, false>(args, a1, a2, b1, b2, st);
    case 9: return launch_instance<T, D, MODE, EMASK_WINDOW, false, true>(args, a1, a2, b1, b2, st);
    case 10: return launch_instance<T, D, MODE, EMASK_WINDOW, true, false>(args, a1, a2, b1, b2, st);
    case 11: return launch_instance<T, D, MODE, EMASK_WINDOW, true, true>(args, a1, a2, b1, b2, st);
    case 0: return launch_instance<T, D, MODE, EMASK_NONE, false, false>(args, a1, a2, b1, b2, st);
    case 1: return launch_instance<T, D, MODE, EMASK_NONE, false, true>(args, a1, a2, b1, b2, st);
    case 2: return launch_instance<T, D, MODE, EMASK_NONE, true, false>(args, a1, a2, b1, b2, st);
    case 3: return launch_instance<T, D, MODE, EMASK_NONE, true, true>(args, a1, a2, b1, b2, st);
    case 4: return launch_instance<T, D, MODE, EMASK_CAUSAL, false, false>(args, a1, a2, b1, b2, st);
    case 5: return launch_instance<T, D, MODE, EMASK_CAUSAL, false, true>(args, a1, a2, b1, b2, st);
    case 6: return launch_instance<T, D, MODE, EMASK_CAUSAL, true, false>(args, a1, a2, b1, b2, st);
    default: return launch_instance<T, D, MODE, EMASK_CAUSAL, true, true>(args, a1, a2, b1, b2, st);
  }
}

int launch_dkv_d64(int dtype, const BwdArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);
int launch_dkv_d128(int dtype, const BwdArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);
int launch_dq_d64(int dtype, const BwdArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);
int launch_dq_d128(int dtype, const BwdArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);
int launch_fused_d128(int dtype, const BwdArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, cudaStream_t);

#define AF_DEFINE_BWD_UNIT(NAME, DIM, MODE)                                                                   \
  int NAME(int dtype, const BwdArgs& args, const CUtensorMap& a1, const CUtensorMap& a2, const CUtensorMap& b1, \
           const CUtensorMap& b2, cudaStream_t st) {                                                          \
    if (dtype == AF_F16) return launch_composition<__half, DIM, MODE>(args, a1, a2, b1, b2, st);              \
    return launch_composition<__nv_bfloat16, DIM, MODE>(args, a1, a2, b1, b2, st);                            \
  }

}  // namespace tcb
}  // namespace af
