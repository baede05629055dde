// Forward attention for two query heads of one KV group per CTA (head dim 128, GQA groups of even
// size, masks none / causal / window, ALiBi, operands already rotated when the graph has RoPE).
//
// Same arithmetic as fwd_tcgen05.cuh (reference: attnfuse/compiler/codegen.py:67-381) on another
// schedule.  A work item is 128 query rows of TWO adjacent query heads that share a KV head; the
// item's K and V tiles are loaded once and feed two S products and two P.V products.  Each head
// ("slot") has an S buffer and an O accumulator of its own in TMEM (2 x 128 + 2 x 128 columns)
// and a softmax group of its own -- four warps, one thread per query row -- so nothing ties the
// two slots together but the K / V tiles: slot q's next S product waits only for slot q's own
// P.V product.  The two warps that share a scheduler belong to different slots, and while one
// waits for its tensor-core chain (P.V, then S of the next tile) the other runs its exponent pass.
//
// A thread walks its row's 128 key columns of a tile as two chunks of 64 -- the online-softmax
// step of fwd_tcgen05.cuh, with P of a chunk written over the chunk's own S columns and handed
// to the MMA thread on its own, so the P.V product of the first chunk runs under the exponent
// pass of the second.
//
// Roles (384 threads): warps 0-3 softmax of slot 0, warps 4-7 softmax of slot 1, warp 8 TMA
// producer (Q of both heads per item, K ring and V ring of two stages each), one thread each of
// warps 9 and 11 issues S_0 / S_1 = Q_q K^T, one thread of warp 10 issues O_q += P_q V.  Every
// wait is bounded.
#pragma once
#include "fwd_tcgen05.cuh"

namespace af {
namespace tc {

struct PairCfg {
  static constexpr int D = 128;
  static constexpr int TILE_BYTES = 2 * PANEL_BYTES;          // 128 rows x 128 elements x 2 bytes
  static constexpr int STAGES = 2;                            // K ring and V ring
  static constexpr int O_STAGE_BYTES = 8 * 32 * 128;          // per softmax warp: 32 rows x 64 columns
  static constexpr int SMEM_BYTES = TILE_BYTES * (2 + 2 * STAGES) + O_STAGE_BYTES + 1024 /*align*/ + 512 /*barriers*/;
  static constexpr int TMEM_COLS = 512;
  __host__ __device__ static constexpr int col_s(int q) { return q * 128; }
  __host__ __device__ static constexpr int col_o(int q) { return 256 + q * 128; }
};

struct PairBarriers {
  uint64_t q_full, q_empty;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2][2];     // [slot][chunk]: the chunk's 64 columns of S_q are in TMEM
  uint64_t p_full[2][2];     // [slot][chunk]: P of the chunk is in TMEM
  uint64_t pv_done[2][2];    // [slot][chunk]: the chunk's P.V product has run
  uint64_t o_free[2];        // [slot]: the item's accumulator has been read out
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(PairBarriers) <= 512, "PairCfg::SMEM_BYTES reserves 512 bytes for the barriers");

// Item w of the pair schedule: the order of get_item with head pairs as units; args.div_hq /
// div_group divide by H_q / 2 and (H_q / H_kv) / 2, and it.h is the first head of the pair.
template <int EMASK>
__device__ __forceinline__ bool get_pair_item(const TcArgs& args, int round, Item& it) {
  const int G = (int)gridDim.x, c = (int)blockIdx.x;
  const int64_t w64 = (int64_t)round * G + ((round & 1) ? G - 1 - c : c);
  if (w64 >= args.total_items) return false;
  const int w = (int)w64;
  const AfProblem& p = args.a.p;
  const int pairs = p.H_q >> 1;
  int w_over_bp, bp;
  split_item(args, w, args.num_m_blocks, w_over_bp, bp);
  it.b = args.div_hq.div(bp);
  const int pr = bp - it.b * pairs;
  it.h = pr * 2;
  it.h_kv = args.div_group.div(pr);
  it.split = 0;
  it.n_kv = p.N_kv;
  const int m_blk = (EMASK == EMASK_CAUSAL) ? (args.num_m_blocks - 1 - w_over_bp) : w_over_bp;
  it.m0 = m_blk * BM;
  it.walk = make_walk(p, args, m_blk, it.h);
  return true;
}

template <int EMASK>
__device__ __forceinline__ bool pair_cursor_next(const TcArgs& args, TileCursor& c) {
  if (c.j + 1 < c.it.walk.n_tiles) { ++c.j; ++c.gg; return true; }
  for (;;) {
    ++c.round;
    if (!get_pair_item<EMASK>(args, c.round, c.it)) return false;
    if (c.it.walk.n_tiles > 0) { c.j = 0; ++c.gg; ++c.qi; return true; }
  }
}

template <typename T, int EMASK, bool ALIBI>
__global__ void __launch_bounds__(384, 1)
fwd_pair_kernel(const TcArgs args, const __grid_constant__ CUtensorMap tmap_q,
                const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                const __grid_constant__ CUtensorMap tmap_o) {
  using C = PairCfg;
  constexpr int D = C::D;
  constexpr int AB_FMT = (Elem<T>::code == AF_BF16) ? 1 : 0;
  constexpr uint32_t IDESC_QK = umma_idesc_f16(AB_FMT, BM, 64, 0, 0);   // one chunk of 64 key columns
  constexpr uint32_t IDESC_PV = umma_idesc_f16(AB_FMT, BM, D, 0, 1);

  const AfFwdParams& a = args.a;
  const AfProblem& p = a.p;

  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base;                                   // Q of slot 0, then of slot 1
  const uint32_t sK0 = sQ + 2 * C::TILE_BYTES;
  const uint32_t sV0 = sK0 + C::STAGES * C::TILE_BYTES;
  const uint32_t sO = sV0 + C::STAGES * C::TILE_BYTES;
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(smem + C::TILE_BYTES * (2 + 2 * C::STAGES) + C::O_STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_empty, 2);      // one S-issuing thread per slot
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 2);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(&bars->o_free[q], BM);
      for (int c = 0; c < 2; ++c) {
        mbar_init(&bars->s_full[q][c], 1);
        mbar_init(&bars->p_full[q][c], BM);
        mbar_init(&bars->pv_done[q][c], 1);
      }
    }
    bars->abort_flag = 0;
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

  // Running counts as in fwd_tcgen05.cuh: gg = key tiles so far (ring stage gg & 1, ring phase
  // (gg >> 1) & 1; the per-slot barriers complete once per tile, phase gg & 1), qi = items so far.
  if (warp == WARP_PRODUCER) {
    // ============================== TMA producer ==============================
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      tma_prefetch_desc(&tmap_o);
      const uint64_t keep = l2_policy_evict_last(), stream = l2_policy_evict_first();
      TileCursor ck, cv;   // K runs one tile ahead of V
      cursor_init(ck);
      cursor_init(cv);
      auto load_k = [&]() -> bool {
        if (ck.j == 0) {
          // both Q buffers are free once the last S product of the previous item has run
          if (ck.qi > 0 && !mbar_wait(&bars->q_empty, (ck.qi - 1) & 1, abort_flag)) return false;
          mbar_arrive_expect_tx(&bars->q_full, 2 * C::TILE_BYTES);
#pragma unroll
          for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int pn = 0; pn < 2; ++pn)
              tma_load_4d_hint(smem + q * C::TILE_BYTES + pn * PANEL_BYTES, &tmap_q, &bars->q_full, pn * 64, ck.it.m0,
                               ck.it.h + q, ck.it.b, stream);
        }
        const int s = ck.gg & 1;
        if (ck.gg >= 2 && !mbar_wait(&bars->k_empty[s], ((ck.gg >> 1) & 1) ^ 1, abort_flag)) return false;
        mbar_arrive_expect_tx(&bars->k_full[s], C::TILE_BYTES);
        const int key0 = ck.it.walk.key0(ck.j);
        unsigned char* dk = smem + C::TILE_BYTES * (2 + s);
#pragma unroll
        for (int pn = 0; pn < 2; ++pn)
          tma_load_4d_hint(dk + pn * PANEL_BYTES, &tmap_k, &bars->k_full[s], pn * 64, key0, ck.it.h_kv, ck.it.b, keep);
        return true;
      };
      auto load_v = [&]() -> bool {
        const int s = cv.gg & 1;
        if (cv.gg >= 2 && !mbar_wait(&bars->v_empty[s], ((cv.gg >> 1) & 1) ^ 1, abort_flag)) return false;
        mbar_arrive_expect_tx(&bars->v_full[s], C::TILE_BYTES);
        const int key0 = cv.it.walk.key0(cv.j);
        unsigned char* dv = smem + C::TILE_BYTES * (2 + C::STAGES + s);
#pragma unroll
        for (int pn = 0; pn < 2; ++pn)
          tma_load_4d_hint(dv + pn * PANEL_BYTES, &tmap_v, &bars->v_full[s], pn * 64, key0, cv.it.h_kv, cv.it.b, keep);
        return true;
      };
      bool more_k = pair_cursor_next<EMASK>(args, ck);
      bool more_v = pair_cursor_next<EMASK>(args, cv);
      // K runs one tile ahead of V (a wait for a V slot never holds up a K load) -- except across
      // an item boundary: the first K load of an item starts with a wait for the Q buffers (the
      // previous item's last S product), so every V tile of the previous item goes out before it.
      while (more_k || more_v) {
        const bool at_boundary = more_k && ck.j == 0 && ck.qi > 0 && more_v && cv.gg < ck.gg;
        if (more_k && !at_boundary && (!more_v || ck.gg <= cv.gg + 1)) {
          if (!load_k()) break;
          more_k = pair_cursor_next<EMASK>(args, ck);
        } else {
          if (!load_v()) break;
          more_v = pair_cursor_next<EMASK>(args, cv);
        }
      }
    }
  } else if (warp == WARP_QK || warp == WARP_ROTATE) {
    // ============================== MMA issuers 1a / 1b: S_q = Q_q K^T ==============================
    // One issuing thread per slot, in warps of different schedulers: the issuing threads take
    // issue slots from the softmax warps they share a scheduler with, and the slowest of a slot's
    // four softmax warps sets the slot's pace.
    if (lane == 0) {
      const int q = (warp == WARP_QK) ? 0 : 1;
      const uint64_t qdesc = umma_desc_sw128(sQ + q * C::TILE_BYTES, 16, 1024);
      const uint64_t desc_k0 = umma_desc_sw128(sK0, 16, 1024);
      TileCursor cu;
      cursor_init(cu);
      bool ok = true;
      while (ok && pair_cursor_next<EMASK>(args, cu)) {
        const int gg = cu.gg, s = gg & 1;
        if (cu.j == 0 && !mbar_wait(&bars->q_full, cu.qi & 1, abort_flag)) break;
        if (!mbar_wait(&bars->k_full[s], (gg >> 1) & 1, abort_flag)) break;
        const uint64_t kdesc = desc_k0 + (uint64_t)((s * C::TILE_BYTES) >> 4);
        for (int c = 0; c < 2 && ok; ++c) {
          // One product per chunk of 64 key columns (rows 64 c .. 64 c + 63 of the K tile): the
          // chunk's S columns hold P of the previous tile's chunk until its P.V product has run,
          // so the first chunk of the next tile is under way while the softmax group is still
          // in the second chunk of this one.
          if (gg >= 1 && !mbar_wait(&bars->pv_done[q][c], (gg - 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem + C::col_s(q) + c * 64;
          const uint64_t kh = kdesc + (uint64_t)((c * 64 * 128) >> 4);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t off = (uint64_t)(((kk >> 2) * PANEL_BYTES + (kk & 3) * 32) >> 4);
            umma_ss(d_tmem, qdesc + off, kh + off, IDESC_QK, kk > 0 ? 1u : 0u);
          }
          umma_commit(&bars->s_full[q][c]);
        }
        if (!ok) break;
        umma_commit(&bars->k_empty[s]);        // both slots' products have to be through before the stage is refilled
        if (cu.j + 1 == cu.it.walk.n_tiles) umma_commit(&bars->q_empty);
      }
    }
  } else if (warp == WARP_PV) {
    // ============================== MMA issuer 2: O_q += P_q V ==============================
    if (lane == 0) {
      const uint64_t desc_v0 = umma_desc_sw128(sV0, PANEL_BYTES, 1024);
      TileCursor cu;
      cursor_init(cu);
      bool ok = true;
      while (ok && pair_cursor_next<EMASK>(args, cu)) {
        const int gg = cu.gg, s = gg & 1;
        if (!mbar_wait(&bars->v_full[s], (gg >> 1) & 1, abort_flag)) break;
        const uint64_t vdesc = desc_v0 + (uint64_t)((s * C::TILE_BYTES) >> 4);
        for (int q = 0; q < 2 && ok; ++q) {
          for (int c = 0; c < 2 && ok; ++c) {
            if (!mbar_wait(&bars->p_full[q][c], gg & 1, abort_flag)) { ok = false; break; }
            // the item's first product overwrites O_q: the previous item's rows must be read out
            if (cu.j == 0 && c == 0 && cu.qi > 0 && !mbar_wait(&bars->o_free[q], (cu.qi - 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t p_tmem = tmem + C::col_s(q) + c * 64;   // P of a chunk sits in the first 32 of its 64 S columns
            const uint32_t o_tmem = tmem + C::col_o(q);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_ts(o_tmem, p_tmem + kk * 8, vdesc + (uint64_t)(((c * 4 + kk) * 2048) >> 4), IDESC_PV,
                      (cu.j > 0 || c > 0 || kk > 0) ? 1u : 0u);
            umma_commit(&bars->pv_done[q][c]);
          }
        }
        if (!ok) break;
        umma_commit(&bars->v_empty[s]);
      }
    }
  } else if (warp < 8) {
    // ============================== softmax / epilogue ==============================
    // One thread per query row of its slot; the row's online softmax runs over chunks of 64 key
    // columns with the standing-reference fast path of fwd_tcgen05.cuh (no maximum pass while the
    // row sum stays below kRowSumBound; otherwise maximum, reference update, accumulator rescale).
    const int q = warp >> 2, rtid = tid & (BM - 1);
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem + lane_base + C::col_s(q);
    const uint32_t o_tmem = tmem + lane_base + C::col_o(q);
    const float scale2 = p.sm_scale * kLog2e;     // > 0 (checked on the host)
    Item it, it_next;
    int g = 0;
    bool alive = true;
    bool have = get_pair_item<EMASK>(args, 0, it);
    for (int round = 0; alive && have; ++round) {
      const TileWalk& walk = it.walk;
      const int n_tiles = walk.n_tiles;
      const int m0 = it.m0, b = it.b, h = it.h + q;
      const int row = m0 + rtid;
      const float slope2 = ALIBI ? load_slope<T>(p.slopes, h) * kLog2e : 0.f;
      float m_ref = -INFINITY, l_row = 0.f;         // m_ref in log2 units of the scaled score
      bool ref_ok = false;   // warp-uniform: every row of the warp has a finite reference (it never becomes -inf again)

      for (int j = 0; j < n_tiles; ++j) {
        const int gg = g + j;
        const int key0 = walk.key0(j);
        const int pos0 = m0 + p.q_offset;           // position of the tile's first row on the key axis
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          if (!mbar_wait(&bars->s_full[q][c], gg & 1, abort_flag)) { alive = false; break; }
          tc_fence_after_sync();
          uint32_t xr[64];   // fp32 bit patterns of this thread's raw scores of the chunk
          tmem_ld32(s_tmem + c * 64, &xr[0]);
          tmem_ld32(s_tmem + c * 64 + 32, &xr[32]);
          tmem_wait_ld();
          const int col0 = key0 + c * 64;           // key index of the chunk's column 0
          // Chunk-level decision: only edge / diagonal chunks pay for element masking.
          bool need_mask = col0 + 64 > p.N_kv;
          if (EMASK == EMASK_CAUSAL) need_mask = need_mask || (col0 + 63 > pos0);
          if (EMASK == EMASK_WINDOW)
            need_mask = need_mask || (pos0 + BM - 1 - col0 >= p.window) || (col0 + 63 - pos0 >= p.window);
          const int rel = row + p.q_offset - col0;  // column x is kept iff ...
          if (need_mask) {
            const int kmax = p.N_kv - col0;         // ... x < kmax
#pragma unroll
            for (int x = 0; x < 64; ++x) {
              bool keep = x < kmax;
              if (EMASK == EMASK_CAUSAL) keep = keep && (x <= rel);
              if (EMASK == EMASK_WINDOW) keep = keep && (x - rel < p.window) && (rel - x < p.window);
              xr[x] = keep ? xr[x] : 0xff800000u;   // -inf
            }
          }
          float slope_c = 0.f, bias0 = 0.f;
          bool affine = true;
          if (ALIBI) {
            const bool below = (EMASK == EMASK_CAUSAL) || rel >= 63;
            affine = (EMASK == EMASK_CAUSAL) || __all_sync(0xffffffffu, below || rel <= 0);
            slope_c = below ? slope2 : -slope2;
            bias0 = -slope_c * (float)rel;
          }
          float alpha = 1.f, rsum = 0.f;
          uint32_t pk[32];
          bool fast = ref_ok && affine;
          if (fast) {
            exp_pass<T, ALIBI ? EXP_AFFINE : EXP_SCALE>(xr, pk, scale2, bias0 - m_ref, slope_c, rsum);
            fast = __all_sync(0xffffffffu, rsum <= kRowSumBound);
          }
          if (!fast) {
            if (ALIBI) {
              const float relf = (float)rel;
#pragma unroll
              for (int x = 0; x < 64; ++x)
                xr[x] = __float_as_uint(fmaf(__uint_as_float(xr[x]), scale2, -slope2 * fabsf(relf - (float)x)));
            }
            float mx = row_max(xr);
            if (!ALIBI) mx *= scale2;
            const bool bump = mx > m_ref + kRescaleThreshold;   // also true for the first finite max
            const float m_next = bump ? mx : m_ref;
            alpha = bump ? ex2_approx(m_ref - m_next) : 1.f;
            m_ref = m_next;
            ref_ok = __all_sync(0xffffffffu, m_ref != -INFINITY);
            const float neg_m = (m_next == -INFINITY) ? 0.f : -m_next;
            if ((j > 0 || c > 0) && __any_sync(0xffffffffu, bump)) {
              // The accumulator is expressed relative to the old reference: rescale it in TMEM once
              // the previous chunk's P.V product has landed.
              const bool prev_ok = (c == 1) ? mbar_wait(&bars->pv_done[q][0], gg & 1, abort_flag)
                                            : mbar_wait(&bars->pv_done[q][1], (gg - 1) & 1, abort_flag);
              if (!prev_ok) { alive = false; break; }
              tc_fence_after_sync();
#pragma unroll
              for (int cc = 0; cc < D / 32; ++cc) {
                uint32_t o[32];
                tmem_ld32(o_tmem + cc * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st32(o_tmem + cc * 32, o);
              }
              tmem_wait_st();
            }
            exp_pass<T, ALIBI ? EXP_PRESCALED : EXP_SCALE>(xr, pk, scale2, neg_m, 0.f, rsum);
          }
          l_row = l_row * alpha + rsum;
          tmem_st32(s_tmem + c * 64, pk);           // P of the chunk over the first half of its own S columns
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(&bars->p_full[q][c]);
        }
        if (!alive) break;
      }

      // Epilogue: O = O_q / l, L = m + log(l); the rows leave through shared memory and a TMA
      // store, 64 columns at a time (the warp's staging region holds 32 rows x 128 bytes).
      if (!alive) break;
      // the next item is decoded here, under the wait for the last P.V product
      const bool have_next = get_pair_item<EMASK>(args, round + 1, it_next);
      if (n_tiles > 0) {
        const int gl = g + n_tiles - 1;
        if (!mbar_wait(&bars->pv_done[q][1], gl & 1, abort_flag)) { alive = false; break; }
        tc_fence_after_sync();
      }
      const float safe_l = (l_row == 0.f) ? 1.f : l_row;
      const float inv = 1.f / safe_l;
      const uint32_t stage = sO + (uint32_t)(warp * 32 * 128);
      const int row0 = m0 + (warp & 3) * 32;
      uint32_t o[D];
      if (n_tiles > 0) {
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) tmem_ld32(o_tmem + cc * 32, &o[cc * 32]);
        tmem_wait_ld();
        tc_fence_before_sync();
        mbar_arrive(&bars->o_free[q]);   // the next item's first P.V product may overwrite O_q
      } else {
        // no key tile in reach of these rows: zeros, and no hand-over (the MMA threads skip the item)
#pragma unroll
        for (int i = 0; i < D; ++i) o[i] = 0u;
      }
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        if (lane == 0) bulk_wait_read_all();   // the region's previous store has read it
        __syncwarp();
#pragma unroll
        for (int q8 = 0; q8 < 8; ++q8) {
          const int i0 = c2 * 64 + q8 * 8;
          uint4 v;
          v.x = Pack2<T>::run(__uint_as_float(o[i0 + 0]) * inv, __uint_as_float(o[i0 + 1]) * inv);
          v.y = Pack2<T>::run(__uint_as_float(o[i0 + 2]) * inv, __uint_as_float(o[i0 + 3]) * inv);
          v.z = Pack2<T>::run(__uint_as_float(o[i0 + 4]) * inv, __uint_as_float(o[i0 + 5]) * inv);
          v.w = Pack2<T>::run(__uint_as_float(o[i0 + 6]) * inv, __uint_as_float(o[i0 + 7]) * inv);
          sts128(stage + (uint32_t)(lane * 128 + ((q8 ^ (lane & 7)) << 4)), v);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row0 < p.N_q) {
          tma_store_4d_hint(&tmap_o, stage, c2 * 64, row0, h, b, l2_policy_evict_first());
          bulk_commit_group();
        }
      }
      if (a.lse != nullptr && row < p.N_q)
        a.lse[(int64_t)b * a.lse_stride[0] + (int64_t)h * a.lse_stride[1] + (int64_t)row * a.lse_stride[2]] =
            m_ref * kLn2 + logf(safe_l);
      g += n_tiles;
      it = it_next;
      have = have_next;
    }
    if (lane == 0) bulk_wait_all();   // the staged rows must have left shared memory before the CTA exits
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

template <typename T, int EMASK, bool ALIBI>
int launch_pair_instance(const TcArgs& args, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                         const CUtensorMap& mo, cudaStream_t st) {
  auto kern = fwd_pair_kernel<T, EMASK, ALIBI>;
  constexpr int smem = PairCfg::SMEM_BYTES;
  static bool configured = false;   // benign race: the attribute call is idempotent
  if (!configured) {
    AF_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  kern<<<(unsigned)args.grid_ctas, 384, smem, st>>>(args, mq, mk, mv, mo);
  count_launch();
  return check_cuda(cudaGetLastError(), "fwd_pair launch");
}

template <typename T>
int launch_pair_composition(const TcArgs& args, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                            const CUtensorMap& mo, cudaStream_t st) {
  const AfProblem& p = args.a.p;
  const int em = p.mask_kind == AF_MASK_CAUSAL ? EMASK_CAUSAL : p.mask_kind == AF_MASK_WINDOW ? EMASK_WINDOW : EMASK_NONE;
  const bool alibi = p.bias_kind == AF_BIAS_ALIBI;
  switch (em * 2 + (alibi ? 1 : 0)) {
    case 0: return launch_pair_instance<T, EMASK_NONE, false>(args, mq, mk, mv, mo, st);
    case 1: return launch_pair_instance<T, EMASK_NONE, true>(args, mq, mk, mv, mo, st);
    case 2: return launch_pair_instance<T, EMASK_CAUSAL, false>(args, mq, mk, mv, mo, st);
    case 3: return launch_pair_instance<T, EMASK_CAUSAL, true>(args, mq, mk, mv, mo, st);
    case 4: return launch_pair_instance<T, EMASK_WINDOW, false>(args, mq, mk, mv, mo, st);
    default: return launch_pair_instance<T, EMASK_WINDOW, true>(args, mq, mk, mv, mo, st);
  }
}

// Entry point of the instantiation unit: dtype is AF_F16 / AF_BF16.
int launch_pair_d128(int dtype, const TcArgs&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                     const CUtensorMap&, cudaStream_t);

}  // namespace tc
}  // namespace af
