/*
 * attnfuse_b200.h -- C ABI of the sm_100a fused-attention library.
 *
 * The reference project has no native layer: its launch boundary is a set of Python
 * functions that pass raw pointers, element strides and scalar flags to Triton kernels.
 * Each entry point below replaces one of those launch sites; the comment above it names
 * the reference function (path within the reference project : line) whose launch it
 * stands in for.  All pointers are device pointers unless stated otherwise, all strides
 * are in ELEMENTS (as in the reference's launches), every call is asynchronous on the
 * given stream, and nothing here allocates or frees device memory unless stated.
 *
 * Return value: 0 on success; a negative AF_ERR_* code otherwise, with a human readable
 * message available from af_last_error() (thread local).
 */
#ifndef ATTNFUSE_B200_H_
#define ATTNFUSE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AF_ABI_VERSION 4

#if defined(__GNUC__)
#define AF_API __attribute__((visibility("default")))
#else
#define AF_API
#endif

typedef void* af_stream_t; /* a cudaStream_t */

enum { AF_F16 = 0, AF_BF16 = 1, AF_F32 = 2 };
/* MASK/BIAS/NORM codes are the reference's constexpr encodings
 * (attnfuse/compiler/codegen.py:17-57), plus AF_MASK_BLOCKS for block lists. */
enum { AF_MASK_FULL = 0, AF_MASK_CAUSAL = 1, AF_MASK_WINDOW = 2, AF_MASK_BLOCKS = 3 };
enum { AF_BIAS_NONE = 0, AF_BIAS_ALIBI = 1, AF_BIAS_ADDITIVE = 2 };
enum { AF_NORM_SOFTMAX = 0, AF_NORM_RELU = 1 };
/* Kernel family: AUTO picks tcgen05 for f16/bf16 with D in {64,128} and softmax. */
enum { AF_FAMILY_AUTO = 0, AF_FAMILY_FFMA = 1, AF_FAMILY_TCGEN05 = 2 };

enum {
  AF_OK = 0,
  AF_ERR_INVALID = -1,     /* bad argument (shape, stride, alignment, enum)            */
  AF_ERR_UNSUPPORTED = -2, /* composition has no kernel instantiation                  */
  AF_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed                      */
  AF_ERR_WORKSPACE = -4    /* caller-provided workspace too small                      */
};

/* Device status word values written by kernels whose bounded waits ran out. */
enum { AF_STATUS_OK = 0, AF_STATUS_WAIT_TIMEOUT = 1 };

/* One attention problem: shapes, composition flags and the read-only operands.
 * Mirrors the argument list of the reference's forward launch
 * (attnfuse/runtime/dispatch.py:196-214). */
typedef struct AfProblem {
  int32_t dtype;      /* AF_F16 / AF_BF16 / AF_F32: type of q,k,v,o,slopes,bias,cos,sin    */
  int32_t family;     /* AF_FAMILY_*                                                       */
  int32_t B, H_q, H_kv, N_q, N_kv, D;
  float   sm_scale;
  int32_t mask_kind;  /* AF_MASK_*                                                          */
  int32_t window;     /* AF_MASK_WINDOW: keys with |i-j| < window are kept                  */
  int32_t bias_kind;  /* AF_BIAS_*                                                          */
  int32_t norm_kind;  /* AF_NORM_*                                                          */
  int32_t rope;       /* 1: rotate Q and K (rotate-half) inside the kernel                  */
  int32_t block_m, block_n; /* AF_MASK_BLOCKS: tile size the lists were built for          */
  const void* q; int64_t q_stride[4];   /* (B, H_q,  N_q,  D)                               */
  const void* k; int64_t k_stride[4];   /* (B, H_kv, N_kv, D)                               */
  const void* v; int64_t v_stride[4];   /* (B, H_kv, N_kv, D)                               */
  const void* slopes;                   /* [H_q], AF_BIAS_ALIBI                             */
  const void* bias; int64_t bias_stride[4]; /* (B, H_q, N_q, N_kv), AF_BIAS_ADDITIVE       */
  const void* cos; const void* sin; int64_t rope_stride_n; /* rows of D, inner stride 1    */
  /* Block lists (int32).  Query-major: kv_num[h][qb], kv_idx[h][qb][slot];
   * key-major (backward only): q_num[h][kb], q_idx[h][kb][slot].  A head stride of 0
   * shares one mask between all heads (the reference's BlockMask has no head axis:
   * attnfuse/runtime/block_mask.py:75-98). */
  const int32_t* kv_num; const int32_t* kv_idx;
  int64_t kv_num_stride_h, kv_idx_stride_h, kv_idx_stride_q;
  const int32_t* q_num; const int32_t* q_idx;
  int64_t q_num_stride_h, q_idx_stride_h, q_idx_stride_k;
  int32_t* status;    /* optional device word, AF_STATUS_*; may be NULL                     */
  int32_t q_offset;   /* position of query row 0 on the key axis (chunked prefill against a
                         cache): row i is masked, biased and rotated as position q_offset + i.
                         Forward only; no counterpart in the reference, whose kernels index
                         rows and columns from 0 (attnfuse/compiler/codegen.py:126-135,216-217)
                         and reject masks when N_q != N_kv (attnfuse/runtime/dispatch.py:140-148) */
  /* Element-exact partial tiles (optional; NULL: every listed tile is fully active, which is all
   * the reference can express because its builder rounds partial tiles up,
   * attnfuse/runtime/block_mask.py:143-154).  kv_slot is parallel to kv_idx (same strides) and
   * q_slot to q_idx: -1 = every element of the listed tile is active, s >= 0 = the tile's
   * elements are given by bit matrix s.  Both orientations of matrix s are stored:
   *   kv_bits[s][r][w] : row r = query within the tile, bit (c & 63) of word w = c >> 6 = key c,
   *                      words per row = ceil(block_n / 64)
   *   q_bits[s][c][w]  : row c = key within the tile, bit (r & 63) of word r >> 6 = query r,
   *                      words per row = ceil(block_m / 64)   (tensor-core backward only) */
  const int32_t* kv_slot; const int32_t* q_slot;
  const uint64_t* kv_bits; const uint64_t* q_bits;
} AfProblem;

typedef struct AfFwdParams {
  AfProblem p;
  void*   o;   int64_t o_stride[4];    /* (B, H_q, N_q, D), caller allocated               */
  float*  lse; int64_t lse_stride[3];  /* (B, H_q, N_q) fp32 log-sum-exp, or NULL          */
  void*   workspace;                   /* optional scratch, see af_fwd_workspace_bytes     */
  int64_t workspace_bytes;
} AfFwdParams;

typedef struct AfBwdParams {
  AfProblem p;
  const void*  o;   int64_t o_stride[4];
  const void*  d_o; int64_t do_stride[4];
  const float* lse; int64_t lse_stride[3];
  float* delta;                       /* scratch (B, H_q, N_q) fp32 contiguous: rowsum(dO*O) */
  void* dq; int64_t dq_stride[4];     /* like q                                            */
  void* dk; int64_t dk_stride[4];     /* like k (summed over the query-head group)         */
  void* dv; int64_t dv_stride[4];
  void*   workspace;                  /* optional scratch, see af_bwd_workspace_bytes      */
  int64_t workspace_bytes;
  int32_t workspace_holds_rotated;    /* 1: the workspace already holds the rotated Q and K of
                                         this problem, as af_fwd left them in its own workspace
                                         (same layout); the RoPE pre-pass is then skipped      */
  void*   dq_accum;                   /* optional scratch of af_bwd_dq_accum_bytes() bytes, 256-byte
                                         aligned: an fp32 (B, H_q, N_q, D) accumulator for dQ.  With
                                         it af_bwd runs the single-pass kernel (S and dP computed
                                         once, dQ summed over key tiles with fp32 atomic adds, so
                                         its last bits depend on scheduling); without it the
                                         deterministic two-pass kernels run                    */
  int64_t dq_accum_bytes;
} AfBwdParams;

/* Split-K decode (query length 1).  Workspaces are fp32:
 *   ws_m, ws_l : [num_splits, B, H_q]      ws_acc : [num_splits, B, H_q, D]
 * ws_acc must be 16-byte aligned (the kernels access its rows with 16-byte vectors); when the
 * three arrays are carved from one allocation, round the m and l parts up to 4 floats each.  */
typedef struct AfDecodeParams {
  int32_t dtype;
  int32_t B, H_q, H_kv, N_kv, D;
  float   sm_scale;
  int32_t bias_kind;            /* AF_BIAS_NONE or AF_BIAS_ALIBI                           */
  int32_t num_splits;
  const void* q; int64_t q_stride[4];
  const void* k; int64_t k_stride[4];
  const void* v; int64_t v_stride[4];
  const void* slopes;
  const int32_t* kv_lens;       /* optional [B]: valid keys per batch row (<= N_kv); the
                                   reference has a scalar N_KV only                       */
  const int32_t* q_positions;   /* optional [B]: global query position used by ALiBi;
                                   default kv_offset + (valid keys) - 1                    */
  int32_t kv_offset;            /* global position of local key 0 (KV-sharded decode)      */
  float* ws_m; float* ws_l; float* ws_acc;
  void*  o; int64_t o_stride[4];  /* (B, H_q, 1, D) final output, or NULL                 */
  float* partial;               /* optional [B, H_q, D+1] fp32: normalised O then LSE      */
  int32_t* status;
  /* The single query row of batch entry b sits at position q_pos[b] of the key axis:
   * q_positions[b] if given, else q_position_p1 - 1 if q_position_p1 > 0, else
   * kv_offset + (valid keys) - 1.
   * ALiBi measures its distance from there; AF_MASK_CAUSAL keeps keys at positions <= q_pos,
   * AF_MASK_WINDOW keys with |q_pos - position| < window; rope = 1 rotates the query at q_pos
   * and every key at its own position (rotate-half, tables as in AfProblem) before the dot;
   * rope = 2 rotates the query only: the cache holds keys that were rotated when they were
   * written (what a serving stack stores), and the step stays bandwidth-bound.
   * None of these exists in the reference, whose decode path takes dense and ALiBi graphs
   * only (attnfuse/runtime/flash_decode.py:46-65).  Zero-initialised fields give the
   * reference's behaviour. */
  int32_t mask_kind, window;
  int32_t rope;
  int32_t q_position_p1;        /* query position + 1; 0 = not given                        */
  const void* cos; const void* sin; int64_t rope_stride_n;
  /* Balanced scheduling: > 0 launches that many CTAs, each taking an equal share of the 64-key
   * tiles of all sequences laid end to end (one wave, equal work whatever the lengths), instead
   * of num_splits CTAs per (batch, kv head).  The workspaces then hold
   * (units + balanced_ctas) * min(group, 64) rows, units = B * H_kv * ceil(group / 64),
   * group = H_q / H_kv; num_splits is ignored.  The reference splits every sequence into the
   * same number of pieces (attnfuse/runtime/flash_decode.py:114-131). */
  int32_t balanced_ctas;
  /* Block-cyclic KV sharding: with kv_pos_block > 0 local key j of this rank sits at position
   * kv_offset + (j / kv_pos_block) * kv_pos_stride + j % kv_pos_block of the key axis (blocks of
   * kv_pos_block keys dealt round-robin to the ranks: kv_offset = rank * block, kv_pos_stride =
   * ranks * block), so that ALiBi, masks and rotation see true positions.  0: local key j sits at
   * kv_offset + j (contiguous shard). */
  int32_t kv_pos_block, kv_pos_stride;
} AfDecodeParams;

/* Replaces the forward launch in run_attention (attnfuse/runtime/dispatch.py:196-214)
 * and, with mask_kind == AF_MASK_BLOCKS, the one in run_block_sparse
 * (attnfuse/runtime/block_mask.py:246-270). */
AF_API int af_fwd(const AfFwdParams* params, af_stream_t stream);

/* Scratch bytes with which af_fwd runs fastest for this problem (0: none needed).  Only RoPE
 * problems with many query tiles per KV head use scratch: K is then rotated once into it
 * instead of once per query tile.  Without (enough) workspace af_fwd rotates K inside the
 * kernel, in shared memory, and gives the same result.  No counterpart in the reference, whose
 * kernel always re-rotates each K tile (attnfuse/compiler/codegen.py:332-341).  Host only. */
AF_API int64_t af_fwd_workspace_bytes(const AfFwdParams* params);

/* Replaces the three launches of run_backward (attnfuse/runtime/backward.py:131-190:
 * preproc, dK/dV, dQ) and of run_block_sparse_backward
 * (attnfuse/runtime/block_mask.py:302-362).  dq/dk/dv are fully overwritten. */
AF_API int af_bwd(const AfBwdParams* params, af_stream_t stream);

/* Scratch bytes the tensor-core backward needs for this problem (0: none).  RoPE problems keep
 * the rotated Q and K there; without it af_bwd runs the exact FFMA kernels.  Host only. */
AF_API int64_t af_bwd_workspace_bytes(const AfBwdParams* params);

/* Bytes of the optional dQ accumulator (AfBwdParams.dq_accum) with which af_bwd runs its
 * single-pass kernel for this problem; 0 when only the two-pass kernels apply (head_dim other than
 * 128, fp32, additive bias, ...).  af_bwd clears the accumulator itself.  No counterpart in the
 * reference, whose backward always recomputes S and dP in both of its kernels
 * (attnfuse/compiler/codegen_backward.py:75-302).  Host only. */
AF_API int64_t af_bwd_dq_accum_bytes(const AfBwdParams* params);

/* Replaces the split launch of run_flash_decode (attnfuse/runtime/flash_decode.py:149-170). */
AF_API int af_decode_split(const AfDecodeParams* params, af_stream_t stream);

/* Replaces the combine launch of run_flash_decode (attnfuse/runtime/flash_decode.py:173-186).
 * Writes o (if non-NULL) and partial (if non-NULL). */
AF_API int af_decode_combine(const AfDecodeParams* params, af_stream_t stream);

/* Decode (split + combine) for callers that cannot allocate device memory.  No counterpart in
 * the reference, whose decode path allocates three fp32 workspaces per call with torch.empty.
 *
 * Who needs it: a host that owns the whole device memory through its own pool and forbids
 * cudaMalloc afterwards, code on a path where the allocator must stay untouched, or a plugin
 * interface that hands over nothing but input and output pointers.  Here the split-K partials
 * go to a fixed array of AF_DECODE_STATIC_SCRATCH_BYTES that is part of the library image (each
 * GPU that loads the library keeps it until the process ends); the call itself performs no
 * cudaMalloc / cudaFree and calls no allocating library routine.
 *
 * params: as for af_decode_split + af_decode_combine; ws_m / ws_l / ws_acc are ignored, and
 * num_splits <= 0 lets the library pick.  With rows = num_splits * B * H_q the problem must
 * satisfy
 *     (2 * roundup(rows, 4) + rows * D) * 4 bytes <= AF_DECODE_STATIC_SCRATCH_BYTES,
 * otherwise AF_ERR_WORKSPACE is returned and nothing is launched.
 *
 * The first call on each device looks up the array's device address (the device must be
 * current); make that first call before starting any stream capture.  All calls share the one
 * array: two calls whose kernels may overlap on the GPU (different streams, no ordering) race
 * on it -- order them.  The array keeps the previous call's partials; every call overwrites all
 * the rows it later reads, so no clearing is required between calls. */
#define AF_DECODE_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
AF_API int af_decode_static(const AfDecodeParams* params, af_stream_t stream);

/* KV-sharded decode: merge G per-rank partials [G, B, H_q, D+1] (normalised O, LSE) that an
 * all-gather placed in this GPU's own memory.  No counterpart in the reference, which is
 * single-GPU. */
AF_API int af_decode_combine_gathered(const float* gathered, int32_t G, int32_t B, int32_t H_q,
                               int32_t D, int32_t dtype, void* o, const int64_t o_stride[4],
                               af_stream_t stream);

/* Exchange of per-rank decode partials over peer memory (KV-sharded decode), fused into the
 * combine kernels instead of a library all-gather between them.  Every rank owns one exchange
 * buffer of af_decode_exchange_bytes() bytes, zero-initialised once, mapped into every other
 * rank's address space (e.g. torch symmetric memory); peer_bases[r] is the address of rank r's
 * buffer as seen from THIS process.  `state` is zero-initialised uint32 words in local device
 * memory: step counter, unit counter, and -- for af_decode_sharded_step -- one ticket word per
 * (batch, kv head, chunk of 64 query heads) unit after them.  All ranks must make the same
 * sequence of calls.
 * No counterpart in the reference, which is single-GPU. */
typedef struct AfPeerExchange {
  int32_t world, rank;
  const uint64_t* peer_bases;   /* device array [world]                                      */
  uint32_t* state;              /* device, local                                             */
  int32_t*  status;             /* optional device word: AF_STATUS_WAIT_TIMEOUT if a peer's
                                   partial did not arrive within wait_cycles                */
  int64_t   wait_cycles;        /* bound of the wait in SM cycles; <= 0: 2^31 (~1 s)          */
} AfPeerExchange;

AF_API int64_t af_decode_exchange_bytes(int32_t world, int32_t B, int32_t H_q, int32_t D);

/* af_decode_combine + push: merge this rank's splits and store the (normalised O, LSE) rows
 * into slot `rank` of every rank's exchange buffer, then raise this rank's flag everywhere. */
AF_API int af_decode_combine_push(const AfDecodeParams* params, const AfPeerExchange* exchange,
                                  af_stream_t stream);

/* Wait (bounded) for all ranks' flags of the current step, merge the partials from this
 * rank's own buffer, write o (B, H_q, 1, D).  Call after af_decode_combine_push on the
 * same stream. */
AF_API int af_decode_wait_merge(const AfPeerExchange* exchange, int32_t B, int32_t H_q, int32_t D,
                                int32_t dtype, void* o, const int64_t o_stride[4],
                                af_stream_t stream);

/* The whole KV-sharded step in ONE launch (mode 3): split-K over this rank's keys; the last CTA
 * of every (batch, kv head) unit merges the unit's splits and stores the rows into every rank's
 * exchange buffer; the CTA that completes the last unit raises the flags; the units' last CTAs
 * then wait (bounded, status word on expiry) for all ranks and merge from this rank's own buffer
 * into o.  All CTAs of the launch must be resident at once (num_splits * units <= resident CTAs;
 * AF_ERR_INVALID otherwise).  Mode 1 (push half) and mode 2 (merge half) as two launches exist for
 * exercising several ranks on one device.  params.ws_* hold the split partials as for
 * af_decode_split; exchange.state needs 2 + units words. */
AF_API int af_decode_sharded_step(const AfDecodeParams* params, const AfPeerExchange* exchange, int32_t mode,
                                  af_stream_t stream);

/* Split count for a decode problem: the reference's _pick_num_splits
 * (attnfuse/runtime/flash_decode.py:69-95) re-tuned for 148 SMs.  `ragged` != 0: the
 * sequences have different valid lengths (kv_lens), so the CTAs of a launch take different
 * times and about five waves of them even out; 0: equal lengths, where the count is chosen so
 * that the last wave of resident CTAs is as full as possible.  Host only. */
AF_API int32_t af_decode_num_splits(int32_t B, int32_t H_q, int32_t H_kv, int32_t N_kv, int32_t sm_count,
                                    int32_t ragged);

/* Which family af_fwd / af_bwd would run for this problem (AF_FAMILY_*), or a negative
 * error.  Host only; stands in for the reference's tile-table lookup
 * (attnfuse/compiler/tiling.py:168-207). */
AF_API int32_t af_query_family(const AfProblem* p, int32_t backward);

/* Number of this library's kernel launches since load (all entry points). */
AF_API int64_t af_launch_count(void);

AF_API const char* af_last_error(void);
AF_API int32_t     af_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ATTNFUSE_B200_H_ */
