// Host side of the tcgen05 forward: support predicate, TMA descriptor encoding, RoPE mode
// selection (fused in shared memory vs. a one-off K pre-rotation into caller workspace) and
// dispatch to the per-(head_dim, RoPE mode) instantiation units.
#include <cstdlib>
#include <mutex>

#include "fwd_tcgen05.cuh"

namespace af {
namespace {

using namespace tc;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

// Encoded maps are remembered: a serving or training loop launches the same tensors (same base,
// extents, strides) over and over, and an encode costs more than the rest of the host side of a
// launch.  Direct-mapped, keyed by everything the encoding depends on; an entry is a plain value
// (a map does not own or pin the memory it describes), so a stale one is simply never matched.
struct MapKey {
  const void* ptr; int64_t s0, s1, s2; int dtype, B, H, N, D, box;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && s0 == o.s0 && s1 == o.s1 && s2 == o.s2 && dtype == o.dtype && B == o.B && H == o.H &&
           N == o.N && D == o.D && box == o.box;
  }
};
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
constexpr int kMapSlots = 256;
std::mutex g_map_mu;
MapSlot g_map_cache[kMapSlots];

size_t map_hash(const MapKey& k) {
  uint64_t h = reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
  h ^= (uint64_t)k.N * 0xC2B2AE3D27D4EB4Full + (uint64_t)k.box * 0x165667B19E3779F9ull + (uint64_t)k.H + ((uint64_t)k.B << 20);
  return (size_t)((h >> 24) % kMapSlots);
}

int encode_map(CUtensorMap* out, int dtype, const void* ptr, int B, int H, int N, int D, const int64_t* st, int box_rows,
               int box_cols);

// (B, H, N, D) tensor with element strides -> 4-D tiled map {D, N, H, B}, box box_cols x box_rows x 1 x 1
// (box_cols * 2 bytes <= 128, the swizzle span).
int make_map(CUtensorMap* out, int dtype, const void* ptr, int B, int H, int N, int D, const int64_t* st,
             int box_rows = 128, int box_cols = 64) {
  const MapKey key{ptr, st[0], st[1], st[2], dtype, B, H, N, D, box_rows + (box_cols << 16)};
  const size_t slot = map_hash(key);
  {
    std::lock_guard<std::mutex> lock(g_map_mu);
    if (g_map_cache[slot].used && g_map_cache[slot].key == key) {
      *out = g_map_cache[slot].map;
      return AF_OK;
    }
  }
  const int rc = encode_map(out, dtype, ptr, B, H, N, D, st, box_rows, box_cols);
  if (rc != AF_OK) return rc;
  std::lock_guard<std::mutex> lock(g_map_mu);
  g_map_cache[slot].key = key;
  g_map_cache[slot].map = *out;
  g_map_cache[slot].used = true;
  return AF_OK;
}

int encode_map(CUtensorMap* out, int dtype, const void* ptr, int B, int H, int N, int D, const int64_t* st, int box_rows,
               int box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(AF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t esz = 2;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
  // Strides of extent-1 dimensions are never used for addressing; give them a legal value.
  cuuint64_t sN = (cuuint64_t)st[2] * esz, sH = (cuuint64_t)st[1] * esz, sB = (cuuint64_t)st[0] * esz;
  if (N == 1) sN = (cuuint64_t)D * esz;
  if (H == 1) sH = sN * (cuuint64_t)N;
  if (B == 1) sB = sH * (cuuint64_t)H;
  cuuint64_t strides[3] = {sN, sH, sB};
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, dtype == AF_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AF_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return AF_OK;
}

bool tma_ok(const void* ptr, int B, int H, int N, const int64_t* st) {
  if (((uintptr_t)ptr & 15) != 0 || st[3] != 1) return false;
  if (N > 1 && (st[2] <= 0 || st[2] % 8 != 0)) return false;
  if (H > 1 && (st[1] <= 0 || st[1] % 8 != 0)) return false;
  if (B > 1 && (st[0] <= 0 || st[0] % 8 != 0)) return false;
  return true;
}

// RoPE pre-pass: dst[b, h, n, :] = rope(src[b, h, n, :]) as contiguous (B, H, N, D) for Q and K
// in one launch; fp32 math, one rounding to T -- the same arithmetic as the in-kernel rotation.
// A thread owns one pair of 16-byte chunks (d, d + D/2) of one position n of one batch entry,
// loads that position's cos / sin once and walks all heads of Q, then of K, four heads per
// step so that eight 16-byte loads are in flight per thread: the traffic is the tensors
// themselves plus one read of the tables per batch entry.
struct RotateJob {
  const void* src; void* dst;   // dst == nullptr: nothing to do
  int64_t s0, s1, s2;
  int H, N;
  int pos0;                     // position of row 0 in the cos / sin tables
};

template <typename T>
__device__ __forceinline__ void rotate_pair(const uint4& xl, const uint4& xh, const uint4& cl, const uint4& ch,
                                            const uint4& sl, const uint4& sh, uint4& ol, uint4& oh) {
  const uint32_t xlw[4] = {xl.x, xl.y, xl.z, xl.w}, xhw[4] = {xh.x, xh.y, xh.z, xh.w};
  const uint32_t clw[4] = {cl.x, cl.y, cl.z, cl.w}, chw[4] = {ch.x, ch.y, ch.z, ch.w};
  const uint32_t slw[4] = {sl.x, sl.y, sl.z, sl.w}, shw[4] = {sh.x, sh.y, sh.z, sh.w};
  uint32_t lo[4], hi[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x1 = Pack2<T>::unpack(xlw[i]), x2 = Pack2<T>::unpack(xhw[i]);
    const float2 c1 = Pack2<T>::unpack(clw[i]), c2 = Pack2<T>::unpack(chw[i]);
    const float2 s1v = Pack2<T>::unpack(slw[i]), s2v = Pack2<T>::unpack(shw[i]);
    lo[i] = Pack2<T>::run(x1.x * c1.x - x2.x * s1v.x, x1.y * c1.y - x2.y * s1v.y);
    hi[i] = Pack2<T>::run(x2.x * c2.x + x1.x * s2v.x, x2.y * c2.y + x1.y * s2v.y);
  }
  ol = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  oh = make_uint4(hi[0], hi[1], hi[2], hi[3]);
}

template <typename T, int D>
__device__ __forceinline__ void rotate_heads(const RotateJob& job, int64_t b, int n, int c, const uint4& cl,
                                             const uint4& ch, const uint4& sl, const uint4& sh) {
  if (job.dst == nullptr || n >= job.N) return;
  const T* src = reinterpret_cast<const T*>(job.src) + b * job.s0 + (int64_t)n * job.s2 + c * 8;
  T* dst = reinterpret_cast<T*>(job.dst) + ((b * job.H) * (int64_t)job.N + n) * D + c * 8;
  const int64_t dst_h = (int64_t)job.N * D;
  int h = 0;
  for (; h + 4 <= job.H; h += 4) {
    uint4 xl[4], xh[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      xl[u] = *reinterpret_cast<const uint4*>(src + (h + u) * job.s1);
      xh[u] = *reinterpret_cast<const uint4*>(src + (h + u) * job.s1 + D / 2);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint4 ol, oh;
      rotate_pair<T>(xl[u], xh[u], cl, ch, sl, sh, ol, oh);
      *reinterpret_cast<uint4*>(dst + (h + u) * dst_h) = ol;
      *reinterpret_cast<uint4*>(dst + (h + u) * dst_h + D / 2) = oh;
    }
  }
  for (; h < job.H; ++h) {
    const uint4 xl = *reinterpret_cast<const uint4*>(src + h * job.s1);
    const uint4 xh = *reinterpret_cast<const uint4*>(src + h * job.s1 + D / 2);
    uint4 ol, oh;
    rotate_pair<T>(xl, xh, cl, ch, sl, sh, ol, oh);
    *reinterpret_cast<uint4*>(dst + h * dst_h) = ol;
    *reinterpret_cast<uint4*>(dst + h * dst_h + D / 2) = oh;
  }
}

template <typename T, int D>
__global__ void rope_prepass_kernel(const RotateJob jq, const RotateJob jk, const T* __restrict__ cos_,
                                    const T* __restrict__ sin_, int64_t sr, int n_max) {
  constexpr int HC = D / 16;                       // chunk pairs per row
  const int c = threadIdx.x % HC;
  const int n = blockIdx.x * (blockDim.x / HC) + threadIdx.x / HC;
  const int64_t b = blockIdx.y;
  if (n >= n_max) return;
  auto load = [&](int pos, uint4& cl, uint4& ch, uint4& sl, uint4& sh) {
    cl = __ldg(reinterpret_cast<const uint4*>(cos_ + (int64_t)pos * sr + c * 8));
    ch = __ldg(reinterpret_cast<const uint4*>(cos_ + (int64_t)pos * sr + D / 2 + c * 8));
    sl = __ldg(reinterpret_cast<const uint4*>(sin_ + (int64_t)pos * sr + c * 8));
    sh = __ldg(reinterpret_cast<const uint4*>(sin_ + (int64_t)pos * sr + D / 2 + c * 8));
  };
  uint4 cl, ch, sl, sh;
  if (n < jk.N || jq.pos0 == 0) load(n, cl, ch, sl, sh);
  rotate_heads<T, D>(jk, b, n, c, cl, ch, sl, sh);
  if (jq.pos0 != 0 && jq.dst != nullptr && n < jq.N) load(n + jq.pos0, cl, ch, sl, sh);   // queries sit further along
  rotate_heads<T, D>(jq, b, n, c, cl, ch, sl, sh);
}

template <typename T, int D>
int launch_prepass(const AfProblem& p, void* q_out, void* k_out, cudaStream_t st) {
  RotateJob jq{p.q, q_out, p.q_stride[0], p.q_stride[1], p.q_stride[2], p.H_q, p.N_q, p.q_offset};
  RotateJob jk{p.k, k_out, p.k_stride[0], p.k_stride[1], p.k_stride[2], p.H_kv, p.N_kv, 0};
  const int n_max = p.N_q > p.N_kv ? p.N_q : p.N_kv;
  constexpr int THREADS = 128, ROWS = THREADS / (D / 16);
  AF_REQUIRE(p.B <= 65535, "batch exceeds the launch grid limit");
  const dim3 grid((unsigned)((n_max + ROWS - 1) / ROWS), (unsigned)p.B);
  rope_prepass_kernel<T, D><<<grid, THREADS, 0, st>>>(jq, jk, reinterpret_cast<const T*>(p.cos),
                                                      reinterpret_cast<const T*>(p.sin), p.rope_stride_n, n_max);
  count_launch();
  return check_cuda(cudaGetLastError(), "rope_prepass launch");
}

}  // namespace

// Multiprocessor count of the current device, looked up once per device.
int tc_sm_count(int* sms) {
  static int cached[64] = {};
  int dev = 0;
  AF_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || cached[dev] == 0) {
    int n = 0;
    AF_CUDA_OK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    if (dev >= 0 && dev < 64) cached[dev] = n;
    *sms = n;
    return AF_OK;
  }
  *sms = cached[dev];
  return AF_OK;
}

int tc_make_map(CUtensorMap* out, int dtype, const void* ptr, int B, int H, int N, int D, const int64_t* st,
                int box_rows) {
  return make_map(out, dtype, ptr, B, H, N, D, st, box_rows);
}
bool tc_tma_ok(const void* ptr, int B, int H, int N, const int64_t* st) { return tma_ok(ptr, B, H, N, st); }
int tc_launch_prepass(const AfProblem& p, void* q_out, void* k_out, cudaStream_t st) {
  if (p.dtype == AF_F16)
    return p.D == 64 ? launch_prepass<__half, 64>(p, q_out, k_out, st) : launch_prepass<__half, 128>(p, q_out, k_out, st);
  return p.D == 64 ? launch_prepass<__nv_bfloat16, 64>(p, q_out, k_out, st)
                   : launch_prepass<__nv_bfloat16, 128>(p, q_out, k_out, st);
}

// Bytes of workspace with which af_fwd rotates Q and K once up front (one extra HBM-bound
// launch) instead of inside the attention kernel, where every query tile re-rotates every K
// tile it visits: O(N_q/128 * group) rotations per key against one.
static int64_t align256(int64_t x) { return (x + 255) & ~(int64_t)255; }

int64_t fwd_tcgen05_workspace_bytes(const AfProblem& p) {
  if (!p.rope) return 0;
  const int64_t q_tiles_per_kv_head = (int64_t)((p.N_q + tc::BM - 1) / tc::BM) * (p.H_q / p.H_kv);
  if (q_tiles_per_kv_head < 4) return 0;   // short sequences: rotate in shared memory, one launch
  return align256((int64_t)p.B * p.H_q * p.N_q * p.D * 2) + align256((int64_t)p.B * p.H_kv * p.N_kv * p.D * 2);
}

bool fwd_tcgen05_supports(const AfProblem& p, const void* o, const int64_t* o_stride, const char** why) {
  auto no = [&](const char* w) { if (why) *why = w; return false; };
  if (p.dtype != AF_F16 && p.dtype != AF_BF16) return no("dtype is not f16/bf16");
  if (p.D != 64 && p.D != 128) return no("head_dim is not 64 or 128");
  if (p.norm_kind != AF_NORM_SOFTMAX) return no("normalisation is not softmax");
  if (p.bias_kind == AF_BIAS_ADDITIVE) return no("additive bias");
  if (!(p.sm_scale > 0.f)) return no("non-positive scale");
  if (p.N_q < 1 || p.N_kv < 1) return no("empty sequence");
  if (p.mask_kind == AF_MASK_BLOCKS && (p.block_m % tc::BM != 0 || p.block_n % tc::BN != 0))
    return no("block size is not a multiple of 128");
  if (!tma_ok(p.q, p.B, p.H_q, p.N_q, p.q_stride) || !tma_ok(p.k, p.B, p.H_kv, p.N_kv, p.k_stride) ||
      !tma_ok(p.v, p.B, p.H_kv, p.N_kv, p.v_stride))
    return no("Q/K/V not TMA-addressable (16-byte aligned base and strides, unit inner stride)");
  if (o_stride[3] != 1 || ((uintptr_t)o & 15) != 0 || o_stride[2] % 8 != 0 || o_stride[1] % 8 != 0 ||
      o_stride[0] % 8 != 0)
    return no("O rows not 16-byte aligned");
  if (p.rope && (p.rope_stride_n % 8 != 0 || ((uintptr_t)p.cos & 15) != 0 || ((uintptr_t)p.sin & 15) != 0))
    return no("cos/sin rows not 16-byte aligned");
  return true;
}

// Units per chunk of the item order (TcArgs::unit_chunk).  While all K and V of the problem fit the
// 126 MB L2 with room to spare (96 MB: measured up to 67 MB, no re-reads from DRAM) the order is the
// plain one, whose item weights the zig-zag deal balances to 0.3 %.  Beyond that every key tile is
// fetched from DRAM many times over (11 x at 201 MB), and the units are taken in chunks: the largest
// divisor of the unit count that is a multiple of `group_units` (the units of a KV group stay
// together) and whose K and V stay inside 24 MB (a line used by SMs of both dies is held by both
// halves of the L2, and Q and O stream through it as well; 24 against 40 MB measured).  Chunking
// costs 2 - 4 % of balance in the static deal and gains 4 - 13 % at 134 - 268 MB of K and V.
// ATTNFUSE_L2_KV_MB overrides the chunk budget and applies it at any size.
static int choose_unit_chunk(int units, int group_units, double kv_bytes_per_unit) {
  double budget = 24.0 * 1048576.0;
  bool forced = false;
  if (const char* e = std::getenv("ATTNFUSE_L2_KV_MB")) {
    const double v = std::atof(e);
    if (v > 0.0) { budget = v * 1048576.0; forced = true; }
  }
  if (group_units < 1) group_units = 1;
  const double total = (double)units * kv_bytes_per_unit;
  if (total <= budget || (!forced && total <= 96.0 * 1048576.0)) return units;
  int best = group_units;
  for (int d = group_units; d <= units; d += group_units)
    if (units % d == 0 && (double)d * kv_bytes_per_unit <= budget) best = d;
  return best;
}

static void set_item_order(tc::TcArgs& args, int units, int unit_chunk, int rows) {
  args.unit_chunk = unit_chunk;
  args.items_per_chunk = rows * unit_chunk;
  args.div_ipc = tc::FastDiv::make((uint32_t)args.items_per_chunk);
  args.div_chunk = tc::FastDiv::make((uint32_t)unit_chunk);
  (void)units;
}

// The two-heads-per-CTA schedule (fwd_pair_tcgen05.cuh): head dim 128, an even number of query
// heads per KV head, element masks only, operands already rotated.  ATTNFUSE_FWD_PAIR=0 in the
// environment (read at every call) keeps the one-head schedule, for comparisons between the two.
static bool pair_schedule_applies(const AfProblem& p, int rope_mode) {
  if (p.D != 128 || rope_mode != tc::ROPE_NONE || p.mask_kind == AF_MASK_BLOCKS) return false;
  if (p.H_kv < 1 || p.H_q % p.H_kv != 0 || ((p.H_q / p.H_kv) & 1) != 0) return false;
  const char* e = std::getenv("ATTNFUSE_FWD_PAIR");
  return !(e != nullptr && e[0] == '0');
}

int launch_fwd_tcgen05(const AfFwdParams& a, cudaStream_t st) {
  const char* why = nullptr;
  if (!fwd_tcgen05_supports(a.p, a.o, a.o_stride, &why))
    return fail(AF_ERR_UNSUPPORTED, "tcgen05 forward: %s", why);
  const AfProblem& p = a.p;
  tc::TcArgs args{};
  args.a = a;
  args.num_m_blocks = (p.N_q + tc::BM - 1) / tc::BM;
  args.kv_tiles_per_block = p.mask_kind == AF_MASK_BLOCKS ? p.block_n / tc::BN : 1;
  args.q_tiles_per_block = p.mask_kind == AF_MASK_BLOCKS ? p.block_m / tc::BM : 1;
  AF_REQUIRE((int64_t)args.num_m_blocks * p.B * p.H_q <= 0x7fffffff, "too many tiles for one launch");
  args.total_items = args.num_m_blocks * p.B * p.H_q;
  args.div_hq = tc::FastDiv::make((uint32_t)p.H_q);
  args.div_group = tc::FastDiv::make((uint32_t)(p.H_q / p.H_kv));
  {
    const int group = p.H_q / p.H_kv;
    const double kv_bytes = 2.0 * 2.0 * (double)p.N_kv * p.D / group;   // K and V of a query head's share
    set_item_order(args, p.B * p.H_q, choose_unit_chunk(p.B * p.H_q, group, kv_bytes), args.num_m_blocks);
  }
  {
    // One CTA fits per SM (shared memory), so the kernel runs persistently: one CTA per SM walks
    // its share of the query tiles with the pipeline kept full across tile boundaries (measured
    // faster than one CTA per query tile at every size, 951 vs 851 TFLOP/s on causal 4x32x4096x128).
    int sms = 0;
    { const int rc_sm = tc_sm_count(&sms); if (rc_sm != AF_OK) return rc_sm; }
    args.grid_ctas = (sms > 0 && sms < args.total_items) ? sms : args.total_items;
  }

  int mode = p.rope ? tc::ROPE_FUSED : tc::ROPE_NONE;
  const void* q_ptr = p.q;
  const void* k_ptr = p.k;
  int64_t q_stride[4] = {p.q_stride[0], p.q_stride[1], p.q_stride[2], p.q_stride[3]};
  int64_t k_stride[4] = {p.k_stride[0], p.k_stride[1], p.k_stride[2], p.k_stride[3]};
  const int64_t need = fwd_tcgen05_workspace_bytes(p);
  if (p.rope && need > 0 && a.workspace != nullptr && a.workspace_bytes >= need &&
      ((uintptr_t)a.workspace & 255) == 0) {
    void* q_rot = a.workspace;
    void* k_rot = static_cast<char*>(a.workspace) + align256((int64_t)p.B * p.H_q * p.N_q * p.D * 2);
    const int rc = tc_launch_prepass(p, q_rot, k_rot, st);
    if (rc != AF_OK) return rc;
    mode = tc::ROPE_NONE;   // operands are rotated: run the plain kernel on them
    q_ptr = q_rot; k_ptr = k_rot;
    q_stride[3] = 1; q_stride[2] = p.D; q_stride[1] = (int64_t)p.N_q * p.D; q_stride[0] = q_stride[1] * p.H_q;
    k_stride[3] = 1; k_stride[2] = p.D; k_stride[1] = (int64_t)p.N_kv * p.D; k_stride[0] = k_stride[1] * p.H_kv;
  }

  CUtensorMap mq, mk, mv, mo;
  int rc;
  if ((rc = make_map(&mq, p.dtype, q_ptr, p.B, p.H_q, p.N_q, p.D, q_stride)) != AF_OK) return rc;
  if ((rc = make_map(&mk, p.dtype, k_ptr, p.B, p.H_kv, p.N_kv, p.D, k_stride)) != AF_OK) return rc;
  if ((rc = make_map(&mv, p.dtype, p.v, p.B, p.H_kv, p.N_kv, p.D, p.v_stride)) != AF_OK) return rc;
  // output rows leave through a TMA store: one box = the 32 rows of a warp x half of the head dim
  if ((rc = make_map(&mo, p.dtype, a.o, p.B, p.H_q, p.N_q, p.D, a.o_stride, 32, p.D / 2)) != AF_OK) return rc;
  if (pair_schedule_applies(p, mode)) {
    // two query heads of a KV group per CTA: one K / V load feeds two S products
    const int pairs = p.H_q / 2;
    args.total_items = args.num_m_blocks * p.B * pairs;
    args.div_hq = tc::FastDiv::make((uint32_t)pairs);
    args.div_group = tc::FastDiv::make((uint32_t)(p.H_q / p.H_kv / 2));
    {
      const int group_pairs = p.H_q / p.H_kv / 2;
      const double kv_bytes = 2.0 * 2.0 * (double)p.N_kv * p.D / group_pairs;
      set_item_order(args, p.B * pairs, choose_unit_chunk(p.B * pairs, group_pairs, kv_bytes), args.num_m_blocks);
    }
    int sms = 0;
    { const int rc_sm = tc_sm_count(&sms); if (rc_sm != AF_OK) return rc_sm; }
    args.grid_ctas = (sms > 0 && sms < args.total_items) ? sms : args.total_items;
    return tc::launch_pair_d128(p.dtype, args, mq, mk, mv, mo, st);
  }
  if (p.D == 64) {
    if (mode == tc::ROPE_NONE) return tc::launch_d64_norope(p.dtype, args, mq, mk, mv, mo, st);
    return tc::launch_d64_fused(p.dtype, args, mq, mk, mv, mo, st);
  }
  if (mode == tc::ROPE_NONE) return tc::launch_d128_norope(p.dtype, args, mq, mk, mv, mo, st);
  return tc::launch_d128_fused(p.dtype, args, mq, mk, mv, mo, st);
}

// ---------------------------------------------------------------------------------------
// Split-K decode on the forward kernel.  With more than 16 query heads per KV head (MQA) the
// mma.sync decode kernel is bound by the legacy tensor path; here the heads of a group are the
// rows of a 128-row query tile (Q viewed as (B, H_kv, group, D)), every (split, batch, kv head)
// is one work item of the persistent kernel, and its epilogue writes the un-normalised partials.
// ---------------------------------------------------------------------------------------
static void decode_q_view(const AfDecodeParams& a, int64_t out[4]) {
  const int group = a.H_q / a.H_kv;
  out[0] = a.q_stride[0]; out[1] = (int64_t)group * a.q_stride[1]; out[2] = a.q_stride[1]; out[3] = a.q_stride[3];
}

bool decode_tc_supports(const AfDecodeParams& a) {
  if (a.H_kv < 1 || a.H_q % a.H_kv != 0) return false;
  const int group = a.H_q / a.H_kv;
  if (group <= 16 || group > tc::BM) return false;   // small groups: the bandwidth-tuned mma.sync kernel
  if (a.dtype != AF_F16 && a.dtype != AF_BF16) return false;
  if (a.D != 64 && a.D != 128) return false;
  if (a.bias_kind != AF_BIAS_NONE || !(a.sm_scale > 0.f) || a.N_kv < 1 || a.num_splits < 1) return false;
  if (a.mask_kind != AF_MASK_FULL || a.rope) return false;   // masks and rotation: the mma.sync kernel
  if (a.ws_acc == nullptr || ((uintptr_t)a.ws_acc & 15) != 0) return false;
  int64_t qs[4];
  decode_q_view(a, qs);
  return tma_ok(a.q, a.B, a.H_kv, group, qs) && tma_ok(a.k, a.B, a.H_kv, a.N_kv, a.k_stride) &&
         tma_ok(a.v, a.B, a.H_kv, a.N_kv, a.v_stride);
}

int launch_decode_split_tc(const AfDecodeParams& a, cudaStream_t st) {
  AF_REQUIRE(decode_tc_supports(a), "tcgen05 decode does not support this problem");
  const int group = a.H_q / a.H_kv;
  int64_t qs[4];
  decode_q_view(a, qs);
  tc::TcArgs args{};
  AfProblem& p = args.a.p;
  p.dtype = a.dtype;
  p.B = a.B; p.H_q = a.H_kv; p.H_kv = a.H_kv; p.N_q = group; p.N_kv = a.N_kv; p.D = a.D;
  p.sm_scale = a.sm_scale;
  p.mask_kind = AF_MASK_FULL; p.bias_kind = AF_BIAS_NONE; p.norm_kind = AF_NORM_SOFTMAX;
  p.status = a.status;
  args.num_m_blocks = 1;
  args.kv_tiles_per_block = args.q_tiles_per_block = 1;
  args.num_splits = a.num_splits;
  args.kv_lens = a.kv_lens;
  args.ws_m = a.ws_m; args.ws_l = a.ws_l; args.ws_acc = a.ws_acc;
  AF_REQUIRE((int64_t)a.num_splits * a.B * a.H_kv <= 0x7fffffff, "too many items for one launch");
  args.total_items = a.num_splits * a.B * a.H_kv;
  args.div_hq = tc::FastDiv::make((uint32_t)p.H_q);
  args.div_group = tc::FastDiv::make(1u);   // one pseudo-head per KV head
  set_item_order(args, p.B * p.H_q, p.B * p.H_q, a.num_splits);   // splits x (batch, pseudo-head), plain order
  int sms = 0;
  { const int rc_sm = tc_sm_count(&sms); if (rc_sm != AF_OK) return rc_sm; }
  args.grid_ctas = (sms > 0 && sms < args.total_items) ? sms : args.total_items;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_map(&mq, a.dtype, a.q, a.B, a.H_kv, group, a.D, qs)) != AF_OK) return rc;
  if ((rc = make_map(&mk, a.dtype, a.k, a.B, a.H_kv, a.N_kv, a.D, a.k_stride)) != AF_OK) return rc;
  if ((rc = make_map(&mv, a.dtype, a.v, a.B, a.H_kv, a.N_kv, a.D, a.v_stride)) != AF_OK) return rc;
  // the split-K epilogue writes fp32 partials with plain stores: the output map is not used
  if (a.D == 64) return tc::launch_d64_norope(a.dtype, args, mq, mk, mv, mq, st);
  return tc::launch_d128_norope(a.dtype, args, mq, mk, mv, mq, st);
}

}  // namespace af
