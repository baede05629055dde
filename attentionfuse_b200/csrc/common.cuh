// Shared declarations of the sm_100a attention library: element-type traits, error
// reporting, launch accounting and the per-family launcher prototypes.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <math.h>

#include "attnfuse_b200.h"

namespace af {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------
// Element types
// ---------------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
  static constexpr int code = AF_F16;
  __device__ __forceinline__ static float to_f32(__half x) { return __half2float(x); }
  __device__ __forceinline__ static __half from_f32(float x) { return __float2half_rn(x); }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int code = AF_BF16;
  __device__ __forceinline__ static float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ __forceinline__ static __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<float> {
  static constexpr int code = AF_F32;
  __device__ __forceinline__ static float to_f32(float x) { return x; }
  __device__ __forceinline__ static float from_f32(float x) { return x; }
};

// Round an fp32 value to T and back (the rounding point of a value the reference casts to
// the input dtype before a matmul).
template <typename T>
__device__ __forceinline__ float round_through(float x) { return Elem<T>::to_f32(Elem<T>::from_f32(x)); }

inline size_t elem_size(int dtype) { return dtype == AF_F32 ? 4 : 2; }

// ---------------------------------------------------------------------------------------
// Errors (thread local message) and launch accounting
// ---------------------------------------------------------------------------------------
int fail(int code, const char* fmt, ...);
void count_launch(int n = 1);
int check_cuda(cudaError_t e, const char* what);

#define AF_CUDA_OK(expr)                                   \
  do {                                                     \
    int _rc = ::af::check_cuda((expr), #expr);             \
    if (_rc != AF_OK) return _rc;                          \
  } while (0)

#define AF_REQUIRE(cond, ...)                              \
  do {                                                     \
    if (!(cond)) return ::af::fail(AF_ERR_INVALID, __VA_ARGS__); \
  } while (0)

// ---------------------------------------------------------------------------------------
// Launchers implemented by the kernel files
// ---------------------------------------------------------------------------------------
int launch_fwd_ffma(const AfFwdParams& a, cudaStream_t st);
int launch_fwd_tcgen05(const AfFwdParams& a, cudaStream_t st);
int64_t fwd_tcgen05_workspace_bytes(const AfProblem& p);
bool fwd_tcgen05_supports(const AfProblem& p, const void* o, const int64_t* o_stride,
                          const char** why);

// Shared host helpers of the tensor-core kernels (defined in fwd_tcgen05_host.cu).

int tc_make_map(CUtensorMap* out, int dtype, const void* ptr, int B, int H, int N, int D, const int64_t* st,
                int box_rows);
bool tc_tma_ok(const void* ptr, int B, int H, int N, const int64_t* st);
int tc_sm_count(int* sms);
int tc_launch_prepass(const AfProblem& p, void* q_out, void* k_out, cudaStream_t st);

int launch_bwd_ffma(const AfBwdParams& a, cudaStream_t st);
int launch_bwd_delta(const AfBwdParams& a, cudaStream_t st);
int64_t bwd_mma_workspace_bytes(const AfBwdParams& a);
int64_t bwd_mma_dq_accum_bytes(const AfBwdParams& a);
int launch_bwd_mma(const AfBwdParams& a, cudaStream_t st);
bool bwd_mma_supports(const AfBwdParams& a, const char** why);

int launch_decode_split(const AfDecodeParams& a, cudaStream_t st);
// Split-K decode of large head groups (MQA) on the tcgen05 forward kernel: the query heads of a KV
// group are the rows of one query tile.  Same partials as launch_decode_split.
bool decode_tc_supports(const AfDecodeParams& a);
int launch_decode_split_tc(const AfDecodeParams& a, cudaStream_t st);
int launch_decode_combine(const AfDecodeParams& a, cudaStream_t st);
int launch_decode_static(const AfDecodeParams& a, cudaStream_t st);
int64_t decode_exchange_bytes(int world, int B, int H_q, int D);
int launch_decode_combine_push(const AfDecodeParams& a, const AfPeerExchange* x, cudaStream_t st);
int launch_decode_sharded_step(const AfDecodeParams& a, const AfPeerExchange* x, int mode, cudaStream_t st);
int launch_decode_wait_merge(const AfPeerExchange* x, int B, int H_q, int D, int dtype, void* o, const int64_t* os,
                             cudaStream_t st);
int launch_decode_combine_gathered(const float* gathered, int G, int B, int H_q, int D,
                                   int dtype, void* o, const int64_t* o_stride, cudaStream_t st);

// ALiBi slope of head h as fp32 (slopes are stored in the input dtype).
template <typename T>
__device__ __forceinline__ float load_slope(const void* slopes, int h) {
  return Elem<T>::to_f32(reinterpret_cast<const T*>(slopes)[h]);
}

}  // namespace af
