// Shared device helpers for the sm_100a kernels: vector access, reductions, fp8 conversion,
// launch-error reporting. Everything here is header-only.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MSGL_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
enum MsglDtype : int { MSGL_BF16 = 0, MSGL_F16 = 1, MSGL_F32 = 2, MSGL_E4M3 = 3 };

// Status codes returned by the C entry points. 0 = launched.
enum MsglStatus : int {
  MSGL_OK = 0,
  MSGL_BAD_ARG = 1,       // shape / alignment / dtype the kernel does not support
  MSGL_CUDA_ERROR = 2,    // a CUDA runtime or driver call failed; see msgl_last_error()
  MSGL_TIMEOUT = 3,       // a bounded device-side wait gave up (read from the status word)
};

namespace msgl {

constexpr float kFp8Max = 448.0f;

template <typename T> struct Vec8;  // eight 16-bit elements = 16 bytes
template <> struct alignas(16) Vec8<__nv_bfloat16> { __nv_bfloat162 v[4]; };
template <> struct alignas(16) Vec8<__half> { __half2 v[4]; };

__device__ __forceinline__ float2 to_float2(__nv_bfloat162 x) { return __bfloat1622float2(x); }
__device__ __forceinline__ float2 to_float2(__half2 x) { return __half22float2(x); }
template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ type make(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <> struct Pack2<__half> {
  using type = __half2;
  static __device__ __forceinline__ type make(float a, float b) { return __floats2half2_rn(a, b); }
};
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_float(float x) { return x; }
template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }

template <typename T> __device__ __forceinline__ void load8(const T* p, float (&out)[8]) {
  Vec8<T> v = *reinterpret_cast<const Vec8<T>*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = to_float2(v.v[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&in)[8]) {
  Vec8<T> v;
#pragma unroll
  for (int i = 0; i < 4; ++i) v.v[i] = Pack2<T>::make(in[2 * i], in[2 * i + 1]);
  *reinterpret_cast<Vec8<T>*>(p) = v;
}

// e4m3 pair from two floats, saturating to +-448
__device__ __forceinline__ uint16_t float2_to_e4m3x2(float a, float b) {
  return (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint8_t float_to_e4m3(float a) {
  return (uint8_t)__nv_cvt_float_to_fp8(a, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float e4m3_to_float(uint8_t x) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(x, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
// eight floats -> eight e4m3 bytes (one 8-byte store). Multiplies by the reciprocal of the scale:
// against x / scale this differs only when the quotient sits within one fp32 ulp of an e4m3
// rounding boundary (about one element in a million), and an IEEE division per element made the
// row kernels compute-bound.
__device__ __forceinline__ uint2 pack8_e4m3(const float (&x)[8], float scale) {
  const float inv = 1.0f / scale;
  uint32_t lo = (uint32_t)float2_to_e4m3x2(x[0] * inv, x[1] * inv) |
                ((uint32_t)float2_to_e4m3x2(x[2] * inv, x[3] * inv) << 16);
  uint32_t hi = (uint32_t)float2_to_e4m3x2(x[4] * inv, x[5] * inv) |
                ((uint32_t)float2_to_e4m3x2(x[6] * inv, x[7] * inv) << 16);
  return make_uint2(lo, hi);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide reductions; `scratch` holds 32 floats. Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nw ? scratch[lane] : 0.f;
  return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nw ? scratch[lane] : -INFINITY;
  return warp_max(r);
}

// Programmatic dependent launch. Every kernel of this library starts with pdl_wait() before it
// touches global memory that an earlier kernel of the stream may still be writing (or reading),
// and raises pdl_trigger() early, so that the next kernel of the stream is scheduled while this
// one still runs: its launch latency and its prologue (barrier initialisation, tensor-memory
// allocation, descriptor prefetch) overlap this kernel's tail. In a kernel launched without the
// attribute both instructions do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
  pdl_wait();
  pdl_trigger();
}

// Bounds-checking build (-DMSGL_CHECK_BOUNDS, library libmsgl_cuda_checked.so): every index a kernel
// takes from a device array (token slot, page id, position, expert id, request slot) goes through
// MSGL_OOB(value, limit) before it is used. A value outside [0, limit) is recorded as
// (source line, value, limit) in a small ring of the translation unit and the macro yields true,
// on which the kernel skips that access; nothing traps. The host collects and clears the rings of
// all translation units with msgl_bounds_report(). In the regular build the macro is `false`
// and the kernels keep their silent clamps.
#ifdef MSGL_CHECK_BOUNDS
struct BoundsRecord {
  int line;
  int pad;
  long long value, limit;
};
constexpr int kBoundsRing = 32;
static __device__ BoundsRecord t_bounds_ring[kBoundsRing];
static __device__ unsigned int t_bounds_count;
__device__ __forceinline__ bool oob_record(long long v, long long limit, int line) {
  if (v >= 0 && v < limit) return false;
  // one record per distinct (line, value): the threads of a block usually trip over the same index,
  // so only the first active lane of a warp records, and not what the ring already holds
  if ((threadIdx.x & 31) != (unsigned)(__ffs(__activemask()) - 1)) return true;
  const unsigned int seen = min(*(volatile unsigned int*)&t_bounds_count, (unsigned)kBoundsRing);
  for (unsigned int j = 0; j < seen; ++j)
    if (*(volatile int*)&t_bounds_ring[j].line == line && *(volatile long long*)&t_bounds_ring[j].value == v) return true;
  const unsigned int i = atomicAdd(&t_bounds_count, 1u);
  if (i < (unsigned)kBoundsRing) {
    t_bounds_ring[i].line = line;
    t_bounds_ring[i].value = v;
    t_bounds_ring[i].limit = limit;
  }
  return true;
}
#define MSGL_OOB(value, limit) ::msgl::oob_record((long long)(value), (long long)(limit), __LINE__)
#else
#define MSGL_OOB(value, limit) false
#endif

}  // namespace msgl

#ifdef MSGL_CHECK_BOUNDS
// Each translation unit registers a collector for its own ring when the library is loaded (host
// code only); msgl_bounds_report (elementwise.cu) walks the collectors.
typedef int (*msgl_bounds_collect_fn)(const char** file, msgl::BoundsRecord* out, int max_records);
void msgl_bounds_register(msgl_bounds_collect_fn fn);
namespace {
int msgl_bounds_collect_tu(const char** file, msgl::BoundsRecord* out, int max_records) {
#ifdef MSGL_TU_NAME
  *file = MSGL_TU_NAME;
#else
  *file = __FILE__;
#endif
  unsigned int n = 0;
  if (cudaMemcpyFromSymbol(&n, msgl::t_bounds_count, sizeof(n)) != cudaSuccess || n == 0) return 0;
  msgl::BoundsRecord ring[msgl::kBoundsRing];
  if (cudaMemcpyFromSymbol(ring, msgl::t_bounds_ring, sizeof(ring)) != cudaSuccess) return 0;
  const unsigned int zero = 0;
  cudaMemcpyToSymbol(msgl::t_bounds_count, &zero, sizeof(zero));
  int k = (int)(n < (unsigned)msgl::kBoundsRing ? n : (unsigned)msgl::kBoundsRing);
  if (k > max_records) k = max_records;
  for (int i = 0; i < k; ++i) out[i] = ring[i];
  return k;
}
struct MsglBoundsRegistrar {
  MsglBoundsRegistrar() { msgl_bounds_register(&msgl_bounds_collect_tu); }
};
MsglBoundsRegistrar g_msgl_bounds_registrar;
}  // namespace
#endif

// Host side: launches go through msgl_launch, which adds the programmatic-stream-serialization
// attribute unless msgl_set_pdl(0) switched it off. The kernel argument list must be complete
// (default arguments do not exist behind a function pointer).
bool msgl_pdl_enabled();
template <typename... P, typename... A>
inline cudaError_t msgl_launch(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               A&&... args) {
  static_assert(sizeof...(P) == sizeof...(A), "msgl_launch: pass every kernel argument");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = msgl_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

// Host side: remember the last CUDA error text for msgl_last_error().
void msgl_set_error(const char* where, cudaError_t err);
void msgl_set_error_text(const char* text);
#define MSGL_CHECK_LAUNCH(where)                      \
  do {                                                \
    cudaError_t _e = cudaGetLastError();              \
    if (_e != cudaSuccess) {                          \
      msgl_set_error(where, _e);                      \
      return MSGL_CUDA_ERROR;                         \
    }                                                 \
  } while (0)
