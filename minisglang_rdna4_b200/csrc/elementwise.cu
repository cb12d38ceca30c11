// Elementwise / row-wise kernels: embedding gather, RMSNorm (+residual add) (+per-token e4m3
// producer), gated activations (+quant), stand-alone activation quantisers.
//
// Replaces the reference's tail_hip package (rms_norm, rms_norm_add, rms_norm_quant,
// rms_norm_add_quant, silu_and_mul, gelu_and_mul; python/minisgl/layers/norm.py:16-168,
// python/minisgl/layers/activation.py:25-64) and its embedding gather
// (python/minisgl/kernel/csrc/jit/index.cu:31-96). All kernels are memory-bound: they read
// each input once with 16-byte accesses and keep the row in shared memory between the
// reduction and the write.
#include "common.cuh"

#include <string>

using namespace msgl;

static thread_local std::string g_last_error;
void msgl_set_error(const char* where, cudaError_t err) {
  g_last_error = std::string(where) + ": " + cudaGetErrorString(err);
}
void msgl_set_error_text(const char* text) { g_last_error = text; }
MSGL_API const char* msgl_last_error() { return g_last_error.c_str(); }

static int g_pdl = 1;
bool msgl_pdl_enabled() { return g_pdl != 0; }
// Programmatic dependent launch of every kernel of the library: 1 on (default), 0 off.
MSGL_API int msgl_set_pdl(int on) {
  const int prev = g_pdl;
  g_pdl = on;
  return prev;
}

// ------------------------------------------------------------------------------------------
// embedding: out[i, :] = (start <= ids[i] < start + len) ? W[ids[i] - start, :] : 0
// ------------------------------------------------------------------------------------------
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const uint4* __restrict__ w,
                                 uint4* __restrict__ out, int row_vecs, int start, int len) {
  pdl_enter();
  int row = blockIdx.x;
  (void)MSGL_OOB(ids[row], 0x7fffffffLL);   // a negative token id
  int id = ids[row] - start;
  bool inside = id >= 0 && id < len;
  const uint4* src = w + (size_t)(inside ? id : 0) * row_vecs;
  uint4* dst = out + (size_t)row * row_vecs;
  for (int i = threadIdx.x; i < row_vecs; i += blockDim.x)
    dst[i] = inside ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
}

MSGL_API int msgl_embedding(const void* ids, const void* w, void* out, int rows, int hidden_bytes,
                            int start, int len, cudaStream_t stream) {
  if (hidden_bytes % 16) return MSGL_BAD_ARG;
  if (rows == 0) return MSGL_OK;
  int vecs = hidden_bytes / 16;
  int threads = vecs < 256 ? ((vecs + 31) / 32) * 32 : 256;
  msgl_launch(embedding_kernel, dim3(rows), dim3(threads), 0, stream, (const int32_t*)ids, (const uint4*)w, (uint4*)out, vecs,
                                                 start, len);
  MSGL_CHECK_LAUNCH("embedding");
  return MSGL_OK;
}

// ------------------------------------------------------------------------------------------
// RMSNorm family. One CTA of 128 threads per row; every thread keeps its VPT 16-byte vectors of
// the (summed) row in registers between the reduction and the write, so the row is read once.
//   ADD   : residual += x (stored back, rounded to T), norm of the sum
//   QUANT : emit e4m3 row + fp32 scale (amax/448) instead of T
// ------------------------------------------------------------------------------------------
constexpr int kRowThreads = 128;

//   PLANES: x is fp32 [planes][rows][hidden], the K ranges of a split-K GEMM; they are summed in
//           ascending order and rounded to T, which is what an unsplit GEMM would have handed over
template <typename T, bool ADD, bool QUANT, int VPT, bool PLANES = false>
__global__ void __launch_bounds__(kRowThreads) rms_norm_kernel(const T* __restrict__ x, T* __restrict__ residual,
                                                               const T* __restrict__ w, T* __restrict__ out,
                                                               uint8_t* __restrict__ out_q,
                                                               float* __restrict__ out_scale, int hidden, float eps,
                                                               float w_offset, int planes = 0,
                                                               size_t plane_stride = 0) {
  pdl_enter();
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  const T* xr = x + (size_t)row * hidden;
  const float* xp = reinterpret_cast<const float*>(x) + (size_t)row * hidden;
  T* rr = ADD ? residual + (size_t)row * hidden : nullptr;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = (j * kRowThreads + threadIdx.x) * 8;
    if (i < hidden) {
      if (PLANES) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j][k] = 0.f;
        for (int p = 0; p < planes; ++p) {
          const float4 lo = __ldg(reinterpret_cast<const float4*>(xp + p * plane_stride + i));
          const float4 hi = __ldg(reinterpret_cast<const float4*>(xp + p * plane_stride + i + 4));
          v[j][0] += lo.x; v[j][1] += lo.y; v[j][2] += lo.z; v[j][3] += lo.w;
          v[j][4] += hi.x; v[j][5] += hi.y; v[j][6] += hi.z; v[j][7] += hi.w;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j][k] = to_float(from_float<T>(v[j][k]));
      } else {
        load8(xr + i, v[j]);
      }
      if (ADD) {
        float r[8];
        load8(rr + i, r);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j][k] += r[k];
        store8(rr + i, v[j]);
        // the norm sees the rounded residual, exactly what the next layer will read
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j][k] = to_float(from_float<T>(v[j][k]));
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += v[j][k] * v[j][k];
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)hidden + eps);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = (j * kRowThreads + threadIdx.x) * 8;
    if (i < hidden) {
      float wv[8];
      load8(w + i, wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        // round to T as the unfused op would, so the quantised row matches norm -> quant
        v[j][k] = to_float(from_float<T>(v[j][k] * rstd * (wv[k] + w_offset)));
        if (QUANT) amax = fmaxf(amax, fabsf(v[j][k]));
      }
      if (!QUANT) store8(out + (size_t)row * hidden + i, v[j]);
    }
  }
  if (QUANT) {
    amax = block_max(amax, scratch);
    const float scale = fmaxf(amax, 1e-8f) / kFp8Max;
    if (threadIdx.x == 0) out_scale[row] = scale;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = (j * kRowThreads + threadIdx.x) * 8;
      if (i < hidden) *reinterpret_cast<uint2*>(out_q + (size_t)row * hidden + i) = pack8_e4m3(v[j], scale);
    }
  }
}

template <typename T, int VPT>
static void launch_rms_vpt(const void* x, void* residual, const void* w, void* out, void* out_q, void* out_scale,
                           int rows, int hidden, float eps, float off, cudaStream_t s) {
  const bool add = residual != nullptr, quant = out_q != nullptr;
#define RMS_LAUNCH(A, Q)                                                                                    \
  msgl_launch(rms_norm_kernel<T, A, Q, VPT>, dim3(rows), dim3(kRowThreads), 0, s, (const T*)x, (T*)residual, (const T*)w, (T*)out, \
                                                            (uint8_t*)out_q, (float*)out_scale, hidden, eps, off, 0, (size_t)0)
  if (add && quant) RMS_LAUNCH(true, true);
  else if (add) RMS_LAUNCH(true, false);
  else if (quant) RMS_LAUNCH(false, true);
  else RMS_LAUNCH(false, false);
#undef RMS_LAUNCH
}

template <typename T>
static int launch_rms(const void* x, void* residual, const void* w, void* out, void* out_q, void* out_scale,
                      int rows, int hidden, float eps, int plus_one, cudaStream_t s) {
  const float off = plus_one ? 1.f : 0.f;
  const int vpt = (hidden / 8 + kRowThreads - 1) / kRowThreads;
  if (vpt <= 1) launch_rms_vpt<T, 1>(x, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else if (vpt <= 2) launch_rms_vpt<T, 2>(x, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else if (vpt <= 3) launch_rms_vpt<T, 3>(x, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else if (vpt <= 4) launch_rms_vpt<T, 4>(x, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else if (vpt <= 6) launch_rms_vpt<T, 6>(x, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else if (vpt <= 8) launch_rms_vpt<T, 8>(x, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else if (vpt <= 16) launch_rms_vpt<T, 16>(x, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("rms_norm");
  return MSGL_OK;
}

template <typename T, int VPT>
static void launch_rms_planes_vpt(const void* x, int planes, void* residual, const void* w, void* out, void* out_q,
                                  void* out_scale, int rows, int hidden, float eps, float off, cudaStream_t s) {
  const size_t stride = (size_t)rows * hidden;
  if (out_q != nullptr)
    msgl_launch(rms_norm_kernel<T, true, true, VPT, true>, dim3(rows), dim3(kRowThreads), 0, s, (const T*)x, (T*)residual, (const T*)w, (T*)out, (uint8_t*)out_q, (float*)out_scale, hidden, eps, off, planes, stride);
  else
    msgl_launch(rms_norm_kernel<T, true, false, VPT, true>, dim3(rows), dim3(kRowThreads), 0, s, (const T*)x, (T*)residual, (const T*)w, (T*)out, (uint8_t*)out_q, (float*)out_scale, hidden, eps, off, planes, stride);
}

template <typename T>
static int launch_rms_planes(const void* x, int planes, void* residual, const void* w, void* out, void* out_q,
                             void* out_scale, int rows, int hidden, float eps, int plus_one, cudaStream_t s) {
  const float off = plus_one ? 1.f : 0.f;
  const int vpt = (hidden / 8 + kRowThreads - 1) / kRowThreads;
  if (vpt <= 1) launch_rms_planes_vpt<T, 1>(x, planes, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else if (vpt <= 2) launch_rms_planes_vpt<T, 2>(x, planes, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else if (vpt <= 3) launch_rms_planes_vpt<T, 3>(x, planes, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else if (vpt <= 4) launch_rms_planes_vpt<T, 4>(x, planes, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else if (vpt <= 8) launch_rms_planes_vpt<T, 8>(x, planes, residual, w, out, out_q, out_scale, rows, hidden, eps, off, s);
  else return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("rms_norm_planes");
  return MSGL_OK;
}

// residual += sum of the fp32 planes [planes][rows][hidden] of a split-K GEMM (ascending order,
// rounded to the 16-bit type first), then the norm of the sum; 16-bit or quantised output.
MSGL_API int msgl_rms_norm_planes(const void* x_planes, int planes, void* residual, const void* w, void* out,
                                  void* out_q, void* out_scale, int rows, int hidden, float eps, int plus_one,
                                  int dtype, cudaStream_t stream) {
  if (hidden % 8 || hidden > 8 * 8 * kRowThreads || planes < 1 || residual == nullptr) return MSGL_BAD_ARG;
  if (rows == 0) return MSGL_OK;
  if (dtype == MSGL_BF16)
    return launch_rms_planes<__nv_bfloat16>(x_planes, planes, residual, w, out, out_q, out_scale, rows, hidden, eps,
                                            plus_one, stream);
  if (dtype == MSGL_F16)
    return launch_rms_planes<__half>(x_planes, planes, residual, w, out, out_q, out_scale, rows, hidden, eps, plus_one,
                                     stream);
  return MSGL_BAD_ARG;
}

// residual == nullptr: plain norm. out_q != nullptr: quantised output (out may be nullptr).
MSGL_API int msgl_rms_norm(const void* x, void* residual, const void* w, void* out, void* out_q,
                           void* out_scale, int rows, int hidden, float eps, int plus_one, int dtype,
                           cudaStream_t stream) {
  if (hidden % 8 || hidden > 16 * 8 * kRowThreads) return MSGL_BAD_ARG;
  if (rows == 0) return MSGL_OK;
  if (dtype == MSGL_BF16)
    return launch_rms<__nv_bfloat16>(x, residual, w, out, out_q, out_scale, rows, hidden, eps, plus_one, stream);
  if (dtype == MSGL_F16)
    return launch_rms<__half>(x, residual, w, out, out_q, out_scale, rows, hidden, eps, plus_one, stream);
  return MSGL_BAD_ARG;
}

// ------------------------------------------------------------------------------------------
// gated activation: out[m, i] = act(x[m, i]) * x[m, I + i]
// ------------------------------------------------------------------------------------------
enum ActKind : int { ACT_SILU = 0, ACT_GELU = 1, ACT_GELU_TANH = 2 };
__device__ __forceinline__ float act_fn(float g, int kind) {
  if (kind == ACT_SILU) {
    // x * sigmoid(x) = h + h * tanh(h) with h = x / 2: one special-function op instead of two
    // (exp and reciprocal); tanh.approx is good to ~2^-11, below the 16-bit rounding of the result
    const float h = 0.5f * g;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
    return fmaf(h, t, h);
  }
  if (kind == ACT_GELU) return 0.5f * g * (1.f + erff(g * 0.70710678118654752f));
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g)));
}

template <typename T>
__global__ void act_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, size_t total_vecs,
                               int kind) {
  pdl_enter();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_vecs) return;
  int vecs_per_row = inter / 8;
  size_t row = idx / vecs_per_row;
  int col = (int)(idx % vecs_per_row) * 8;
  const T* g = x + row * 2 * inter + col;
  float a[8], b[8], y[8];
  load8(g, a);
  load8(g + inter, b);
#pragma unroll
  for (int k = 0; k < 8; ++k) y[k] = act_fn(a[k], kind) * b[k];
  store8(out + row * inter + col, y);
}

template <typename T, int VPT, int THREADS>
__global__ void __launch_bounds__(THREADS) act_mul_quant_kernel(const T* __restrict__ x,
                                                                    uint8_t* __restrict__ out_q,
                                                                    float* __restrict__ out_scale, int inter,
                                                                    int kind) {
  pdl_enter();
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  const T* g = x + (size_t)row * 2 * inter;
  float v[VPT][8];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = (j * THREADS + threadIdx.x) * 8;
    if (i < inter) {
      float a[8], b[8];
      load8(g + i, a);
      load8(g + inter + i, b);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        v[j][k] = to_float(from_float<T>(act_fn(a[k], kind) * b[k]));
        amax = fmaxf(amax, fabsf(v[j][k]));
      }
    }
  }
  amax = block_max(amax, scratch);
  const float scale = fmaxf(amax, 1e-8f) / kFp8Max;
  if (threadIdx.x == 0) out_scale[row] = scale;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = (j * THREADS + threadIdx.x) * 8;
    if (i < inter) *reinterpret_cast<uint2*>(out_q + (size_t)row * inter + i) = pack8_e4m3(v[j], scale);
  }
}

template <typename T>
static int launch_act_quant(const void* x, void* out_q, void* out_scale, int rows, int inter, int kind,
                            cudaStream_t s) {
  // few rows (decode): 512 threads per row keep more loads in flight per row; many rows
  // (prefill): 128 threads, rows in flight come from the grid
  const bool wide = rows <= 2048 && inter >= 4096;
  const int threads = wide ? 512 : kRowThreads;
  const int vpt = (inter / 8 + threads - 1) / threads;
#define ACT_LAUNCH(V, TH) \
  msgl_launch(act_mul_quant_kernel<T, V, TH>, dim3(rows), dim3(TH), 0, s, (const T*)x, (uint8_t*)out_q, (float*)out_scale, inter, kind)
  if (wide) {
    if (vpt <= 1) ACT_LAUNCH(1, 512);
    else if (vpt <= 2) ACT_LAUNCH(2, 512);
    else if (vpt <= 3) ACT_LAUNCH(3, 512);
    else if (vpt <= 4) ACT_LAUNCH(4, 512);
    else if (vpt <= 7) ACT_LAUNCH(7, 512);
    else return MSGL_BAD_ARG;
    return MSGL_OK;
  }
  if (inter >= 2048) {
    // many long rows (prefill): 256 threads per row halve the registers a thread holds between the
    // two passes, which doubles the resident warps
    const int v256 = (inter / 8 + 255) / 256;
    if (v256 <= 1) ACT_LAUNCH(1, 256);
    else if (v256 <= 2) ACT_LAUNCH(2, 256);
    else if (v256 <= 3) ACT_LAUNCH(3, 256);
    else if (v256 <= 5) ACT_LAUNCH(5, 256);
    else if (v256 <= 8) ACT_LAUNCH(8, 256);
    else if (v256 <= 14) ACT_LAUNCH(14, 256);
    else return MSGL_BAD_ARG;
    return MSGL_OK;
  }
  if (vpt <= 1) ACT_LAUNCH(1, kRowThreads);
  else if (vpt <= 2) ACT_LAUNCH(2, kRowThreads);
  else if (vpt <= 4) ACT_LAUNCH(4, kRowThreads);
  else return MSGL_BAD_ARG;
#undef ACT_LAUNCH
  return MSGL_OK;
}

MSGL_API int msgl_act_and_mul(const void* x, void* out, void* out_q, void* out_scale, int rows, int inter,
                              int kind, int dtype, cudaStream_t stream) {
  if (inter % 8) return MSGL_BAD_ARG;
  if (rows == 0) return MSGL_OK;
  if (out_q == nullptr) {
    size_t vecs = (size_t)rows * (inter / 8);
    int threads = 256;
    unsigned blocks = (unsigned)((vecs + threads - 1) / threads);
    if (dtype == MSGL_BF16)
      msgl_launch(act_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)out,
                                                                    inter, vecs, kind);
    else if (dtype == MSGL_F16)
      msgl_launch(act_mul_kernel<__half>, dim3(blocks), dim3(threads), 0, stream, (const __half*)x, (__half*)out, inter, vecs, kind);
    else
      return MSGL_BAD_ARG;
  } else {
    int rc;
    if (dtype == MSGL_BF16) rc = launch_act_quant<__nv_bfloat16>(x, out_q, out_scale, rows, inter, kind, stream);
    else if (dtype == MSGL_F16) rc = launch_act_quant<__half>(x, out_q, out_scale, rows, inter, kind, stream);
    else return MSGL_BAD_ARG;
    if (rc) return rc;
  }
  MSGL_CHECK_LAUNCH("act_and_mul");
  return MSGL_OK;
}

// ------------------------------------------------------------------------------------------
// stand-alone activation quantisers: per token (group == hidden) or per `group` elements
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void quant_group_kernel(const T* __restrict__ x, uint8_t* __restrict__ out_q,
                                   float* __restrict__ out_scale, int group, size_t total_groups) {
  pdl_enter();
  // one warp per group; groups are contiguous runs of `group` elements (group % 8 == 0)
  const size_t gidx = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gidx >= total_groups) return;
  const int lane = threadIdx.x & 31;
  const T* src = x + gidx * group;
  float amax = 0.f;
  for (int i = lane * 8; i < group; i += 256) {
    float v[8];
    load8(src + i, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(v[k]));
  }
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-8f) / kFp8Max;
  if (lane == 0) out_scale[gidx] = scale;
  for (int i = lane * 8; i < group; i += 256) {
    float v[8];
    load8(src + i, v);
    *reinterpret_cast<uint2*>(out_q + gidx * group + i) = pack8_e4m3(v, scale);
  }
}

MSGL_API int msgl_quant_fp8(const void* x, void* out_q, void* out_scale, int rows, int hidden, int group,
                            int dtype, cudaStream_t stream) {
  if (group <= 0) group = hidden;
  if (hidden % group || group % 8) return MSGL_BAD_ARG;
  if (rows == 0) return MSGL_OK;
  size_t total = (size_t)rows * (hidden / group);
  int warps = 8;
  unsigned blocks = (unsigned)((total + warps - 1) / warps);
  if (dtype == MSGL_BF16)
    msgl_launch(quant_group_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), 0, stream, (const __nv_bfloat16*)x, (uint8_t*)out_q,
                                                                        (float*)out_scale, group, total);
  else if (dtype == MSGL_F16)
    msgl_launch(quant_group_kernel<__half>, dim3(blocks), dim3(warps * 32), 0, stream, (const __half*)x, (uint8_t*)out_q,
                                                                 (float*)out_scale, group, total);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("quant_fp8");
  return MSGL_OK;
}


// ---------------------------------------------------------------------------------- bounds-check report
#ifdef MSGL_CHECK_BOUNDS
namespace {
constexpr int kMaxCollectors = 64;
msgl_bounds_collect_fn g_collectors[kMaxCollectors];
int g_num_collectors = 0;
}  // namespace
void msgl_bounds_register(msgl_bounds_collect_fn fn) {
  if (g_num_collectors < kMaxCollectors) g_collectors[g_num_collectors++] = fn;
}
#endif

// 1 when this library was built with the device-side bounds checks.
MSGL_API int msgl_bounds_enabled() {
#ifdef MSGL_CHECK_BOUNDS
  return 1;
#else
  return 0;
#endif
}

// Collects (and clears) the out-of-range indices the kernels of this library have recorded on the
// current device since the last call. Writes up to `max_lines` text lines of `line_bytes` bytes each
// ("file.cu:LINE value V limit L") into `text`; returns the number of records. Synchronises the device.
MSGL_API int msgl_bounds_report(char* text, int max_lines, int line_bytes) {
#ifdef MSGL_CHECK_BOUNDS
  cudaDeviceSynchronize();
  int total = 0;
  for (int c = 0; c < g_num_collectors; ++c) {
    const char* file = "";
    msgl::BoundsRecord recs[msgl::kBoundsRing];
    const int n = g_collectors[c](&file, recs, msgl::kBoundsRing);
    const char* base = file;
    for (const char* p = file; *p; ++p)
      if (*p == '/') base = p + 1;
    for (int i = 0; i < n; ++i) {
      if (total < max_lines && text != nullptr)
        snprintf(text + (size_t)total * line_bytes, line_bytes, "%s:%d value %lld limit %lld", base, recs[i].line,
                 recs[i].value, recs[i].limit);
      ++total;
    }
  }
  return total;
#else
  (void)text; (void)max_lines; (void)line_bytes;
  return 0;
#endif
}
