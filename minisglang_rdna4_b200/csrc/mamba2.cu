// Mamba-2 mixer kernels (the state-space layers of the Nemotron-H hybrid family): the selective
// state-space recurrence with a per-(request, head) state, the gate-first grouped RMSNorm of its
// output, and the squared-ReLU activation of the family's non-gated MLPs. The depthwise causal
// convolution in front of the recurrence is the one in gdn.cu (with a bias). Replaces the
// reference's mamba2 package (python/minisgl/mamba2/: causal_conv1d_fwd / _update, selective scan
// prefill / decode, rmsnorm_gated).
//
// One code path serves prefill chunks, decode and multi-token verification: sequences are packed
// rows described by cu_q, every sequence owns a state slot, and a sequence without a state yet
// (has_state == 0) starts from zeros.
#include "common.cuh"

using namespace msgl;

namespace {

// ------------------------------------------------------------------------------------------
// Selective scan, recurrent form. grid = (H, B), block = P threads: thread p owns row p of the
// head's state S [P][N] in registers, so the decay, the rank-one update and the read-out S C need
// no exchange between threads; B_t and C_t (shared by the H / G heads of a group) are broadcast
// through shared memory, two tokens deep so that the loads of token t + 1 overlap the math of t.
//   xbc   [T, H * P + 2 * G * N]  rows after the convolution: x heads, B groups, C groups
//   dt    [T, H] (row stride ld_dt)  raw step sizes
//   state [slots, H, P, N] fp32
//   out   [T, H, P]
//   dt' = max(softplus(dt + dt_bias), dt_min);  S = S exp(-exp(A_log) dt') + dt' x (x) B;  y = S C + D x
// ------------------------------------------------------------------------------------------
template <typename T, int P, int N>
__global__ void __launch_bounds__(P) mamba2_scan_kernel(const T* __restrict__ xbc, const T* __restrict__ dt,
                                                        long long ld_dt, const float* __restrict__ a_log,
                                                        const float* __restrict__ d_skip,
                                                        const float* __restrict__ dt_bias, float* __restrict__ state,
                                                        const int32_t* __restrict__ cu_q,
                                                        const int32_t* __restrict__ slots,
                                                        const int32_t* __restrict__ has_state, T* __restrict__ out,
                                                        int H, int G, float dt_min) {
  pdl_enter();
  __shared__ float bc[2][2 * N];
  const int h = blockIdx.x, b = blockIdx.y, p = threadIdx.x;
  const int lo = cu_q[b], hi = cu_q[b + 1];
  if (hi <= lo) return;
  const int g = h / (H / G);
  const int row = H * P + 2 * G * N;
  float* S = state + (((size_t)slots[b] * H + h) * P + p) * N;
  float s[N];
  const bool keep = has_state[b] != 0;
#pragma unroll
  for (int n = 0; n < N; ++n) s[n] = keep ? S[n] : 0.f;
  const float A = -__expf(a_log[h]), D = d_skip[h], bias = dt_bias[h];
  auto stage = [&](int t, int buf) {
    const T* r = xbc + (size_t)t * row + H * P + g * N;        // B of the group, then C at + G * N
    for (int i = p; i < 2 * N; i += P) bc[buf][i] = to_float(i < N ? r[i] : r[G * N + i - N]);
  };
  stage(lo, 0);
  __syncthreads();
  for (int t = lo; t < hi; ++t) {
    const int cur = (t - lo) & 1;
    if (t + 1 < hi) stage(t + 1, cur ^ 1);
    const float x = to_float(xbc[(size_t)t * row + h * P + p]);
    const float raw = to_float(dt[(size_t)t * ld_dt + h]) + bias;
    const float step = fmaxf(raw > 20.f ? raw : log1pf(__expf(raw)), dt_min);
    const float decay = __expf(step * A), dx = step * x;
    float y = 0.f;
#pragma unroll
    for (int n = 0; n < N; ++n) {
      s[n] = fmaf(s[n], decay, dx * bc[cur][n]);
      y = fmaf(s[n], bc[cur][N + n], y);
    }
    out[((size_t)t * H + h) * P + p] = from_float<T>(fmaf(D, x, y));
    __syncthreads();
  }
#pragma unroll
  for (int n = 0; n < N; ++n) S[n] = s[n];
}

// out[r, :] = w * norm_group(x[r, :] * silu(z[r, :])): one warp per (row, group of `group` channels).
template <typename T>
__global__ void rms_norm_gate_first_kernel(const T* __restrict__ x, const T* __restrict__ z, long long ldz,
                                           const T* __restrict__ w, T* __restrict__ out, int rows, int D, int group,
                                           float eps) {
  pdl_enter();
  const int groups = D / group;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= rows * groups) return;
  const int r = item / groups, gi = item % groups;
  const int lane = threadIdx.x & 31;
  const T* xr = x + (size_t)r * D + gi * group;
  const T* zr = z + (size_t)r * ldz + gi * group;
  float ss = 0.f;
  for (int i = lane; i < group; i += 32) {
    const float g = to_float(zr[i]);
    const float v = to_float(xr[i]) * (g / (1.f + __expf(-g)));
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)group + eps);
  for (int i = lane; i < group; i += 32) {
    const float g = to_float(zr[i]);
    const float v = to_float(xr[i]) * (g / (1.f + __expf(-g)));
    const float y = to_float(from_float<T>(v * rstd));          // rounded before the weight, as the model does
    out[(size_t)r * D + gi * group + i] = from_float<T>(to_float(w[gi * group + i]) * y);
  }
}

template <typename T>
__global__ void relu2_kernel(const T* __restrict__ x, T* __restrict__ out, size_t n_vec) {
  pdl_enter();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  float v[8];
  load8(x + i * 8, v);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float r = fmaxf(v[e], 0.f);
    v[e] = r * r;
  }
  store8(out + i * 8, v);
}

}  // namespace

MSGL_API int msgl_mamba2_scan(const void* xbc, const void* dt, long long ld_dt, const void* a_log, const void* d_skip,
                              const void* dt_bias, void* state, const void* cu_q, const void* slots,
                              const void* has_state, void* out, int B, int H, int G, int P, int N, float dt_min,
                              int dtype, cudaStream_t stream) {
  if (B <= 0) return B == 0 ? MSGL_OK : MSGL_BAD_ARG;
  if (H <= 0 || G <= 0 || H % G) return MSGL_BAD_ARG;
  dim3 grid(H, B);
#define SCAN(T, P_, N_)                                                                                          \
  msgl_launch(mamba2_scan_kernel<T, P_, N_>, grid, dim3(P_), 0, stream, (const T*)xbc, (const T*)dt, ld_dt,      \
              (const float*)a_log, (const float*)d_skip, (const float*)dt_bias, (float*)state,                   \
              (const int32_t*)cu_q, (const int32_t*)slots, (const int32_t*)has_state, (T*)out, H, G, dt_min)
#define SCAN_T(T)                                                                                                \
  do {                                                                                                           \
    if (P == 64 && N == 128) SCAN(T, 64, 128);                                                                   \
    else if (P == 64 && N == 64) SCAN(T, 64, 64);                                                                \
    else if (P == 32 && N == 16) SCAN(T, 32, 16);                                                                \
    else if (P == 128 && N == 128) SCAN(T, 128, 128);                                                            \
    else {                                                                                                       \
      msgl_set_error_text("mamba2_scan: built for (head dim, state) = (64, 128), (64, 64), (128, 128), (32, 16)"); \
      return MSGL_BAD_ARG;                                                                                       \
    }                                                                                                            \
  } while (0)
  if (dtype == MSGL_BF16) SCAN_T(__nv_bfloat16);
  else if (dtype == MSGL_F16) SCAN_T(__half);
  else return MSGL_BAD_ARG;
#undef SCAN_T
#undef SCAN
  MSGL_CHECK_LAUNCH("mamba2_scan");
  return MSGL_OK;
}

// x [rows, D] contiguous, z [rows, D] with row stride ldz, w [D]; RMS over groups of `group` channels
MSGL_API int msgl_rms_norm_gate_first(const void* x, const void* z, long long ldz, const void* w, void* out, int rows,
                                      int D, int group, float eps, int dtype, cudaStream_t stream) {
  if (rows <= 0) return rows == 0 ? MSGL_OK : MSGL_BAD_ARG;
  if (group <= 0 || D % group) return MSGL_BAD_ARG;
  const int warps = 8;
  const long long items = (long long)rows * (D / group);
  dim3 grid((unsigned)((items + warps - 1) / warps));
  if (dtype == MSGL_BF16)
    msgl_launch(rms_norm_gate_first_kernel<__nv_bfloat16>, grid, dim3(warps * 32), 0, stream, (const __nv_bfloat16*)x,
                (const __nv_bfloat16*)z, ldz, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, rows, D, group, eps);
  else if (dtype == MSGL_F16)
    msgl_launch(rms_norm_gate_first_kernel<__half>, grid, dim3(warps * 32), 0, stream, (const __half*)x,
                (const __half*)z, ldz, (const __half*)w, (__half*)out, rows, D, group, eps);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("rms_norm_gate_first");
  return MSGL_OK;
}

MSGL_API int msgl_relu2(const void* x, void* out, long long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return n == 0 ? MSGL_OK : MSGL_BAD_ARG;
  if (n % 8) return MSGL_BAD_ARG;
  const size_t n_vec = (size_t)n / 8;
  dim3 grid((unsigned)((n_vec + 255) / 256));
  if (dtype == MSGL_BF16)
    msgl_launch(relu2_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)out,
                n_vec);
  else if (dtype == MSGL_F16)
    msgl_launch(relu2_kernel<__half>, grid, dim3(256), 0, stream, (const __half*)x, (__half*)out, n_vec);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("relu2");
  return MSGL_OK;
}
