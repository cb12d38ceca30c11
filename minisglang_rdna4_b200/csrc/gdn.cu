// Gated delta net (the linear-attention mixer of the Qwen3.5 / Qwen3-Next hybrid family):
// depthwise causal convolution with a per-request rolling state, the gated delta rule with a
// per-(request, head) recurrent state matrix, and the gated RMSNorm of its output. Replaces the
// reference's gdn_hip package (causal_conv1d_fwd / _update, gdn_prefill / gdn_decode,
// rmsnorm_gated; python/minisgl/gdn/layer.py:346-760, python/minisgl/kvcache/gdn_state.py:128-372).
//
// One code path serves prefill chunks, decode and multi-token verification: sequences are packed
// rows described by cu_q, every sequence owns a state slot, and a sequence without a state yet
// (has_state == 0) starts from zeros.
#include "common.cuh"

using namespace msgl;

namespace {

// ------------------------------------------------------------------------------------------
// Causal depthwise conv1d + SiLU. One thread per channel walks its sequence with the last KW-1
// inputs in registers (loads of consecutive tokens are independent, so they pipeline); channels
// of a CTA are contiguous, so every load / store is coalesced. grid = (ceil(C / 128), B).
// ------------------------------------------------------------------------------------------
template <typename T, int KW>
__global__ void __launch_bounds__(128) gdn_conv1d_kernel(const T* __restrict__ x, long long ldx,
                                                         const T* __restrict__ w, T* __restrict__ state,
                                                         const int32_t* __restrict__ cu_q,
                                                         const int32_t* __restrict__ slots,
                                                         const int32_t* __restrict__ has_state, T* __restrict__ out,
                                                         int channels, const T* __restrict__ bias) {
  pdl_enter();
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= channels) return;
  const int b = blockIdx.y;
  const int lo = cu_q[b], hi = cu_q[b + 1];
  if (hi <= lo) return;
  T* st = state + ((size_t)slots[b] * channels + c) * (KW - 1);
  float hist[KW - 1];
  const bool keep = has_state[b] != 0;
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) hist[j] = keep ? to_float(st[j]) : 0.f;
  float wv[KW];
#pragma unroll
  for (int j = 0; j < KW; ++j) wv[j] = to_float(w[(size_t)c * KW + j]);
  const float bv = bias != nullptr ? to_float(bias[c]) : 0.f;
#pragma unroll 4
  for (int t = lo; t < hi; ++t) {
    const float cur = to_float(x[(size_t)t * ldx + c]);
    float acc = fmaf(cur, wv[KW - 1], bv);
#pragma unroll
    for (int j = 0; j < KW - 1; ++j) acc = fmaf(hist[j], wv[j], acc);
#pragma unroll
    for (int j = 0; j < KW - 2; ++j) hist[j] = hist[j + 1];
    hist[KW - 2] = cur;
    const float h = 0.5f * acc;   // silu(acc) = h + h * tanh(h)
    out[(size_t)t * channels + c] = from_float<T>(fmaf(h, tanhf(h), h));
  }
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) st[j] = from_float<T>(hist[j]);
}

// ------------------------------------------------------------------------------------------
// Gated delta rule, recurrent form. grid = (Hv, B), block = DV threads: thread t owns column t
// of the state matrix S [DK][DV] in registers, so the three passes over S per token (decay +
// S^T k, rank-one update, S^T q) need no exchange between threads; q and k (L2-normalised here)
// are broadcast through shared memory.
//   qkv    [T, 2 * Hk * DK + Hv * DV]  rows after the convolution: q heads, k heads, v heads
//   a, b   [T, Hv] (row stride ld_ab)  raw gate projections
//   state  [slots, Hv, DK, DV] fp32
//   out    [T, Hv, DV]
// ------------------------------------------------------------------------------------------
template <typename T, int DK, int DV>
__global__ void __launch_bounds__(DV) gdn_recurrent_kernel(const T* __restrict__ qkv, const T* __restrict__ a,
                                                           const T* __restrict__ bgate, long long ld_ab,
                                                           const float* __restrict__ a_log,
                                                           const float* __restrict__ dt_bias,
                                                           float* __restrict__ state,
                                                           const int32_t* __restrict__ cu_q,
                                                           const int32_t* __restrict__ slots,
                                                           const int32_t* __restrict__ has_state,
                                                           T* __restrict__ out, int Hk, int Hv) {
  pdl_enter();
  static_assert(DK == DV, "one thread per state column, and per q / k element");
  __shared__ float s_q[2][DK];
  __shared__ float s_k[2][DK];
  __shared__ float s_red[2][2][DV / 32];
  const int h = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x;
  const int lo = cu_q[b], hi = cu_q[b + 1];
  if (hi <= lo) return;
  const int hk = h / (Hv / Hk);
  const int row_w = 2 * Hk * DK + Hv * DV;
  float* S = state + (((size_t)slots[b] * Hv + h) * DK) * DV + tid;
  float s[DK];
  if (has_state[b] != 0) {
#pragma unroll
    for (int i = 0; i < DK; ++i) s[i] = S[(size_t)i * DV];
  } else {
#pragma unroll
    for (int i = 0; i < DK; ++i) s[i] = 0.f;
  }
  const float neg_a = -__expf(a_log[h]);
  const float dtb = dt_bias[h];
  const float q_scale = rsqrtf((float)DK);
  int buf = 0;
  for (int t = lo; t < hi; ++t, buf ^= 1) {
    const T* row = qkv + (size_t)t * row_w;
    const float qv = to_float(row[hk * DK + tid]);
    const float kv_in = to_float(row[Hk * DK + hk * DK + tid]);
    const float vv = to_float(row[2 * Hk * DK + h * DV + tid]);
    // L2 norms of q and k over the head dimension
    float q2 = warp_sum(qv * qv), k2 = warp_sum(kv_in * kv_in);
    if ((tid & 31) == 0) {
      s_red[buf][0][tid >> 5] = q2;
      s_red[buf][1][tid >> 5] = k2;
    }
    s_q[buf][tid] = qv;
    s_k[buf][tid] = kv_in;
    __syncthreads();   // one barrier per token: the buffers alternate
    q2 = 0.f;
    k2 = 0.f;
#pragma unroll
    for (int i = 0; i < DV / 32; ++i) {
      q2 += s_red[buf][0][i];
      k2 += s_red[buf][1][i];
    }
    const float qn = rsqrtf(q2 + 1e-6f) * q_scale, kn = rsqrtf(k2 + 1e-6f);
    const float av = to_float(a[(size_t)t * ld_ab + h]) + dtb;
    const float sp = av > 20.f ? av : log1pf(__expf(av));      // softplus
    const float decay = __expf(neg_a * sp);
    const float beta = 1.f / (1.f + __expf(-to_float(bgate[(size_t)t * ld_ab + h])));
    float mem = 0.f;
#pragma unroll
    for (int i = 0; i < DK; ++i) mem = fmaf(s[i], s_k[buf][i], mem);
    const float delta = (vv - decay * kn * mem) * beta;
    const float kd = kn * delta;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      s[i] = fmaf(s[i], decay, s_k[buf][i] * kd);
      o = fmaf(s[i], s_q[buf][i], o);
    }
    out[((size_t)t * Hv + h) * DV + tid] = from_float<T>(o * qn);
  }
#pragma unroll
  for (int i = 0; i < DK; ++i) S[(size_t)i * DV] = s[i];
}

// out[r, :] = rmsnorm(x[r, :]) * w * silu(z[r, :]) over rows of D elements; one warp per row.
template <typename T>
__global__ void rms_norm_gated_kernel(const T* __restrict__ x, const T* __restrict__ z, long long ldz, int heads,
                                      const T* __restrict__ w, T* __restrict__ out, int rows, int D, float eps) {
  pdl_enter();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const T* xr = x + (size_t)r * D;
  const T* zr = z + (size_t)(r / heads) * ldz + (size_t)(r % heads) * D;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    const float v = to_float(xr[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)D + eps);
  for (int i = lane; i < D; i += 32) {
    const float y = to_float(from_float<T>(to_float(xr[i]) * rstd));   // rounded before the weight, as the model does
    const float g = to_float(zr[i]);
    out[(size_t)r * D + i] = from_float<T>(to_float(w[i]) * y * (g / (1.f + __expf(-g))));
  }
}

}  // namespace

// x [T, channels] with row stride ldx, w [channels, kw], state [slots, channels, kw - 1], out [T, channels];
// bias [channels] or null
MSGL_API int msgl_gdn_conv1d(const void* x, long long ldx, const void* w, void* state, const void* cu_q,
                             const void* slots, const void* has_state, void* out, int B, int channels, int kw,
                             const void* bias, int dtype, cudaStream_t stream) {
  if (B <= 0 || channels <= 0) return B == 0 ? MSGL_OK : MSGL_BAD_ARG;
  if (kw != 4) {
    msgl_set_error_text("gdn_conv1d: only a kernel of 4 taps is built");
    return MSGL_BAD_ARG;
  }
  dim3 grid((channels + 127) / 128, B);
  if (dtype == MSGL_BF16)
    msgl_launch(gdn_conv1d_kernel<__nv_bfloat16, 4>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)x, ldx,
                (const __nv_bfloat16*)w, (__nv_bfloat16*)state, (const int32_t*)cu_q, (const int32_t*)slots,
                (const int32_t*)has_state, (__nv_bfloat16*)out, channels, (const __nv_bfloat16*)bias);
  else if (dtype == MSGL_F16)
    msgl_launch(gdn_conv1d_kernel<__half, 4>, grid, dim3(128), 0, stream, (const __half*)x, ldx, (const __half*)w,
                (__half*)state, (const int32_t*)cu_q, (const int32_t*)slots, (const int32_t*)has_state, (__half*)out,
                channels, (const __half*)bias);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("gdn_conv1d");
  return MSGL_OK;
}

MSGL_API int msgl_gdn_recurrent(const void* qkv, const void* a, const void* bgate, long long ld_ab, const void* a_log,
                                const void* dt_bias, void* state, const void* cu_q, const void* slots,
                                const void* has_state, void* out, int B, int Hk, int Hv, int dk, int dv, int dtype,
                                cudaStream_t stream) {
  if (B <= 0) return B == 0 ? MSGL_OK : MSGL_BAD_ARG;
  if (dk != dv || (dk != 128 && dk != 64) || Hk <= 0 || Hv % Hk) {
    msgl_set_error_text("gdn_recurrent: built for key / value head dims 64 and 128 (equal), Hv a multiple of Hk");
    return MSGL_BAD_ARG;
  }
  dim3 grid(Hv, B);
#define GDN_LAUNCH(T, D)                                                                                        \
  msgl_launch(gdn_recurrent_kernel<T, D, D>, grid, dim3(D), 0, stream, (const T*)qkv, (const T*)a, (const T*)bgate, \
              ld_ab, (const float*)a_log, (const float*)dt_bias, (float*)state, (const int32_t*)cu_q,            \
              (const int32_t*)slots, (const int32_t*)has_state, (T*)out, Hk, Hv)
  if (dtype == MSGL_BF16) {
    if (dk == 128) GDN_LAUNCH(__nv_bfloat16, 128); else GDN_LAUNCH(__nv_bfloat16, 64);
  } else if (dtype == MSGL_F16) {
    if (dk == 128) GDN_LAUNCH(__half, 128); else GDN_LAUNCH(__half, 64);
  } else {
    return MSGL_BAD_ARG;
  }
#undef GDN_LAUNCH
  MSGL_CHECK_LAUNCH("gdn_recurrent");
  return MSGL_OK;
}

// x [rows, D] contiguous (rows = tokens * heads); z [tokens, ...] with row stride ldz holding heads * D gate values
MSGL_API int msgl_rms_norm_gated(const void* x, const void* z, long long ldz, int heads, const void* w, void* out,
                                 int rows, int D, float eps, int dtype, cudaStream_t stream) {
  if (rows <= 0) return rows == 0 ? MSGL_OK : MSGL_BAD_ARG;
  const int warps = 8;
  dim3 grid((rows + warps - 1) / warps);
  if (dtype == MSGL_BF16)
    msgl_launch(rms_norm_gated_kernel<__nv_bfloat16>, grid, dim3(warps * 32), 0, stream, (const __nv_bfloat16*)x,
                (const __nv_bfloat16*)z, ldz, heads, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, rows, D, eps);
  else if (dtype == MSGL_F16)
    msgl_launch(rms_norm_gated_kernel<__half>, grid, dim3(warps * 32), 0, stream, (const __half*)x, (const __half*)z,
                ldz, heads, (const __half*)w, (__half*)out, rows, D, eps);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("rms_norm_gated");
  return MSGL_OK;
}
