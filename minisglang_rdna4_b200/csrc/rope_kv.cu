// Fused per-head QK-RMSNorm + rotary embedding + paged KV store, and a stand-alone KV store.
//
// Replaces the reference's tail_hip.qk_norm_rope / rope / store_kv
// (python/minisgl/layers/attention.py:137-141, python/minisgl/layers/rotary.py:104-129,
// python/minisgl/kvcache/mha_pool.py:189-192) and the upstream store kernel
// (python/minisgl/kernel/csrc/jit/store.cu:25-53) with one pass over the QKV projection:
// q heads are normed, rotated and written to a packed [T, Hq, D] buffer; k heads are normed,
// rotated and scattered into the paged pool; v heads are scattered. The pool layout is
// [pages, Hk, page_size, D]; with fp8 storage a row is divided by its per-head descale and
// saturated to e4m3.
#include "common.cuh"

using namespace msgl;

// One warp per (token, head). The head row is staged in shared memory as fp32.
template <typename T, int D>
__global__ void __launch_bounds__(128) qk_norm_rope_store_kernel(
    const T* __restrict__ qkv, const T* __restrict__ q_w, const T* __restrict__ k_w,
    const int32_t* __restrict__ positions, const float* __restrict__ cos_sin, T* __restrict__ q_out,
    void* __restrict__ k_cache, void* __restrict__ v_cache, const int32_t* __restrict__ out_loc,
    const float* __restrict__ k_scale, const float* __restrict__ v_scale, int hq, int hk, int rot,
    int page_size, float eps, int interleaved, int cache_fp8, int max_pos, int num_slots) {
  __shared__ float rows[4][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.x;
  const int head = blockIdx.y * 4 + warp;
  const int heads_total = hq + 2 * hk;
  if (head >= heads_total) return;
  constexpr int PER = D / 32;
  float* row = rows[warp];
  const T* src = qkv + (size_t)token * heads_total * D + (size_t)head * D;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    float v = to_float(src[lane * PER + i]);
    row[lane * PER + i] = v;
    ss += v * v;
  }
  const bool is_q = head < hq, is_k = !is_q && head < hq + hk;
  const T* w = is_q ? q_w : k_w;
  if (!(is_q || is_k)) {
    // V head: straight scatter
  } else {
    if (w != nullptr) {
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        int d = lane * PER + i;
        // the normed value is rounded to T before the rotation, as the unfused ops would
        row[d] = to_float(from_float<T>(row[d] * rstd * to_float(w[d])));
      }
    }
    __syncwarp();
    int pos = positions[token];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + (size_t)pos * rot;
    const int half = rot >> 1;
    // each lane rotates pairs p = lane, lane + 32, ...
    for (int p = lane; p < half; p += 32) {
      const float c = cs[p], s = cs[half + p];
      const int i0 = interleaved ? 2 * p : p, i1 = interleaved ? 2 * p + 1 : p + half;
      const float a = row[i0], b = row[i1];
      row[i0] = a * c - b * s;
      row[i1] = b * c + a * s;
    }
  }
  __syncwarp();
  if (is_q) {
    T* dst = q_out + ((size_t)token * hq + head) * D;
#pragma unroll
    for (int i = 0; i < PER; ++i) dst[lane * PER + i] = from_float<T>(row[lane * PER + i]);
    return;
  }
  const int kvh = is_k ? head - hq : head - hq - hk;
  int slot = out_loc[token];
  if (slot < 0 || slot >= num_slots) return;  // padded row: nothing to store
  const int page = slot / page_size, off = slot % page_size;
  const size_t base = (((size_t)page * hk + kvh) * page_size + off) * D;
  void* cache = is_k ? k_cache : v_cache;
  if (cache_fp8) {
    const float sc = is_k ? k_scale[kvh] : v_scale[kvh];
    uint8_t* dst = (uint8_t*)cache + base;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      dst[lane * PER + i] = float_to_e4m3(to_float(from_float<T>(row[lane * PER + i])) / sc);
  } else {
    T* dst = (T*)cache + base;
#pragma unroll
    for (int i = 0; i < PER; ++i) dst[lane * PER + i] = from_float<T>(row[lane * PER + i]);
  }
}

MSGL_API int msgl_qk_norm_rope_store(const void* qkv, const void* q_w, const void* k_w, const void* positions,
                                     const void* cos_sin, void* q_out, void* k_cache, void* v_cache,
                                     const void* out_loc, const void* k_scale, const void* v_scale, int tokens,
                                     int hq, int hk, int head_dim, int rot, int page_size, float eps,
                                     int interleaved, int cache_fp8, int max_pos, int num_slots, int dtype,
                                     cudaStream_t stream) {
  if (tokens == 0) return MSGL_OK;
  if (rot > head_dim || rot % 2) return MSGL_BAD_ARG;
  dim3 grid(tokens, (hq + 2 * hk + 3) / 4);
#define LAUNCH(T, D)                                                                                        \
  qk_norm_rope_store_kernel<T, D><<<grid, 128, 0, stream>>>(                                                \
      (const T*)qkv, (const T*)q_w, (const T*)k_w, (const int32_t*)positions, (const float*)cos_sin,        \
      (T*)q_out, k_cache, v_cache, (const int32_t*)out_loc, (const float*)k_scale, (const float*)v_scale,   \
      hq, hk, rot, page_size, eps, interleaved, cache_fp8, max_pos, num_slots)
  if (dtype == MSGL_BF16) {
    if (head_dim == 128) LAUNCH(__nv_bfloat16, 128);
    else if (head_dim == 64) LAUNCH(__nv_bfloat16, 64);
    else if (head_dim == 256) LAUNCH(__nv_bfloat16, 256);
    else return MSGL_BAD_ARG;
  } else if (dtype == MSGL_F16) {
    if (head_dim == 128) LAUNCH(__half, 128);
    else if (head_dim == 64) LAUNCH(__half, 64);
    else if (head_dim == 256) LAUNCH(__half, 256);
    else return MSGL_BAD_ARG;
  } else {
    return MSGL_BAD_ARG;
  }
#undef LAUNCH
  MSGL_CHECK_LAUNCH("qk_norm_rope_store");
  return MSGL_OK;
}

// ------------------------------------------------------------------------------------------
// stand-alone store: k, v [T, Hk, D] -> paged pool
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void store_kv_kernel(const T* __restrict__ k, const T* __restrict__ v, void* __restrict__ k_cache,
                                void* __restrict__ v_cache, const int32_t* __restrict__ out_loc,
                                const float* __restrict__ k_scale, const float* __restrict__ v_scale, int hk,
                                int d, int page_size, int cache_fp8, int num_slots) {
  const int token = blockIdx.x;
  const int slot = out_loc[token];
  if (slot < 0 || slot >= num_slots) return;
  const int page = slot / page_size, off = slot % page_size;
  for (int i = threadIdx.x; i < hk * d; i += blockDim.x) {
    const int h = i / d, e = i % d;
    const size_t dst = (((size_t)page * hk + h) * page_size + off) * d + e;
    const float kv = to_float(k[(size_t)token * hk * d + i]), vv = to_float(v[(size_t)token * hk * d + i]);
    if (cache_fp8) {
      ((uint8_t*)k_cache)[dst] = float_to_e4m3(kv / k_scale[h]);
      ((uint8_t*)v_cache)[dst] = float_to_e4m3(vv / v_scale[h]);
    } else {
      ((T*)k_cache)[dst] = from_float<T>(kv);
      ((T*)v_cache)[dst] = from_float<T>(vv);
    }
  }
}

MSGL_API int msgl_store_kv(const void* k, const void* v, void* k_cache, void* v_cache, const void* out_loc,
                           const void* k_scale, const void* v_scale, int tokens, int hk, int head_dim,
                           int page_size, int cache_fp8, int num_slots, int dtype, cudaStream_t stream) {
  if (tokens == 0) return MSGL_OK;
  if (dtype == MSGL_BF16)
    store_kv_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(
        (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, k_cache, v_cache, (const int32_t*)out_loc,
        (const float*)k_scale, (const float*)v_scale, hk, head_dim, page_size, cache_fp8, num_slots);
  else if (dtype == MSGL_F16)
    store_kv_kernel<__half><<<tokens, 256, 0, stream>>>(
        (const __half*)k, (const __half*)v, k_cache, v_cache, (const int32_t*)out_loc, (const float*)k_scale,
        (const float*)v_scale, hk, head_dim, page_size, cache_fp8, num_slots);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("store_kv");
  return MSGL_OK;
}
