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
  pdl_enter();
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
    (void)MSGL_OOB(pos, max_pos);
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
  if (slot >= 0) (void)MSGL_OOB(slot, num_slots);
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

// E consecutive 16-bit elements as one access (E = 1, 2 or 4)
template <typename T, int E> __device__ __forceinline__ void load_run(const T* p, float (&out)[E]) {
  if constexpr (E == 1) {
    out[0] = to_float(p[0]);
  } else if constexpr (E == 2) {
    typename Pack2<T>::type v = *reinterpret_cast<const typename Pack2<T>::type*>(p);
    float2 f = to_float2(v);
    out[0] = f.x; out[1] = f.y;
  } else {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    float2 f0 = to_float2(*reinterpret_cast<typename Pack2<T>::type*>(&raw.x));
    float2 f1 = to_float2(*reinterpret_cast<typename Pack2<T>::type*>(&raw.y));
    out[0] = f0.x; out[1] = f0.y; out[2] = f1.x; out[3] = f1.y;
  }
}
template <typename T, int E> __device__ __forceinline__ void store_run(T* p, const float (&in)[E]) {
  if constexpr (E == 1) {
    p[0] = from_float<T>(in[0]);
  } else if constexpr (E == 2) {
    *reinterpret_cast<typename Pack2<T>::type*>(p) = Pack2<T>::make(in[0], in[1]);
  } else {
    typename Pack2<T>::type lo = Pack2<T>::make(in[0], in[1]), hi = Pack2<T>::make(in[2], in[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  }
}

// Fast path for full rotary (rot == D): no shared memory. A lane owns E = D/64 elements of each
// half of the head (NeoX pairing i <-> i + D/2) or 2E consecutive elements (interleaved pairing),
// so both members of every rotation pair live in the same lane; the per-head RMS statistic is a
// warp reduction.
template <typename T, int D>
__global__ void __launch_bounds__(128) qk_norm_rope_store_fast_kernel(
    const T* __restrict__ qkv, const T* __restrict__ q_w, const T* __restrict__ k_w,
    const int32_t* __restrict__ positions, const float* __restrict__ cos_sin, T* __restrict__ q_out,
    void* __restrict__ k_cache, void* __restrict__ v_cache, const int32_t* __restrict__ out_loc,
    const float* __restrict__ k_scale, const float* __restrict__ v_scale, int hq, int hk, int page_size, float eps,
    int interleaved, int cache_fp8, int max_pos, int num_slots) {
  pdl_enter();
  constexpr int E = D / 64, H2 = D / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.x;
  const int head = blockIdx.y * 4 + warp;
  const int heads_total = hq + 2 * hk;
  if (head >= heads_total) return;
  const T* src = qkv + (size_t)token * heads_total * D + (size_t)head * D;
  // element indices owned by this lane: lo[t], hi[t]
  int idx_lo[E], idx_hi[E];
#pragma unroll
  for (int t = 0; t < E; ++t) {
    if (interleaved) { idx_lo[t] = 2 * (E * lane + t); idx_hi[t] = idx_lo[t] + 1; }
    else { idx_lo[t] = E * lane + t; idx_hi[t] = idx_lo[t] + H2; }
  }
  float a[E], b[E];
  float ss = 0.f;
  if (interleaved) {
#pragma unroll
    for (int t = 0; t < E; ++t) {
      a[t] = to_float(src[idx_lo[t]]);
      b[t] = to_float(src[idx_hi[t]]);
    }
  } else {
    load_run<T, E>(src + E * lane, a);
    load_run<T, E>(src + H2 + E * lane, b);
  }
#pragma unroll
  for (int t = 0; t < E; ++t) ss += a[t] * a[t] + b[t] * b[t];
  const bool is_q = head < hq, is_k = !is_q && head < hq + hk;
  if (is_q || is_k) {
    const T* w = is_q ? q_w : k_w;
    if (w != nullptr) {
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
      for (int t = 0; t < E; ++t) {
        a[t] = to_float(from_float<T>(a[t] * rstd * to_float(w[idx_lo[t]])));
        b[t] = to_float(from_float<T>(b[t] * rstd * to_float(w[idx_hi[t]])));
      }
    }
    int pos = positions[token];
    (void)MSGL_OOB(pos, max_pos);
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + (size_t)pos * D;
#pragma unroll
    for (int t = 0; t < E; ++t) {
      const int p = E * lane + t;
      const float c = cs[p], sn = cs[H2 + p];
      const float x0 = a[t], x1 = b[t];
      a[t] = x0 * c - x1 * sn;
      b[t] = x1 * c + x0 * sn;
    }
  }
  if (is_q) {
    T* dst = q_out + ((size_t)token * hq + head) * D;
    if (interleaved) {
#pragma unroll
      for (int t = 0; t < E; ++t) {
        dst[idx_lo[t]] = from_float<T>(a[t]);
        dst[idx_hi[t]] = from_float<T>(b[t]);
      }
    } else {
      store_run<T, E>(dst + E * lane, a);
      store_run<T, E>(dst + H2 + E * lane, b);
    }
    return;
  }
  const int kvh = is_k ? head - hq : head - hq - hk;
  const int slot = out_loc[token];
  if (slot >= 0) (void)MSGL_OOB(slot, num_slots);
  if (slot < 0 || slot >= num_slots) return;
  const int page = slot / page_size, off = slot % page_size;
  const size_t base = (((size_t)page * hk + kvh) * page_size + off) * D;
  void* cache = is_k ? k_cache : v_cache;
  if (cache_fp8) {
    const float sc = is_k ? k_scale[kvh] : v_scale[kvh];
    uint8_t* dst = (uint8_t*)cache + base;
#pragma unroll
    for (int t = 0; t < E; ++t) {
      dst[idx_lo[t]] = float_to_e4m3(to_float(from_float<T>(a[t])) / sc);
      dst[idx_hi[t]] = float_to_e4m3(to_float(from_float<T>(b[t])) / sc);
    }
  } else {
    T* dst = (T*)cache + base;
#pragma unroll
    for (int t = 0; t < E; ++t) {
      dst[idx_lo[t]] = from_float<T>(a[t]);
      dst[idx_hi[t]] = from_float<T>(b[t]);
    }
  }
}

// Vectorised variant for the common case (head_dim 128, full NeoX rotation): eight lanes own one
// head, each lane holding eight consecutive elements of the low half and the matching eight of
// the high half (one 16-byte load each), so a warp covers four heads; the per-head RMS is a
// reduction over the eight lanes; q leaves as 16-byte stores and fp8 K/V as 8-byte stores.
template <typename T>
__global__ void __launch_bounds__(128) qk_norm_rope_store_vec128_kernel(
    const T* __restrict__ qkv, const T* __restrict__ q_w, const T* __restrict__ k_w,
    const int32_t* __restrict__ positions, const float* __restrict__ cos_sin, T* __restrict__ q_out,
    void* __restrict__ k_cache, void* __restrict__ v_cache, const int32_t* __restrict__ out_loc,
    const float* __restrict__ k_scale, const float* __restrict__ v_scale, int hq, int hk, int page_size, float eps,
    int cache_fp8, int max_pos, int num_slots) {
  pdl_enter();
  constexpr int D = 128, H2 = 64;
  const int token = blockIdx.x;
  const int sub = threadIdx.x & 7;                       // lane within the head's group of eight
  const int head = blockIdx.y * 16 + (threadIdx.x >> 3);
  const int heads_total = hq + 2 * hk;
  const bool live = head < heads_total;
  const int hd = live ? head : heads_total - 1;          // idle groups shadow the last head (no stores)
  const T* src = qkv + (size_t)token * heads_total * D + (size_t)hd * D;
  float a[8], b[8];
  load8(src + sub * 8, a);
  load8(src + H2 + sub * 8, b);
  float ss = 0.f;
#pragma unroll
  for (int t = 0; t < 8; ++t) ss += a[t] * a[t] + b[t] * b[t];
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  ss += __shfl_xor_sync(0xffffffffu, ss, 4);
  if (!live) return;
  const bool is_q = head < hq, is_k = !is_q && head < hq + hk;
  if (is_q || is_k) {
    const T* w = is_q ? q_w : k_w;
    if (w != nullptr) {
      const float rstd = rsqrtf(ss / (float)D + eps);
      float wl[8], wh[8];
      load8(w + sub * 8, wl);
      load8(w + H2 + sub * 8, wh);
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        a[t] = to_float(from_float<T>(a[t] * rstd * wl[t]));
        b[t] = to_float(from_float<T>(b[t] * rstd * wh[t]));
      }
    }
    int pos = positions[token];
    (void)MSGL_OOB(pos, max_pos);
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float4* cs = reinterpret_cast<const float4*>(cos_sin + (size_t)pos * D + sub * 8);
    const float4* sn = reinterpret_cast<const float4*>(cos_sin + (size_t)pos * D + H2 + sub * 8);
    const float4 c0 = cs[0], c1 = cs[1], s0 = sn[0], s1 = sn[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const float x0 = a[t], x1 = b[t];
      a[t] = x0 * c[t] - x1 * sv[t];
      b[t] = x1 * c[t] + x0 * sv[t];
    }
  }
  if (is_q) {
    T* dst = q_out + ((size_t)token * hq + head) * D;
    store8(dst + sub * 8, a);
    store8(dst + H2 + sub * 8, b);
    return;
  }
  const int kvh = is_k ? head - hq : head - hq - hk;
  const int slot = out_loc[token];
  if (slot >= 0) (void)MSGL_OOB(slot, num_slots);
  if (slot < 0 || slot >= num_slots) return;
  const int page = slot / page_size, off = slot % page_size;
  const size_t base = (((size_t)page * hk + kvh) * page_size + off) * D;
  void* cache = is_k ? k_cache : v_cache;
  if (cache_fp8) {
    const float sc = is_k ? k_scale[kvh] : v_scale[kvh];
    uint8_t* dst = (uint8_t*)cache + base;
    float ra[8], rb[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      ra[t] = to_float(from_float<T>(a[t])) / sc;   // same rounding and division as the scalar kernel
      rb[t] = to_float(from_float<T>(b[t])) / sc;
    }
    uint2 pa, pb;
    pa.x = (uint32_t)float_to_e4m3(ra[0]) | ((uint32_t)float_to_e4m3(ra[1]) << 8) | ((uint32_t)float_to_e4m3(ra[2]) << 16) |
           ((uint32_t)float_to_e4m3(ra[3]) << 24);
    pa.y = (uint32_t)float_to_e4m3(ra[4]) | ((uint32_t)float_to_e4m3(ra[5]) << 8) | ((uint32_t)float_to_e4m3(ra[6]) << 16) |
           ((uint32_t)float_to_e4m3(ra[7]) << 24);
    pb.x = (uint32_t)float_to_e4m3(rb[0]) | ((uint32_t)float_to_e4m3(rb[1]) << 8) | ((uint32_t)float_to_e4m3(rb[2]) << 16) |
           ((uint32_t)float_to_e4m3(rb[3]) << 24);
    pb.y = (uint32_t)float_to_e4m3(rb[4]) | ((uint32_t)float_to_e4m3(rb[5]) << 8) | ((uint32_t)float_to_e4m3(rb[6]) << 16) |
           ((uint32_t)float_to_e4m3(rb[7]) << 24);
    *reinterpret_cast<uint2*>(dst + sub * 8) = pa;
    *reinterpret_cast<uint2*>(dst + H2 + sub * 8) = pb;
  } else {
    T* dst = (T*)cache + base;
    store8(dst + sub * 8, a);
    store8(dst + H2 + sub * 8, b);
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
  do {                                                                                                      \
  if (rot == head_dim && D == 128 && !interleaved)                                                          \
    msgl_launch(qk_norm_rope_store_vec128_kernel<T>, dim3(dim3(tokens, (hq + 2 * hk + 15) / 16)), dim3(128), 0, stream, \
        (const T*)qkv, (const T*)q_w, (const T*)k_w, (const int32_t*)positions, (const float*)cos_sin,      \
        (T*)q_out, k_cache, v_cache, (const int32_t*)out_loc, (const float*)k_scale, (const float*)v_scale, \
        hq, hk, page_size, eps, cache_fp8, max_pos, num_slots);                                             \
  else if (rot == head_dim)                                                                                 \
    msgl_launch(qk_norm_rope_store_fast_kernel<T, D>, dim3(grid), dim3(128), 0, stream, \
        (const T*)qkv, (const T*)q_w, (const T*)k_w, (const int32_t*)positions, (const float*)cos_sin,      \
        (T*)q_out, k_cache, v_cache, (const int32_t*)out_loc, (const float*)k_scale, (const float*)v_scale, \
        hq, hk, page_size, eps, interleaved, cache_fp8, max_pos, num_slots);                                \
  else                                                                                                      \
                                                                                        \
  msgl_launch(qk_norm_rope_store_kernel<T, D>, dim3(grid), dim3(128), 0, stream, \
      (const T*)qkv, (const T*)q_w, (const T*)k_w, (const int32_t*)positions, (const float*)cos_sin,        \
      (T*)q_out, k_cache, v_cache, (const int32_t*)out_loc, (const float*)k_scale, (const float*)v_scale,   \
      hq, hk, rot, page_size, eps, interleaved, cache_fp8, max_pos, num_slots);                            \
  } while (0)
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
  pdl_enter();
  const int token = blockIdx.x;
  const int slot = out_loc[token];
  if (slot >= 0) (void)MSGL_OOB(slot, num_slots);
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
    msgl_launch(store_kv_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, k_cache, v_cache, (const int32_t*)out_loc,
        (const float*)k_scale, (const float*)v_scale, hk, head_dim, page_size, cache_fp8, num_slots);
  else if (dtype == MSGL_F16)
    msgl_launch(store_kv_kernel<__half>, dim3(tokens), dim3(256), 0, stream, (const __half*)k, (const __half*)v, k_cache, v_cache, (const int32_t*)out_loc, (const float*)k_scale,
        (const float*)v_scale, hk, head_dim, page_size, cache_fp8, num_slots);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("store_kv");
  return MSGL_OK;
}
