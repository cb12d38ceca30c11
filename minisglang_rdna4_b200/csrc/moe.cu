// Mixture-of-experts routing and data movement around the grouped tcgen05 GEMMs.
//
//   moe_route      : scores (softmax or sigmoid) -> top-k -> renormalise, one warp per token,
//                    plus per-expert counts (the reference's moe_route_align / moe_topk_*;
//                    python/minisgl/quant/kernels.py:423-481)
//   moe_align      : pad every expert's row count to the 128-row GEMM tile, assign each
//                    (token, k) pair a row in the expert-sorted order, record the expert of
//                    every tile (sgl_kernel.moe_align_block_size in the reference's CUDA path,
//                    python/minisgl/moe/fused.py:96-117)
//   moe_permute    : gather token rows into expert-sorted order
//   moe_combine    : out[t] = sum_k w[t,k] * y[row_of(t,k)] in a fixed k order
//                    (mmq_fp8_moe_gather_reduce, python/minisgl/quant/kernels.py:877)
//
// Shapes are static for CUDA graphs: the sorted buffers are sized for the worst case
// T*k + E*127 rows and tiles past the live count carry expert id -1, which the GEMM skips.
#include "common.cuh"

using namespace msgl;

namespace {

constexpr int kMaxExperts = 512;
constexpr int kMaxTopK = 16;

// one warp per token; E <= 512 (16 values per lane)
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ logits, const float* __restrict__ bias,
                                 float* __restrict__ topk_w, int32_t* __restrict__ topk_ids,
                                 int32_t* __restrict__ counts, int tokens, int E, int k, int renorm, int sigmoid,
                                 float scale, int e_start, int e_local) {
  pdl_enter();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const int lane = threadIdx.x & 31;
  constexpr int PER = kMaxExperts / 32;
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? to_float(logits[(size_t)t * E + e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  if (sigmoid) {
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = (lane + 32 * i) < E ? 1.f / (1.f + expf(-v[i])) : -INFINITY;
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      v[i] = (lane + 32 * i) < E ? expf(v[i] - mx) : 0.f;
      sum += v[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = (lane + 32 * i) < E ? v[i] * inv : -INFINITY;
  }
  // experts are chosen by score + selection bias (when given); the weights are the scores themselves
  float c[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    c[i] = (bias != nullptr && e < E) ? v[i] + bias[e] : v[i];
  }
  float wsel[kMaxTopK];
  int isel[kMaxTopK];
  float total = 0.f;
  for (int kk = 0; kk < k; ++kk) {
    // arg-max over the remaining choice scores, lowest expert id on ties
    float best = -INFINITY, bw = 0.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (c[i] > best || (c[i] == best && e < bi)) { best = c[i]; bi = e; bw = v[i]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const float ow = __shfl_xor_sync(0xffffffffu, bw, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; bw = ow; }
    }
    wsel[kk] = bw;
    isel[kk] = bi;
    total += bw;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (lane + 32 * i == bi) c[i] = -INFINITY;
  }
  if (lane == 0) {
    const float norm = renorm ? 1.f / fmaxf(total, 1e-20f) : 1.f;
    for (int kk = 0; kk < k; ++kk) {
      topk_w[(size_t)t * k + kk] = wsel[kk] * norm * scale;
      topk_ids[(size_t)t * k + kk] = isel[kk];
      const int local = isel[kk] - e_start;
      if (counts != nullptr && local >= 0 && local < e_local) atomicAdd(counts + local, 1);
    }
  }
}

// single CTA: padded offsets + tile -> expert map
__global__ void moe_offsets_kernel(const int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                                   int32_t* __restrict__ cursor, int32_t* __restrict__ tile_expert,
                                   int32_t* __restrict__ meta, int e_local, int max_tiles, int block) {
  pdl_enter();
  __shared__ int s_off[kMaxExperts + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < e_local; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + block - 1) / block * block;
    }
    s_off[e_local] = acc;
    meta[0] = acc / block;   // live tiles
    meta[1] = acc;           // live (padded) rows
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= e_local; e += blockDim.x) {
    offsets[e] = s_off[e];
    if (e < e_local) cursor[e] = 0;
  }
  for (int m = threadIdx.x; m < max_tiles; m += blockDim.x) {
    const int row = m * block;
    int ex = -1;
    if (row < s_off[e_local]) {
      // binary search for the expert whose padded range holds this row
      int lo = 0, hi = e_local;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid;
      }
      ex = lo;
    }
    tile_expert[m] = ex;
  }
}

// one thread per (token, k) pair: claim a row in the expert's range
__global__ void moe_scatter_kernel(const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ offsets,
                                   int32_t* __restrict__ cursor, int32_t* __restrict__ sorted_pair,
                                   int32_t* __restrict__ pair_row, int pairs, int e_start, int e_local) {
  pdl_enter();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= pairs) return;
  const int local = topk_ids[p] - e_start;
  if (local < 0 || local >= e_local) {
    pair_row[p] = -1;
    return;
  }
  const int row = offsets[local] + atomicAdd(cursor + local, 1);
  sorted_pair[row] = p;
  pair_row[p] = row;
}

template <typename T>
__global__ void moe_permute_kernel(const T* __restrict__ x, const int32_t* __restrict__ sorted_pair,
                                   T* __restrict__ out, int hidden, int k, int rows) {
  pdl_enter();
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int pair = sorted_pair[row];
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * hidden);
  const int vecs = hidden / 8;
  if (pair < 0) {
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(pair / k) * hidden);
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) dst[i] = src[i];
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const float* __restrict__ topk_w,
                                   const int32_t* __restrict__ pair_row, T* __restrict__ out, int hidden, int k) {
  pdl_enter();
  const int t = blockIdx.x;
  for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int kk = 0; kk < k; ++kk) {
      const int row = pair_row[(size_t)t * k + kk];
      if (row < 0) continue;
      const float w = topk_w[(size_t)t * k + kk];
      float v[8];
      load8(y + (size_t)row * hidden + i, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += w * v[e];
    }
    store8(out + (size_t)t * hidden + i, acc);
  }
}

}  // namespace

MSGL_API int msgl_moe_route(const void* logits, const void* bias, void* topk_w, void* topk_ids, void* counts,
                            int tokens, int E, int k, int renorm, int sigmoid, float scale, int e_start, int e_local,
                            int dtype, cudaStream_t stream) {
  if (E > kMaxExperts || k > kMaxTopK || k > E) return MSGL_BAD_ARG;
  // counts (optional): tokens per local expert, for the alignment step; zeroed here
  if (counts != nullptr) cudaMemsetAsync(counts, 0, sizeof(int32_t) * e_local, stream);
  if (tokens == 0) return MSGL_OK;
  const int warps = 4;
  const int blocks = (tokens + warps - 1) / warps;
#define ROUTE(T)                                                                                                   \
  msgl_launch(moe_route_kernel<T>, dim3(blocks), dim3(warps * 32), 0, stream, (const T*)logits, (const float*)bias, \
              (float*)topk_w, (int32_t*)topk_ids, (int32_t*)counts, tokens, E, k, renorm, sigmoid, scale, e_start,   \
              e_local)
  if (dtype == MSGL_F32) ROUTE(float);
  else if (dtype == MSGL_BF16) ROUTE(__nv_bfloat16);
  else if (dtype == MSGL_F16) ROUTE(__half);
  else return MSGL_BAD_ARG;
#undef ROUTE
  MSGL_CHECK_LAUNCH("moe_route");
  return MSGL_OK;
}

// counts [e_local] (from msgl_moe_route) -> offsets [e_local+1], tile_expert [max_tiles], meta [2],
// sorted_pair [max_rows] (filled with -1 first), pair_row [tokens*k]
MSGL_API int msgl_moe_align(const void* topk_ids, const void* counts, void* offsets, void* cursor, void* tile_expert,
                            void* meta, void* sorted_pair, void* pair_row, int tokens, int k, int e_start,
                            int e_local, int max_rows, int block, cudaStream_t stream) {
  if (tokens == 0) return MSGL_OK;
  if (e_local > kMaxExperts) return MSGL_BAD_ARG;
  cudaMemsetAsync(sorted_pair, 0xff, sizeof(int32_t) * (size_t)max_rows, stream);
  msgl_launch(moe_offsets_kernel, dim3(1), dim3(256), 0, stream, (const int32_t*)counts, (int32_t*)offsets, (int32_t*)cursor,
                                            (int32_t*)tile_expert, (int32_t*)meta, e_local, max_rows / block, block);
  const int pairs = tokens * k;
  msgl_launch(moe_scatter_kernel, dim3((pairs + 255) / 256), dim3(256), 0, stream, (const int32_t*)topk_ids, (const int32_t*)offsets,
                                                              (int32_t*)cursor, (int32_t*)sorted_pair,
                                                              (int32_t*)pair_row, pairs, e_start, e_local);
  MSGL_CHECK_LAUNCH("moe_align");
  return MSGL_OK;
}

MSGL_API int msgl_moe_permute(const void* x, const void* sorted_pair, void* out, int hidden, int k, int rows,
                              int dtype, cudaStream_t stream) {
  if (rows == 0) return MSGL_OK;
  if (hidden % 8) return MSGL_BAD_ARG;
  int threads = hidden / 8 < 256 ? ((hidden / 8 + 31) / 32) * 32 : 256;
  if (dtype == MSGL_BF16)
    msgl_launch(moe_permute_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, (const __nv_bfloat16*)x, (const int32_t*)sorted_pair,
                                                                   (__nv_bfloat16*)out, hidden, k, rows);
  else if (dtype == MSGL_F16)
    msgl_launch(moe_permute_kernel<__half>, dim3(rows), dim3(threads), 0, stream, (const __half*)x, (const int32_t*)sorted_pair,
                                                            (__half*)out, hidden, k, rows);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("moe_permute");
  return MSGL_OK;
}

MSGL_API int msgl_moe_combine(const void* y, const void* topk_w, const void* pair_row, void* out, int tokens,
                              int hidden, int k, int dtype, cudaStream_t stream) {
  if (tokens == 0) return MSGL_OK;
  if (hidden % 8) return MSGL_BAD_ARG;
  int threads = hidden / 8 < 256 ? ((hidden / 8 + 31) / 32) * 32 : 256;
  if (dtype == MSGL_BF16)
    msgl_launch(moe_combine_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)y, (const float*)topk_w,
                                                                     (const int32_t*)pair_row, (__nv_bfloat16*)out,
                                                                     hidden, k);
  else if (dtype == MSGL_F16)
    msgl_launch(moe_combine_kernel<__half>, dim3(tokens), dim3(threads), 0, stream, (const __half*)y, (const float*)topk_w,
                                                              (const int32_t*)pair_row, (__half*)out, hidden, k);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("moe_combine");
  return MSGL_OK;
}
