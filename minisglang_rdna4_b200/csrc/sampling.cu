// Sampling kernels: row-wise arg-max over fp32 logits (greedy decoding and speculative verify)
// and temperature / top-k / top-p / min-p sampling by bisection on the probability threshold.
//
// Replaces the reference's sampler_hip.top_k_top_p_sampling_from_logits_
// (python/minisgl/engine/_sampler_hip.py:42-63) and the torch arg-max of its greedy path.
// The sampling kernel never sorts the vocabulary: top-k and top-p both keep "every token
// whose probability is at least some pivot", so the pivot is found by bisection over
// probability values (each probe is one pass over the row held in shared memory or re-read
// from L2), then the token is drawn by an inverse-CDF scan in vocabulary order over the kept
// set. Semantics follow python/minisgl/engine/sample.py:108-142 (min-p floor, then top-k, then
// top-p over the surviving mass, renormalise, draw).
#include "common.cuh"

using namespace msgl;

namespace {

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  // larger value wins; on ties the lower index wins (matches torch.argmax on the first maximum)
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int32_t* __restrict__ out,
                                                      int vocab, long long stride) {
  pdl_enter();
  __shared__ ArgMax red[32];
  const float* row = logits + (size_t)blockIdx.x * stride;
  ArgMax best{-INFINITY, 0x7fffffff};
  const int vec_end = (vocab / 4) * 4;
  const bool aligned = ((uintptr_t)row % 16) == 0;
  if (aligned) {
    for (int i = threadIdx.x * 4; i < vec_end; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(row + i);
      best = better(best, ArgMax{v.x, i});
      best = better(best, ArgMax{v.y, i + 1});
      best = better(best, ArgMax{v.z, i + 2});
      best = better(best, ArgMax{v.w, i + 3});
    }
    for (int i = vec_end + threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgMax{row[i], i});
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgMax{row[i], i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = best;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? red[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, other);
    }
    if (lane == 0) out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
  }
}

// ---- sampling --------------------------------------------------------------------------
// count and mass of probabilities > pivot (strict) or >= pivot
__device__ __forceinline__ void probe(const float* __restrict__ row, int vocab, float mx, float inv_t, float inv_z,
                                      float pivot, bool strict, float* scratch, float& count, float& mass) {
  float c = 0.f, m = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float p = __expf((row[i] - mx) * inv_t) * inv_z;
    if (strict ? (p > pivot) : (p >= pivot)) { c += 1.f; m += p; }
  }
  count = block_sum(c, scratch);
  mass = block_sum(m, scratch);
}

__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, long long stride,
                                                      const float* __restrict__ temps, const int32_t* __restrict__ top_k,
                                                      const float* __restrict__ top_p, const float* __restrict__ min_p,
                                                      const float* __restrict__ uniform, int32_t* __restrict__ out,
                                                      int vocab) {
  pdl_enter();
  __shared__ float scratch[32];
  __shared__ ArgMax red[32];
  __shared__ float warp_mass[32];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * stride;
  const float t = temps[r];
  // row maximum and arg-max
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgMax{row[i], i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = best;
  __syncthreads();
  best = red[0];
  for (int w = 1; w < nw; ++w) best = better(best, red[w]);
  if (t <= 0.f) {
    if (threadIdx.x == 0) out[r] = best.i;
    return;
  }
  const float mx = best.v, inv_t = 1.f / fmaxf(t, 1e-6f);
  float z = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) z += __expf((row[i] - mx) * inv_t);
  z = block_sum(z, scratch);
  const float inv_z = 1.f / z;
  const float p_max = inv_z;  // probability of the arg-max token
  // pivot = smallest probability that is still kept
  float pivot = 0.f;
  if (min_p != nullptr && min_p[r] > 0.f) pivot = p_max * min_p[r];
  const int k = top_k != nullptr ? top_k[r] : 0;
  const float pp = top_p != nullptr ? top_p[r] : 1.f;
  if ((k > 0 && k < vocab) || pp < 1.f) {
    // A token of probability x survives iff fewer than k tokens are more probable and the mass of
    // the more probable tokens does not exceed top-p. Both tests are monotone in x, so the kept
    // set is {p >= x*}; bisect for x*. `hi` always passes the test, `lo` does not.
    float lo = 0.f, hi = p_max;
    for (int it = 0; it < 40; ++it) {
      const float mid = 0.5f * (lo + hi);
      if (mid <= lo || mid >= hi) break;
      float cnt, mass;
      probe(row, vocab, mx, inv_t, inv_z, mid, true, scratch, cnt, mass);
      const bool keep = !((k > 0 && k < vocab) && cnt >= (float)k) && !(pp < 1.f && mass > pp);
      if (keep) hi = mid; else lo = mid;
    }
    pivot = fmaxf(pivot, hi);
  }
  // kept mass
  float cnt, mass;
  probe(row, vocab, mx, inv_t, inv_z, pivot, false, scratch, cnt, mass);
  const float target = uniform[r] * mass;
  // inverse-CDF scan in vocabulary order over kept tokens: each thread owns a contiguous span
  const int per = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(threadIdx.x * per, vocab), end = min(begin + per, vocab);
  float local = 0.f;
  for (int i = begin; i < end; ++i) {
    const float p = __expf((row[i] - mx) * inv_t) * inv_z;
    if (p >= pivot) local += p;
  }
  // exclusive prefix over threads
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) warp_mass[warp] = incl;
  __syncthreads();
  float warp_off = 0.f;
  for (int w = 0; w < warp; ++w) warp_off += warp_mass[w];
  const float excl = warp_off + incl - local;
  __shared__ int chosen;
  if (threadIdx.x == 0) chosen = -1;
  __syncthreads();
  if (local > 0.f && target >= excl && target < excl + local) {
    float run = excl;
    int pick = -1;
    for (int i = begin; i < end; ++i) {
      const float p = __expf((row[i] - mx) * inv_t) * inv_z;
      if (p >= pivot) {
        run += p;
        pick = i;
        if (target < run) break;
      }
    }
    if (pick >= 0) atomicMax(&chosen, pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = chosen >= 0 ? chosen : best.i;
}

}  // namespace

MSGL_API int msgl_argmax(const void* logits, void* out, int rows, int vocab, long long stride, cudaStream_t stream) {
  if (rows == 0) return MSGL_OK;
  msgl_launch(argmax_kernel, dim3(rows), dim3(1024), 0, stream, (const float*)logits, (int32_t*)out, vocab, stride);
  MSGL_CHECK_LAUNCH("argmax");
  return MSGL_OK;
}

MSGL_API int msgl_sample(const void* logits, long long stride, const void* temps, const void* top_k,
                         const void* top_p, const void* min_p, const void* uniform, void* out, int rows, int vocab,
                         cudaStream_t stream) {
  if (rows == 0) return MSGL_OK;
  msgl_launch(sample_kernel, dim3(rows), dim3(1024), 0, stream, (const float*)logits, stride, (const float*)temps, (const int32_t*)top_k,
                                           (const float*)top_p, (const float*)min_p, (const float*)uniform,
                                           (int32_t*)out, vocab);
  MSGL_CHECK_LAUNCH("sample");
  return MSGL_OK;
}
