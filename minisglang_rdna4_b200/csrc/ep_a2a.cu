// Expert-parallel all-to-all over NVLink peer memory, fused with the routing-side work.
//
//   ep_dispatch      (source rank)  for every (token, k) pair: pick the rank that owns the expert,
//                                   claim a slot in that rank's receive region and store the token
//                                   row there with P2P stores, together with (local expert id,
//                                   pair index); the last CTA publishes the per-destination counts
//                                   and raises the sequence flags
//                                   With a quantised expert stack the row is quantised to e4m3
//                                   on the way out (one scale per token, or per 128 elements for
//                                   block-scaled experts), which halves the bytes on the links;
//                                   the scales travel beside the row
//   ep_recv_prepare  (owner rank)   bounded wait for every source's flag; expand counts into a
//                                   flat expert-id list (-1 past the count) that the local
//                                   align / permute / grouped-GEMM pipeline consumes
//   ep_return        (owner rank)   store every expert output row back into the source rank's
//                                   return region (same slot it arrived in), then raise flags
//   ep_combine       (source rank)  bounded wait for the owners' flags; out[t] = sum_k w[t,k] *
//                                   returned row of pair (t,k)   (gate-weighted sum fused in)
//
// Replaces the reference's gather-everything exchange (all_gather of an (N, 2H + 8k) byte blob
// and an all_reduce of (ep*N, H); python/minisgl/layers/moe.py:1244-1311): only the rows an
// expert owner needs cross the links, once in each direction. Regions are sized for the worst
// case (every pair of a source going to one owner) so shapes are static under CUDA graphs.
// Peer memory is only ever written; every wait is bounded and reports through a status word.
#include "common.cuh"

using namespace msgl;

namespace {

constexpr int kMaxRanks = 8;

struct EpBuffers {
  // per-rank symmetric region layout (byte offsets from the region base)
  //   recv_rows [R][cap][H]      T
  //   ret_rows  [R][cap][H]      T
  //   recv_meta [R][cap][2]      int32 (local expert id, source pair index)
  //   recv_count[R], recv_flag[R], ret_flag[R]   uint32
  //   recv_scale[R][cap][S]      fp32 (S = 0 for 16-bit rows, 1 per token, H / 128 per group)
  unsigned char* base[kMaxRanks];
  long long off_recv_rows, off_ret_rows, off_recv_scale, off_recv_meta, off_recv_count, off_recv_flag, off_ret_flag;
  int rank, nranks, cap, hidden;
  int qmode;      // 0: 16-bit rows, 1: e4m3 + one scale per token, 2: e4m3 + one scale per 128 elements
  int nscale;     // scales per row
  int active;     // rows per source that can be in use this step (<= cap): bounds every slot loop
};

__device__ int g_ep_status = 0;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t seq, unsigned long long limit_ns, int code) {
  if ((int)(ld_acquire_sys(p) - seq) >= 0) return true;
  const unsigned long long t0 = gtimer();
  while ((int)(ld_acquire_sys(p) - seq) < 0) {
    if (gtimer() - t0 > limit_ns) {
      atomicCAS(&g_ep_status, 0, code);
      return false;
    }
  }
  return true;
}

// grid = tokens, block = 128. state: [0..R) cursors, [R] done counter, [R+1] sequence (device-resident)
template <typename T>
__global__ void ep_dispatch_kernel(EpBuffers b, const T* __restrict__ x, const int32_t* __restrict__ topk_ids,
                                   int32_t* __restrict__ send_slot, uint32_t* __restrict__ state, int tokens, int k,
                                   int experts_per_rank) {
  pdl_enter();
  __shared__ int s_slot[16];
  __shared__ int s_dst[16];
  const int t = blockIdx.x;
  if (threadIdx.x < k) {
    const int e = topk_ids[(size_t)t * k + threadIdx.x];
    int dst = -1, slot = -1;
    if (e >= 0 && e < experts_per_rank * b.nranks) {
      dst = e / experts_per_rank;
      slot = (int)atomicAdd(&state[dst], 1u);
      if (slot >= b.active) { slot = -1; dst = -1; }   // cannot happen while tokens * k <= active
      else {
        int32_t* meta = reinterpret_cast<int32_t*>(b.base[dst] + b.off_recv_meta) +
                        ((size_t)b.rank * b.cap + slot) * 2;
        meta[0] = e % experts_per_rank;
        meta[1] = t * k + threadIdx.x;
      }
    }
    s_dst[threadIdx.x] = dst;
    s_slot[threadIdx.x] = slot;
    send_slot[(size_t)t * k + threadIdx.x] = dst < 0 ? -1 : dst * b.cap + slot;
  }
  __syncthreads();
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * b.hidden);
  const int vecs = b.hidden / 8;
  for (int kk = 0; kk < k; ++kk) {
    const int dst = s_dst[kk];
    if (dst < 0) continue;
    uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<T*>(b.base[dst] + b.off_recv_rows) +
                                          ((size_t)b.rank * b.cap + s_slot[kk]) * b.hidden);
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) out[i] = src[i];
  }
  // last CTA publishes counts and flags. Every CTA first makes its own peer stores visible
  // system-wide: a GPU-scope fence does not wait for stores that are still on their way to another
  // GPU, so the last CTA's flag could overtake a sibling CTA's rows on a different NVLink path.
  __threadfence_system();
  __syncthreads();
  __shared__ bool s_last;
  if (threadIdx.x == 0) s_last = atomicAdd(&state[b.nranks], 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last && threadIdx.x < b.nranks) {
    const int dst = threadIdx.x;
    const uint32_t seq = state[b.nranks + 1] + 1u;
    uint32_t* cnt = reinterpret_cast<uint32_t*>(b.base[dst] + b.off_recv_count) + b.rank;
    const uint32_t c = atomicAdd(&state[dst], 0u);
    *cnt = c < (uint32_t)b.active ? c : (uint32_t)b.active;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(b.base[dst] + b.off_recv_flag) + b.rank, seq);
  }
  if (s_last) {
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int r = 0; r < b.nranks; ++r) state[r] = 0u;   // ready for the next call
      state[b.nranks] = 0u;
      state[b.nranks + 1] += 1u;
    }
  }
}

// Same exchange with the row quantised to e4m3 on the way out. QMODE 1: one scale per token
// (amax / 448); QMODE 2: one scale per 128 elements. grid = tokens, block = 128, hidden <= 8192.
template <typename T, int QMODE>
__global__ void ep_dispatch_quant_kernel(EpBuffers b, const T* __restrict__ x, const int32_t* __restrict__ topk_ids,
                                         int32_t* __restrict__ send_slot, uint32_t* __restrict__ state, int tokens,
                                         int k, int experts_per_rank) {
  pdl_enter();
  __shared__ int s_slot[16];
  __shared__ int s_dst[16];
  __shared__ float s_amax[1024];   // per 8-element vector
  __shared__ float s_scale[64];    // per group (QMODE 2) or [0] (QMODE 1)
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  if (threadIdx.x < k) {
    const int e = topk_ids[(size_t)t * k + threadIdx.x];
    int dst = -1, slot = -1;
    if (e >= 0 && e < experts_per_rank * b.nranks) {
      dst = e / experts_per_rank;
      slot = (int)atomicAdd(&state[dst], 1u);
      if (slot >= b.active) { slot = -1; dst = -1; }
      else {
        int32_t* meta = reinterpret_cast<int32_t*>(b.base[dst] + b.off_recv_meta) +
                        ((size_t)b.rank * b.cap + slot) * 2;
        meta[0] = e % experts_per_rank;
        meta[1] = t * k + threadIdx.x;
      }
    }
    s_dst[threadIdx.x] = dst;
    s_slot[threadIdx.x] = slot;
    send_slot[(size_t)t * k + threadIdx.x] = dst < 0 ? -1 : dst * b.cap + slot;
  }
  const T* src = x + (size_t)t * b.hidden;
  const int vecs = b.hidden / 8;
  float amax_t = 0.f;
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
    float v[8];
    load8(src + i * 8, v);
    float a = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) a = fmaxf(a, fabsf(v[e]));
    s_amax[i] = a;
    amax_t = fmaxf(amax_t, a);
  }
  if (QMODE == 1) {
    amax_t = block_max(amax_t, scratch);
    if (threadIdx.x == 0) s_scale[0] = fmaxf(amax_t, 1e-8f) / kFp8Max;
  }
  __syncthreads();
  if (QMODE == 2 && threadIdx.x < b.nscale) {
    float a = 0.f;
    for (int i = 0; i < 16; ++i) a = fmaxf(a, s_amax[threadIdx.x * 16 + i]);
    s_scale[threadIdx.x] = fmaxf(a, 1e-8f) / kFp8Max;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
    float v[8];
    load8(src + i * 8, v);
    const uint2 q = pack8_e4m3(v, QMODE == 1 ? s_scale[0] : s_scale[i >> 4]);
    for (int kk = 0; kk < k; ++kk) {
      const int dst = s_dst[kk];
      if (dst < 0) continue;
      uint2* out = reinterpret_cast<uint2*>(b.base[dst] + b.off_recv_rows +
                                            ((size_t)b.rank * b.cap + s_slot[kk]) * b.hidden);
      out[i] = q;
    }
  }
  if (threadIdx.x < b.nscale) {
    for (int kk = 0; kk < k; ++kk) {
      const int dst = s_dst[kk];
      if (dst < 0) continue;
      float* sc = reinterpret_cast<float*>(b.base[dst] + b.off_recv_scale) +
                  ((size_t)b.rank * b.cap + s_slot[kk]) * b.nscale;
      sc[threadIdx.x] = s_scale[threadIdx.x];
    }
  }
  __threadfence_system();   // this CTA's peer stores first (see ep_dispatch_kernel)
  __syncthreads();
  __shared__ bool s_last;
  if (threadIdx.x == 0) s_last = atomicAdd(&state[b.nranks], 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last && threadIdx.x < b.nranks) {
    const int dst = threadIdx.x;
    const uint32_t seq = state[b.nranks + 1] + 1u;
    uint32_t* cnt = reinterpret_cast<uint32_t*>(b.base[dst] + b.off_recv_count) + b.rank;
    const uint32_t c = atomicAdd(&state[dst], 0u);
    *cnt = c < (uint32_t)b.active ? c : (uint32_t)b.active;
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(b.base[dst] + b.off_recv_flag) + b.rank, seq);
  }
  if (s_last) {
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int r = 0; r < b.nranks; ++r) state[r] = 0u;
      state[b.nranks] = 0u;
      state[b.nranks + 1] += 1u;
    }
  }
}

// Owner side: expert-sorted row r <- the received row behind sorted_pair[r] = src * active + pos
// (bytes of the row and, for quantised rows, its scales); padding rows (negative) are zero-filled
// with scale 0. grid = sorted rows, block = 128.
__global__ void ep_gather_kernel(EpBuffers b, const int32_t* __restrict__ sorted_pair, uint8_t* __restrict__ xrows,
                                 float* __restrict__ xs) {
  pdl_enter();
  const int r = blockIdx.x;
  const int flat = sorted_pair[r];
  const int row_bytes = b.hidden * (b.qmode == 0 ? 2 : 1);
  const int vecs = row_bytes / 16;
  uint4* out = reinterpret_cast<uint4*>(xrows + (size_t)r * row_bytes);
  if (flat < 0) {
    for (int i = threadIdx.x; i < vecs; i += blockDim.x) out[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x < b.nscale) xs[(size_t)r * b.nscale + threadIdx.x] = 0.f;
    return;
  }
  const size_t slot = (size_t)(flat / b.active) * b.cap + (size_t)(flat % b.active);
  const uint4* in = reinterpret_cast<const uint4*>(b.base[b.rank] + b.off_recv_rows + slot * row_bytes);
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) out[i] = in[i];
  if (threadIdx.x < b.nscale)
    xs[(size_t)r * b.nscale + threadIdx.x] =
        reinterpret_cast<const float*>(b.base[b.rank] + b.off_recv_scale)[slot * b.nscale + threadIdx.x];
}

// grid = R * ceil(active/256); expert_ids [R*active] <- local expert id or -1
__global__ void ep_recv_prepare_kernel(EpBuffers b, int32_t* __restrict__ expert_ids, const uint32_t* __restrict__ seq_ptr,
                                       unsigned long long limit_ns) {
  pdl_enter();
  const int blocks_per_src = (b.active + 255) / 256;
  const int src = blockIdx.x / blocks_per_src;
  const int pos = (blockIdx.x % blocks_per_src) * 256 + threadIdx.x;
  __shared__ uint32_t s_count;
  if (threadIdx.x == 0) {
    const uint32_t seq = *seq_ptr;   // the local dispatch of this step has already advanced it
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(b.base[b.rank] + b.off_recv_flag) + src;
    const bool ok = wait_flag(flag, seq, limit_ns, 400 + src);
    s_count = ok ? reinterpret_cast<const uint32_t*>(b.base[b.rank] + b.off_recv_count)[src] : 0u;
  }
  __syncthreads();
  if (pos >= b.active) return;
  const int32_t* meta = reinterpret_cast<const int32_t*>(b.base[b.rank] + b.off_recv_meta) + ((size_t)src * b.cap + pos) * 2;
  expert_ids[(size_t)src * b.active + pos] = pos < (int)s_count ? meta[0] : -1;
}

// grid = R * active rows (one CTA per slot in use); y_sorted rows are addressed through pair_row
template <typename T>
__global__ void ep_return_kernel(EpBuffers b, const T* __restrict__ y_sorted, const int32_t* __restrict__ pair_row,
                                 uint32_t* __restrict__ state, const uint32_t* __restrict__ seq_ptr) {
  pdl_enter();
  const int idx = blockIdx.x;           // src * active + pos
  const int src = idx / b.active, pos = idx % b.active;
  const int row = pair_row[idx];
  if (row >= 0) {
    const uint4* in = reinterpret_cast<const uint4*>(y_sorted + (size_t)row * b.hidden);
    uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<T*>(b.base[src] + b.off_ret_rows) +
                                          ((size_t)b.rank * b.cap + pos) * b.hidden);
    for (int i = threadIdx.x; i < b.hidden / 8; i += blockDim.x) out[i] = in[i];
  }
  __threadfence_system();   // this CTA's peer stores first (see ep_dispatch_kernel)
  __syncthreads();
  __shared__ bool s_last;
  if (threadIdx.x == 0) s_last = atomicAdd(&state[b.nranks + 2], 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < b.nranks)
      st_release_sys(reinterpret_cast<uint32_t*>(b.base[threadIdx.x] + b.off_ret_flag) + b.rank, *seq_ptr);
    __syncthreads();
    if (threadIdx.x == 0) state[b.nranks + 2] = 0u;
  }
}

// grid = tokens
template <typename T>
__global__ void ep_combine_kernel(EpBuffers b, const float* __restrict__ topk_w, const int32_t* __restrict__ send_slot,
                                  T* __restrict__ out, const uint32_t* __restrict__ seq_ptr, int k,
                                  unsigned long long limit_ns) {
  pdl_enter();
  const int t = blockIdx.x;
  if (threadIdx.x < b.nranks) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(b.base[b.rank] + b.off_ret_flag) + threadIdx.x;
    wait_flag(flag, *seq_ptr, limit_ns, 420 + threadIdx.x);
  }
  __syncthreads();
  const T* ret = reinterpret_cast<const T*>(b.base[b.rank] + b.off_ret_rows);
  for (int i = threadIdx.x * 8; i < b.hidden; i += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int kk = 0; kk < k; ++kk) {
      const int slot = send_slot[(size_t)t * k + kk];
      if (slot < 0) continue;
      const float w = topk_w[(size_t)t * k + kk];
      float v[8];
      load8(ret + (size_t)slot * b.hidden + i, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += w * v[e];
    }
    store8(out + (size_t)t * b.hidden + i, acc);
  }
}

int scales_per_row(int hidden, int qmode) { return qmode == 0 ? 0 : (qmode == 1 ? 1 : hidden / 128); }

EpBuffers make_buffers(void* const* bases, int rank, int nranks, int cap, int hidden, int qmode, int active) {
  EpBuffers b;
  for (int r = 0; r < nranks; ++r) b.base[r] = (unsigned char*)bases[r];
  b.rank = rank; b.nranks = nranks; b.cap = cap; b.hidden = hidden;
  b.qmode = qmode;
  b.nscale = scales_per_row(hidden, qmode);
  b.active = active <= 0 || active > cap ? cap : active;
  const long long recv = (long long)nranks * cap * hidden * (qmode == 0 ? 2 : 1);
  const long long ret = (long long)nranks * cap * hidden * 2;
  const long long scl = ((long long)nranks * cap * b.nscale * 4 + 255) / 256 * 256;
  b.off_recv_rows = 0;
  b.off_ret_rows = (recv + 255) / 256 * 256;
  b.off_recv_scale = b.off_ret_rows + ret;
  b.off_recv_meta = b.off_recv_scale + scl;
  b.off_recv_count = b.off_recv_meta + (long long)nranks * cap * 8;
  b.off_recv_flag = b.off_recv_count + 256;
  b.off_ret_flag = b.off_recv_flag + 256;
  return b;
}

}  // namespace

// qmode: 0 = 16-bit rows, 1 = e4m3 rows + one scale per token, 2 = e4m3 rows + one scale per 128 elements
MSGL_API long long msgl_ep_region_bytes(int nranks, int cap, int hidden, int qmode) {
  void* none[kMaxRanks] = {};
  EpBuffers b = make_buffers(none, 0, nranks, cap, hidden, qmode, cap);
  return b.off_ret_flag + 256;
}

// state: device array of nranks + 4 uint32, zero-initialised once. `active` = largest number of
// (token, k) pairs any rank can send this step (the same value on every rank): bounds the slot loops.
MSGL_API int msgl_ep_dispatch(void* const* bases, int rank, int nranks, int cap, int active, int qmode, const void* x,
                              const void* topk_ids, void* send_slot, void* state, int tokens, int hidden, int k,
                              int experts_per_rank, int dtype, cudaStream_t stream) {
  if (nranks > kMaxRanks || k > 16 || hidden % 8 || tokens * k > active || active > cap || qmode < 0 || qmode > 2) {
    msgl_set_error_text("ep_dispatch: shape does not fit the exchange regions");
    return MSGL_BAD_ARG;
  }
  if (qmode != 0 && (hidden % 128 || hidden > 8192)) {
    msgl_set_error_text("ep_dispatch: quantised rows need hidden % 128 == 0 and hidden <= 8192");
    return MSGL_BAD_ARG;
  }
  if (tokens == 0) return MSGL_BAD_ARG;   // every rank must take part: pad to at least one token
  if (dtype != MSGL_BF16 && dtype != MSGL_F16) return MSGL_BAD_ARG;
  EpBuffers b = make_buffers(bases, rank, nranks, cap, hidden, qmode, active);
  const int32_t* ids = (const int32_t*)topk_ids;
  int32_t* ss = (int32_t*)send_slot;
  uint32_t* st = (uint32_t*)state;
#define EP_DISPATCH(T)                                                                                              \
  do {                                                                                                              \
    if (qmode == 0)                                                                                                 \
      msgl_launch(ep_dispatch_kernel<T>, dim3(tokens), dim3(128), 0, stream, b, (const T*)x, ids, ss, st, tokens, k, \
                  experts_per_rank);                                                                                \
    else if (qmode == 1)                                                                                            \
      msgl_launch(ep_dispatch_quant_kernel<T, 1>, dim3(tokens), dim3(128), 0, stream, b, (const T*)x, ids, ss, st,  \
                  tokens, k, experts_per_rank);                                                                     \
    else                                                                                                            \
      msgl_launch(ep_dispatch_quant_kernel<T, 2>, dim3(tokens), dim3(128), 0, stream, b, (const T*)x, ids, ss, st,  \
                  tokens, k, experts_per_rank);                                                                     \
  } while (0)
  if (dtype == MSGL_BF16) EP_DISPATCH(__nv_bfloat16);
  else EP_DISPATCH(__half);
#undef EP_DISPATCH
  MSGL_CHECK_LAUNCH("ep_dispatch");
  return MSGL_OK;
}

// expert_ids [nranks * active] <- local expert id of every slot in use, -1 elsewhere
MSGL_API int msgl_ep_recv_prepare(void* const* bases, int rank, int nranks, int cap, int active, int qmode, int hidden,
                                  void* expert_ids, void* state, long long wait_us, cudaStream_t stream) {
  EpBuffers b = make_buffers(bases, rank, nranks, cap, hidden, qmode, active);
  const int blocks = nranks * ((b.active + 255) / 256);
  msgl_launch(ep_recv_prepare_kernel, dim3(blocks), dim3(256), 0, stream, b, (int32_t*)expert_ids,
              (const uint32_t*)state + nranks + 1, (unsigned long long)wait_us * 1000ull);
  MSGL_CHECK_LAUNCH("ep_recv_prepare");
  return MSGL_OK;
}

// sorted_pair [rows]: flat index (src * active + pos) of the received row behind every expert-sorted
// row, -1 for padding. Copies the rows (and the scales of quantised rows) into xrows [rows, row bytes],
// xs [rows, scales per row].
MSGL_API int msgl_ep_gather(void* const* bases, int rank, int nranks, int cap, int active, int qmode, int hidden,
                            const void* sorted_pair, void* xrows, void* xs, int rows, cudaStream_t stream) {
  if (qmode < 0 || qmode > 2 || hidden % 8 || (qmode != 0 && hidden % 128)) return MSGL_BAD_ARG;
  if (rows == 0) return MSGL_OK;
  EpBuffers b = make_buffers(bases, rank, nranks, cap, hidden, qmode, active);
  msgl_launch(ep_gather_kernel, dim3(rows), dim3(128), 0, stream, b, (const int32_t*)sorted_pair, (uint8_t*)xrows,
              (float*)xs);
  MSGL_CHECK_LAUNCH("ep_gather");
  return MSGL_OK;
}

// pair_row [nranks * active]: expert-sorted row of every slot in use (-1: none)
MSGL_API int msgl_ep_return(void* const* bases, int rank, int nranks, int cap, int active, int qmode, int hidden,
                            const void* y_sorted, const void* pair_row, void* state, int dtype, cudaStream_t stream) {
  EpBuffers b = make_buffers(bases, rank, nranks, cap, hidden, qmode, active);
  const int blocks = nranks * b.active;
  if (dtype == MSGL_BF16)
    msgl_launch(ep_return_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, b, (const __nv_bfloat16*)y_sorted,
                (const int32_t*)pair_row, (uint32_t*)state, (const uint32_t*)state + nranks + 1);
  else if (dtype == MSGL_F16)
    msgl_launch(ep_return_kernel<__half>, dim3(blocks), dim3(128), 0, stream, b, (const __half*)y_sorted,
                (const int32_t*)pair_row, (uint32_t*)state, (const uint32_t*)state + nranks + 1);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("ep_return");
  return MSGL_OK;
}

MSGL_API int msgl_ep_combine(void* const* bases, int rank, int nranks, int cap, int qmode, int hidden, const void* topk_w,
                             const void* send_slot, void* out, void* state, int tokens, int k, long long wait_us,
                             int dtype, cudaStream_t stream) {
  EpBuffers b = make_buffers(bases, rank, nranks, cap, hidden, qmode, cap);
  int threads = hidden / 8 < 256 ? ((hidden / 8 + 31) / 32) * 32 : 256;
  if (threads < 32) threads = 32;
  if (dtype == MSGL_BF16)
    msgl_launch(ep_combine_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, b, (const float*)topk_w,
                (const int32_t*)send_slot, (__nv_bfloat16*)out, (const uint32_t*)state + nranks + 1, k,
                (unsigned long long)wait_us * 1000ull);
  else if (dtype == MSGL_F16)
    msgl_launch(ep_combine_kernel<__half>, dim3(tokens), dim3(threads), 0, stream, b, (const float*)topk_w,
                (const int32_t*)send_slot, (__half*)out, (const uint32_t*)state + nranks + 1, k,
                (unsigned long long)wait_us * 1000ull);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("ep_combine");
  return MSGL_OK;
}

MSGL_API int msgl_ep_status(int reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_ep_status, sizeof(int));
  if (reset && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_ep_status, &z, sizeof(int));
  }
  return v;
}
