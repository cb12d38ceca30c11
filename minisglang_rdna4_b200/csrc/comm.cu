// Peer-memory collectives over NVLink / NVSwitch, fused with the ops that follow them.
//
//   * symmetric buffers: cudaMalloc'd per rank, exported with CUDA IPC handles, mapped by every
//     peer (the handle exchange runs over the gloo control plane in parallel/symm.py);
//   * one-shot all-reduce fused with residual add + RMSNorm (+ per-token e4m3 producer):
//     every rank pushes its partial row straight into each peer's slot (P2P stores), raises a
//     per-row sequence flag, waits for the peers' flags and reduces the rows that are now in
//     its own memory, in rank order, so every rank computes bit-identical sums;
//   * the same kernel without the norm serves as a plain in-place all-reduce.
//
// Replaces the reference's custom_ar package (one_shot_ar, one_shot_ar_push;
// python/minisgl/distributed/impl.py:178-209,351-392), which is limited to two PCIe peers, and
// the rms_norm_add that followed it. No load ever targets peer memory and nothing here uses
// TMA: peers are written with plain st.global, flags with st.release.sys / ld.acquire.sys.
//
// Every wait is bounded: after `wait_ns` a row gives up, records a status code and still runs
// to completion on whatever data it has, so the context stays usable and the host can fall
// back to the NCCL path.
#include "common.cuh"

#include <string.h>

using namespace msgl;

namespace {

constexpr int kMaxRanks = 8;

struct ArArgs {
  const void* x;             // [rows, hidden] local partial
  void* residual;            // [rows, hidden] in/out, or nullptr (plain all-reduce)
  const void* weight;        // [hidden] or nullptr
  void* out;                 // [rows, hidden] 16-bit result (normed, or the sum for a plain AR)
  uint8_t* out_q;            // optional e4m3 result
  float* out_scale;          // [rows]
  void* slots[kMaxRanks];    // slots[p]: base of rank p's data region (peer-mapped)
  uint32_t* flags[kMaxRanks];  // flags[p]: base of rank p's flag region
  uint32_t* seq;             // [max_rows] local per-row sequence counters
  int* status;
  int rank, nranks, rows, hidden, max_rows;
  long long slot_stride;     // elements between consecutive (parity, src) planes = max_rows * max_hidden
  int max_hidden;
  float eps, w_offset;
  unsigned long long wait_ns;
  // ---- in-switch reduction (NVLS): every rank keeps only its own partial rows, in a buffer that is
  // also mapped through an NVLink multicast object; one multimem.ld_reduce returns the sum over ranks
  void* my_rows;             // local address of this rank's row region [2 parity][max_rows][max_hidden]
  const void* mc_rows;       // multicast address of the same region
  uint32_t* my_count;        // local address of the arrival counters [max_rows]
  uint32_t* mc_count;        // multicast address of the counters (a reduction adds on every rank)
};

__device__ int g_comm_status = 0;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t atom_add_acq_rel_gpu(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// eight 16-bit values summed over all ranks by the switch (fp32 accumulation, one rounding)
template <typename T> __device__ __forceinline__ uint4 multimem_ld_reduce8(const void* mc_addr);
template <> __device__ __forceinline__ uint4 multimem_ld_reduce8<__nv_bfloat16>(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
  return r;
}
template <> __device__ __forceinline__ uint4 multimem_ld_reduce8<__half>(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
  return r;
}
__device__ __forceinline__ void multimem_red_release_add(uint32_t* mc_addr, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}

// One 128-thread CTA per row, the row held in registers (VPT 16-byte vectors per thread) from the
// push to the final store. NORM: residual add + RMSNorm after the reduction. QUANT: e4m3 output.
// NVLS: the reduction happens inside the NVSwitch (see ArArgs) instead of by stores into every peer.
constexpr int kArThreads = 128;

template <typename T, bool NORM, bool QUANT, int VPT, bool NVLS = false>
__global__ void __launch_bounds__(kArThreads) ar_oneshot_kernel(const ArArgs a) {
  pdl_enter();
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  const int H = a.hidden;
  const uint32_t seq = a.seq[row] + 1u;
  const int parity = (int)(seq & 1u);
  const T* xr = reinterpret_cast<const T*>(a.x) + (size_t)row * H;
  if (NVLS) {
    // 1. this rank's partial row goes into its own buffer (a local store)
    T* mine = reinterpret_cast<T*>(a.my_rows) + ((size_t)parity * a.max_rows + row) * a.max_hidden;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = (j * kArThreads + threadIdx.x) * 8;
      if (i < H) *reinterpret_cast<uint4*>(mine + i) = *reinterpret_cast<const uint4*>(xr + i);
    }
    __syncthreads();
    // 2. one multicast reduction bumps this row's arrival counter on every rank; then wait until all
    //    ranks have arrived here (the counter counts arrivals over all calls: seq * nranks by now)
    if (threadIdx.x == 0) {
      multimem_red_release_add(a.mc_count + row, 1u);
      const uint32_t want = seq * (uint32_t)a.nranks;
      const uint32_t* cnt = a.my_count + row;
      if ((int)(ld_acquire_sys(cnt) - want) < 0) {
        const unsigned long long t0 = gtimer();
        while ((int)(ld_acquire_sys(cnt) - want) < 0) {
          if (gtimer() - t0 > a.wait_ns) {
            atomicCAS(a.status, 0, 320);
            break;
          }
        }
      }
    }
    __syncthreads();
    // 3. the switch returns the sum over ranks; residual add and norm as in the push form
    const T* mc = reinterpret_cast<const T*>(a.mc_rows) + ((size_t)parity * a.max_rows + row) * a.max_hidden;
    T* rr = NORM ? reinterpret_cast<T*>(a.residual) + (size_t)row * H : nullptr;
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = (j * kArThreads + threadIdx.x) * 8;
      if (i < H) {
        const uint4 red = multimem_ld_reduce8<T>(mc + i);
        const T* rp = reinterpret_cast<const T*>(&red);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j][k] = to_float(rp[k]);
        if (NORM) {
          float r[8];
          load8(rr + i, r);
#pragma unroll
          for (int k = 0; k < 8; ++k) v[j][k] += r[k];
          store8(rr + i, v[j]);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            v[j][k] = to_float(from_float<T>(v[j][k]));
            ss += v[j][k] * v[j][k];
          }
        } else {
          store8(reinterpret_cast<T*>(a.out) + (size_t)row * H + i, v[j]);
        }
      }
    }
    if (NORM) {
      ss = block_sum(ss, scratch);
      const float rstd = rsqrtf(ss / (float)H + a.eps);
      const T* w = reinterpret_cast<const T*>(a.weight);
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int i = (j * kArThreads + threadIdx.x) * 8;
        if (i < H) {
          float wv[8];
          load8(w + i, wv);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            v[j][k] = to_float(from_float<T>(v[j][k] * rstd * (wv[k] + a.w_offset)));
            if (QUANT) amax = fmaxf(amax, fabsf(v[j][k]));
          }
          if (!QUANT) store8(reinterpret_cast<T*>(a.out) + (size_t)row * H + i, v[j]);
        }
      }
      if (QUANT) {
        amax = block_max(amax, scratch);
        const float scale = fmaxf(amax, 1e-8f) / kFp8Max;
        if (threadIdx.x == 0) a.out_scale[row] = scale;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
          const int i = (j * kArThreads + threadIdx.x) * 8;
          if (i < H) *reinterpret_cast<uint2*>(a.out_q + (size_t)row * H + i) = pack8_e4m3(v[j], scale);
        }
      }
    }
    if (threadIdx.x == 0) a.seq[row] = seq;
    return;
  }

  // 1. push this rank's partial row into every PEER's slot (its own copy stays in registers)
  uint4 mine_raw[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = (j * kArThreads + threadIdx.x) * 8;
    if (i < H) mine_raw[j] = *reinterpret_cast<const uint4*>(xr + i);
  }
  for (int p = 0; p < a.nranks; ++p) {
    if (p == a.rank) continue;
    T* dst = reinterpret_cast<T*>(a.slots[p]) + (size_t)(parity * a.nranks + a.rank) * a.slot_stride +
             (size_t)row * a.max_hidden;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = (j * kArThreads + threadIdx.x) * 8;
      if (i < H) *reinterpret_cast<uint4*>(dst + i) = mine_raw[j];
    }
  }
  __syncthreads();
  // 2. raise the flag on every peer, then wait for every peer's flag here
  if (threadIdx.x < a.nranks && threadIdx.x != a.rank) {
    const int p = threadIdx.x;
    // the barrier above orders the CTA's row stores before this thread; the release store makes
    // them visible system-wide before the flag (no separate fence: a system-scope fence per row
    // costs microseconds)
    st_release_sys(a.flags[p] + (size_t)a.rank * a.max_rows + row, seq);
    const uint32_t* mine = a.flags[a.rank] + (size_t)p * a.max_rows + row;
    if ((int)(ld_acquire_sys(mine) - seq) < 0) {
      const unsigned long long t0 = gtimer();
      while ((int)(ld_acquire_sys(mine) - seq) < 0) {
        if (gtimer() - t0 > a.wait_ns) {
          atomicCAS(a.status, 0, 300 + p);
          break;
        }
      }
    }
  }
  __syncthreads();
  // 3. reduce in rank order (identical on every rank), add the residual, normalise
  const T* base = reinterpret_cast<const T*>(a.slots[a.rank]) + (size_t)(parity * a.nranks) * a.slot_stride +
                  (size_t)row * a.max_hidden;
  T* rr = NORM ? reinterpret_cast<T*>(a.residual) + (size_t)row * H : nullptr;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = (j * kArThreads + threadIdx.x) * 8;
    if (i < H) {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[j][k] = 0.f;
      for (int q = 0; q < a.nranks; ++q) {
        float x[8];
        if (q == a.rank) {
          const T* own = reinterpret_cast<const T*>(&mine_raw[j]);
#pragma unroll
          for (int k = 0; k < 8; ++k) x[k] = to_float(own[k]);
        } else {
          load8(base + (size_t)q * a.slot_stride + i, x);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j][k] += x[k];
      }
      if (NORM) {
        float r[8];
        load8(rr + i, r);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j][k] += r[k];
        store8(rr + i, v[j]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          v[j][k] = to_float(from_float<T>(v[j][k]));
          ss += v[j][k] * v[j][k];
        }
      } else {
        store8(reinterpret_cast<T*>(a.out) + (size_t)row * H + i, v[j]);
      }
    }
  }
  if (NORM) {
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)H + a.eps);
    const T* w = reinterpret_cast<const T*>(a.weight);
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = (j * kArThreads + threadIdx.x) * 8;
      if (i < H) {
        float wv[8];
        load8(w + i, wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          v[j][k] = to_float(from_float<T>(v[j][k] * rstd * (wv[k] + a.w_offset)));
          if (QUANT) amax = fmaxf(amax, fabsf(v[j][k]));
        }
        if (!QUANT) store8(reinterpret_cast<T*>(a.out) + (size_t)row * H + i, v[j]);
      }
    }
    if (QUANT) {
      amax = block_max(amax, scratch);
      const float scale = fmaxf(amax, 1e-8f) / kFp8Max;
      if (threadIdx.x == 0) a.out_scale[row] = scale;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int i = (j * kArThreads + threadIdx.x) * 8;
        if (i < H) *reinterpret_cast<uint2*>(a.out_q + (size_t)row * H + i) = pack8_e4m3(v[j], scale);
      }
    }
  }
  if (threadIdx.x == 0) a.seq[row] = seq;
}

template <typename T, int VPT>
void launch_ar_vpt(const ArArgs& a, cudaStream_t stream) {
  const bool norm = a.residual != nullptr, quant = a.out_q != nullptr;
  if (a.mc_rows != nullptr) {
    if (norm && quant) msgl_launch(ar_oneshot_kernel<T, true, true, VPT, true>, dim3(a.rows), dim3(kArThreads), 0, stream, a);
    else if (norm) msgl_launch(ar_oneshot_kernel<T, true, false, VPT, true>, dim3(a.rows), dim3(kArThreads), 0, stream, a);
    else msgl_launch(ar_oneshot_kernel<T, false, false, VPT, true>, dim3(a.rows), dim3(kArThreads), 0, stream, a);
    return;
  }
  if (norm && quant) msgl_launch(ar_oneshot_kernel<T, true, true, VPT>, dim3(a.rows), dim3(kArThreads), 0, stream, a);
  else if (norm) msgl_launch(ar_oneshot_kernel<T, true, false, VPT>, dim3(a.rows), dim3(kArThreads), 0, stream, a);
  else msgl_launch(ar_oneshot_kernel<T, false, false, VPT>, dim3(a.rows), dim3(kArThreads), 0, stream, a);
}

template <typename T>
int launch_ar(const ArArgs& a, cudaStream_t stream) {
  const int vpt = (a.hidden / 8 + kArThreads - 1) / kArThreads;
  if (vpt <= 1) launch_ar_vpt<T, 1>(a, stream);
  else if (vpt <= 2) launch_ar_vpt<T, 2>(a, stream);
  else if (vpt <= 3) launch_ar_vpt<T, 3>(a, stream);
  else if (vpt <= 4) launch_ar_vpt<T, 4>(a, stream);
  else if (vpt <= 6) launch_ar_vpt<T, 6>(a, stream);
  else if (vpt <= 8) launch_ar_vpt<T, 8>(a, stream);
  else if (vpt <= 16) launch_ar_vpt<T, 16>(a, stream);
  else return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("ar_oneshot");
  return MSGL_OK;
}

// ------------------------------------------------------------------------------------------
// Reduce-scatter consumer fused with residual add + RMSNorm (+ e4m3 producer) + all-gather.
//
// The row-parallel GEMM before this kernel pushed its partial rows straight into the slots of
// the rank that owns each row (gemm_tcgen05.cu, rs_* arguments). 128-row block b belongs to rank
// b % nranks and is its local block b / nranks. One CTA per owned row: wait (bounded) until all sources have delivered the
// row's 128-row block, sum the partials in rank order, add the residual (kept only for owned
// rows: the residual stream is sharded by rows between these calls), normalise, and store the
// normed row into EVERY rank's activation buffer (P2P stores). The CTA that completes a
// 128-row block raises that block's ready flag on every rank; the next column-parallel GEMM
// waits on those flags block by block in its TMA producer, so the gather overlaps its math.
// ------------------------------------------------------------------------------------------
struct RsArgs {
  const void* slots;          // local: [src][local block][128][ld]
  const uint32_t* flags;      // local: [src][flag_stride]
  void* residual;             // [M, hidden]; rows of this rank are read and rewritten
  const void* weight;
  void* out[kMaxRanks];       // per destination: 16-bit [M, hidden] (when not quantising)
  uint8_t* out_q[kMaxRanks];  // per destination: e4m3 [M, hidden]
  float* out_scale[kMaxRanks];
  uint32_t* ready[kMaxRanks];  // per destination: [M / 128]
  uint32_t* count;            // local self-resetting per-block row counters
  int* status;
  long long plane;
  int ld, rank, nranks, flag_stride, hidden;
  uint32_t rs_seq, ag_seq;
  float eps, w_offset;
  unsigned long long wait_ns;
};

// One 128-thread CTA per owned row, the row held in registers between the passes (VPT 16-byte
// vectors per thread): the row time is latency, so throughput comes from many resident rows.
constexpr int kRsThreads = 128;

template <typename T, bool QUANT, int VPT>
__global__ void __launch_bounds__(kRsThreads) rs_norm_ag_kernel(const RsArgs a) {
  pdl_enter();
  __shared__ float scratch[32];
  const int lrow = blockIdx.x;
  const int lblk = lrow >> 7;
  const int gblk = lblk * a.nranks + a.rank;
  const int grow = (gblk << 7) + (lrow & 127);
  const int H = a.hidden;
  if (threadIdx.x < a.nranks) {
    const uint32_t* f = a.flags + (size_t)threadIdx.x * a.flag_stride + lblk;
    if ((int)(ld_acquire_sys(f) - a.rs_seq) < 0) {
      const unsigned long long t0 = gtimer();
      while ((int)(ld_acquire_sys(f) - a.rs_seq) < 0) {
        if (gtimer() - t0 > a.wait_ns) {
          atomicCAS(a.status, 0, 320 + threadIdx.x);
          break;
        }
      }
    }
  }
  __syncthreads();
  const T* base = reinterpret_cast<const T*>(a.slots) + (size_t)lrow * a.ld;
  T* res = reinterpret_cast<T*>(a.residual) + (size_t)grow * H;
  const T* w = reinterpret_cast<const T*>(a.weight);
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = (j * kRsThreads + threadIdx.x) * 8;
    if (i < H) {
      load8(res + i, v[j]);
      for (int q = 0; q < a.nranks; ++q) {  // rank order: every rank would compute the same sum
        float x[8];
        load8(base + (size_t)q * a.plane + i, x);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j][k] += x[k];
      }
      store8(res + i, v[j]);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        v[j][k] = to_float(from_float<T>(v[j][k]));
        ss += v[j][k] * v[j][k];
      }
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + a.eps);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = (j * kRsThreads + threadIdx.x) * 8;
    if (i < H) {
      float wv[8];
      load8(w + i, wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        v[j][k] = to_float(from_float<T>(v[j][k] * rstd * (wv[k] + a.w_offset)));
        if (QUANT) amax = fmaxf(amax, fabsf(v[j][k]));
      }
      if (!QUANT)
        for (int p = 0; p < a.nranks; ++p) store8(reinterpret_cast<T*>(a.out[p]) + (size_t)grow * H + i, v[j]);
    }
  }
  if (QUANT) {
    amax = block_max(amax, scratch);
    const float scale = fmaxf(amax, 1e-8f) / kFp8Max;
    if (threadIdx.x < a.nranks) a.out_scale[threadIdx.x][grow] = scale;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = (j * kRsThreads + threadIdx.x) * 8;
      if (i < H) {
        const uint2 packed = pack8_e4m3(v[j], scale);
        for (int p = 0; p < a.nranks; ++p) *reinterpret_cast<uint2*>(a.out_q[p] + (size_t)grow * H + i) = packed;
      }
    }
  }
  // publish: every thread first makes its own peer stores visible system-wide (a GPU-scope release
  // does not wait for stores still on their way to another GPU); the barrier then orders them before
  // thread 0, release / acquire at GPU scope chains the rows of the block, and the CTA that
  // completes the block raises the flags
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t seen = atom_add_acq_rel_gpu(a.count + lblk, 1u);
    if (seen + 1u == 128u) {
      a.count[lblk] = 0u;
      for (int p = 0; p < a.nranks; ++p) st_release_sys(a.ready[p] + gblk, a.ag_seq);
    }
  }
}

// Bounded wait until flags[0..n) have all reached `seq`: for consumers of gathered rows that
// are not a GEMM with its own per-block wait.
__global__ void wait_flags_kernel(const uint32_t* flags, int n, uint32_t seq, unsigned long long wait_ns,
                                  int* status) {
  pdl_enter();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    if ((int)(ld_acquire_sys(flags + i) - seq) >= 0) continue;
    const unsigned long long t0 = gtimer();
    while ((int)(ld_acquire_sys(flags + i) - seq) < 0) {
      if (gtimer() - t0 > wait_ns) {
        atomicCAS(status, 0, 340);
        break;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// Vocabulary-parallel arg-max: every rank holds the logits of its vocabulary shard. One CTA per
// row reduces the shard to (max, global index), stores the pair into every rank's slot, raises
// the row's sequence flag there, waits (bounded) for the peers' pairs and picks the winner.
// Ranks own ascending index ranges, so "first maximum in rank order" is the lowest index, the
// same tie rule as an arg-max over the full row. Replaces gathering rows x vocabulary logits.
// ------------------------------------------------------------------------------------------
struct ArgmaxArgs {
  const float* logits;       // [rows, ld] this rank's shard
  long long ld;
  int len;                   // valid columns of the shard (0: this rank holds none)
  int start;                 // global index of column 0
  int32_t* out;              // [rows] winning token ids
  uint2* pairs[kMaxRanks];   // pairs[p]: rank p's region [2 (parity)][src][max_rows]
  uint32_t* flags[kMaxRanks];  // flags[p]: rank p's region [src][max_rows]
  uint32_t* seq;             // local per-row sequence counters
  int* status;
  int rank, nranks, max_rows;
  unsigned long long wait_ns;
};

__global__ void __launch_bounds__(256) argmax_exchange_kernel(const ArgmaxArgs a) {
  pdl_enter();
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
  __shared__ uint2 s_peer[kMaxRanks];
  const int row = blockIdx.x;
  const uint32_t seq = a.seq[row] + 1u;
  const int parity = (int)(seq & 1u);
  const float* x = a.logits + (size_t)row * a.ld;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < a.len; i += blockDim.x) {
    const float v = x[i];
    if (v > best || (v == best && i < idx)) { best = v; idx = i; }
  }
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (s_val[w] > best || (s_val[w] == best && s_idx[w] < idx)) { best = s_val[w]; idx = s_idx[w]; }
    const uint2 mine = make_uint2(__float_as_uint(best), (uint32_t)(a.len > 0 && idx != 0x7fffffff ? idx + a.start : 0));
    for (int p = 0; p < a.nranks; ++p)
      a.pairs[p][((size_t)parity * a.nranks + a.rank) * a.max_rows + row] = mine;
    for (int p = 0; p < a.nranks; ++p) st_release_sys(a.flags[p] + (size_t)a.rank * a.max_rows + row, seq);
  }
  if (threadIdx.x < a.nranks) {
    const int p = threadIdx.x;
    const uint32_t* f = a.flags[a.rank] + (size_t)p * a.max_rows + row;
    if ((int)(ld_acquire_sys(f) - seq) < 0) {
      const unsigned long long t0 = gtimer();
      while ((int)(ld_acquire_sys(f) - seq) < 0) {
        if (gtimer() - t0 > a.wait_ns) {
          atomicCAS(a.status, 0, 360 + p);
          break;
        }
      }
    }
    const volatile uint32_t* src =
        reinterpret_cast<const volatile uint32_t*>(&a.pairs[a.rank][((size_t)parity * a.nranks + p) * a.max_rows + row]);
    s_peer[p] = make_uint2(src[0], src[1]);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float bv = __uint_as_float(s_peer[0].x);
    uint32_t bi = s_peer[0].y;
    for (int p = 1; p < a.nranks; ++p) {
      const float v = __uint_as_float(s_peer[p].x);
      if (v > bv) { bv = v; bi = s_peer[p].y; }
    }
    a.out[row] = (int32_t)bi;
    a.seq[row] = seq;
  }
}

template <typename T, int VPT>
void launch_rs_vpt(const RsArgs& a, int owned_rows, bool quant, cudaStream_t stream) {
  if (quant) msgl_launch(rs_norm_ag_kernel<T, true, VPT>, dim3(owned_rows), dim3(kRsThreads), 0, stream, a);
  else msgl_launch(rs_norm_ag_kernel<T, false, VPT>, dim3(owned_rows), dim3(kRsThreads), 0, stream, a);
}

template <typename T>
int launch_rs(const RsArgs& a, int owned_rows, bool quant, cudaStream_t stream) {
  const int vpt = (a.hidden / 8 + kRsThreads - 1) / kRsThreads;
  if (vpt <= 1) launch_rs_vpt<T, 1>(a, owned_rows, quant, stream);
  else if (vpt <= 2) launch_rs_vpt<T, 2>(a, owned_rows, quant, stream);
  else if (vpt <= 3) launch_rs_vpt<T, 3>(a, owned_rows, quant, stream);
  else if (vpt <= 4) launch_rs_vpt<T, 4>(a, owned_rows, quant, stream);
  else if (vpt <= 6) launch_rs_vpt<T, 6>(a, owned_rows, quant, stream);
  else if (vpt <= 8) launch_rs_vpt<T, 8>(a, owned_rows, quant, stream);
  else if (vpt <= 16) launch_rs_vpt<T, 16>(a, owned_rows, quant, stream);
  else return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("rs_norm_ag");
  return MSGL_OK;
}

}  // namespace

// ---------------------------------------------------------------- symmetric memory plumbing
MSGL_API void* msgl_symm_alloc(long long bytes) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) { msgl_set_error("symm_alloc", e); return nullptr; }
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) { msgl_set_error("symm_alloc memset", e); cudaFree(p); return nullptr; }
  return p;
}
MSGL_API int msgl_symm_free(void* p) {
  cudaError_t e = cudaFree(p);
  if (e != cudaSuccess) { msgl_set_error("symm_free", e); return MSGL_CUDA_ERROR; }
  return MSGL_OK;
}
MSGL_API int msgl_ipc_get_handle(void* p, void* out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { msgl_set_error("ipc_get_handle", e); return MSGL_CUDA_ERROR; }
  memcpy(out64, &h, sizeof(h));
  return MSGL_OK;
}
MSGL_API void* msgl_ipc_open(const void* handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { msgl_set_error("ipc_open", e); return nullptr; }
  return p;
}
MSGL_API int msgl_ipc_close(void* p) {
  cudaError_t e = cudaIpcCloseMemHandle(p);
  if (e != cudaSuccess) { msgl_set_error("ipc_close", e); return MSGL_CUDA_ERROR; }
  return MSGL_OK;
}

// slots / flags: arrays of `nranks` device pointers (this rank's own buffer at index `rank`).
// residual == nullptr: plain all-reduce into `out`. out_q != nullptr: e4m3 row + scale.
MSGL_API int msgl_ar_oneshot(const void* x, void* residual, const void* weight, void* out, void* out_q,
                             void* out_scale, void* const* slots, void* const* flags, void* seq, int rank,
                             int nranks, int rows, int hidden, int max_rows, int max_hidden, float eps,
                             int plus_one, long long wait_us, int dtype, cudaStream_t stream) {
  if (rows == 0) return MSGL_OK;
  if (nranks > kMaxRanks || rows > max_rows || hidden > max_hidden || hidden % 8 || hidden > 16 * 8 * 128) {
    msgl_set_error_text("ar_oneshot: message does not fit the symmetric slots");
    return MSGL_BAD_ARG;
  }
  ArArgs a;
  a.x = x; a.residual = residual; a.weight = weight; a.out = out;
  a.out_q = (uint8_t*)out_q; a.out_scale = (float*)out_scale;
  for (int p = 0; p < nranks; ++p) { a.slots[p] = slots[p]; a.flags[p] = (uint32_t*)flags[p]; }
  a.seq = (uint32_t*)seq;
  int* status = nullptr;
  cudaGetSymbolAddress((void**)&status, g_comm_status);
  a.status = status;
  a.rank = rank; a.nranks = nranks; a.rows = rows; a.hidden = hidden; a.max_rows = max_rows;
  a.max_hidden = max_hidden;
  a.slot_stride = (long long)max_rows * max_hidden;
  a.eps = eps; a.w_offset = plus_one ? 1.f : 0.f;
  a.wait_ns = (unsigned long long)wait_us * 1000ull;
  a.my_rows = nullptr; a.mc_rows = nullptr; a.my_count = nullptr; a.mc_count = nullptr;
  if (dtype == MSGL_BF16) return launch_ar<__nv_bfloat16>(a, stream);
  if (dtype == MSGL_F16) return launch_ar<__half>(a, stream);
  return MSGL_BAD_ARG;
}

// The same fused all-reduce (+ residual add + RMSNorm (+ e4m3)) with the reduction done inside the
// NVSwitch. `local` / `mc` are this rank's address and the multicast address of one symmetric
// buffer laid out as [counters: max_rows u32, padded to 256 bytes][rows: 2 x max_rows x max_hidden
// 16-bit]; the buffer starts zeroed. Every rank stores only its own rows (locally) and reads the
// sum once through the multicast mapping: per-rank NVLink traffic is one row set in, however many
// ranks there are. `seq` [max_rows] are local per-row call counters (device-resident, so a
// captured graph replays unchanged).
MSGL_API int msgl_ar_nvls(const void* x, void* residual, const void* weight, void* out, void* out_q, void* out_scale,
                          void* local, void* mc, void* seq, int rank, int nranks, int rows, int hidden, int max_rows,
                          int max_hidden, float eps, int plus_one, long long wait_us, int dtype,
                          cudaStream_t stream) {
  if (rows == 0) return MSGL_OK;
  if (local == nullptr || mc == nullptr || nranks > kMaxRanks || rows > max_rows || hidden > max_hidden || hidden % 8 ||
      max_hidden % 8 || hidden > 16 * 8 * 128) {
    msgl_set_error_text("ar_nvls: message does not fit the symmetric buffer");
    return MSGL_BAD_ARG;
  }
  const size_t count_bytes = ((size_t)max_rows * 4 + 255) / 256 * 256;
  ArArgs a;
  a.x = x; a.residual = residual; a.weight = weight; a.out = out;
  a.out_q = (uint8_t*)out_q; a.out_scale = (float*)out_scale;
  for (int p = 0; p < kMaxRanks; ++p) { a.slots[p] = nullptr; a.flags[p] = nullptr; }
  a.seq = (uint32_t*)seq;
  int* status = nullptr;
  cudaGetSymbolAddress((void**)&status, g_comm_status);
  a.status = status;
  a.rank = rank; a.nranks = nranks; a.rows = rows; a.hidden = hidden; a.max_rows = max_rows;
  a.max_hidden = max_hidden;
  a.slot_stride = (long long)max_rows * max_hidden;
  a.eps = eps; a.w_offset = plus_one ? 1.f : 0.f;
  a.wait_ns = (unsigned long long)wait_us * 1000ull;
  a.my_count = (uint32_t*)local;
  a.mc_count = (uint32_t*)mc;
  a.my_rows = (unsigned char*)local + count_bytes;
  a.mc_rows = (const unsigned char*)mc + count_bytes;
  if (dtype == MSGL_BF16) return launch_ar<__nv_bfloat16>(a, stream);
  if (dtype == MSGL_F16) return launch_ar<__half>(a, stream);
  return MSGL_BAD_ARG;
}

// Consumer of a GEMM -> reduce-scatter push (see rs_norm_ag_kernel). slots / flags / count are
// this rank's own regions; out / out_q / out_scale / ready are arrays of `nranks` peer-mapped
// pointers. quant != 0 writes e4m3 rows + scales, else 16-bit rows.
MSGL_API int msgl_rs_norm_ag(const void* slots, const void* flags, void* residual, const void* weight,
                             void* const* out, void* const* out_q, void* const* out_scale, void* const* ready,
                             void* count, long long plane, int ld, int rank, int nranks, int rows,
                             int flag_stride, int hidden, unsigned int rs_seq, unsigned int ag_seq, float eps, int plus_one,
                             int quant, long long wait_us, int dtype, cudaStream_t stream) {
  if (nranks > kMaxRanks || hidden % 8 || hidden > 16 * 8 * 128 || rows <= 0 || rows % 128) {
    msgl_set_error_text("rs_norm_ag: unsupported shape");
    return MSGL_BAD_ARG;
  }
  const int blocks = rows / 128;
  const int owned_blocks = (blocks - rank + nranks - 1) / nranks;  // blocks rank, rank + nranks, ...
  if (owned_blocks <= 0) return MSGL_OK;
  const int owned_rows = owned_blocks * 128;
  RsArgs a;
  a.slots = slots; a.flags = (const uint32_t*)flags; a.residual = residual; a.weight = weight;
  for (int p = 0; p < nranks; ++p) {
    a.out[p] = out ? out[p] : nullptr;
    a.out_q[p] = out_q ? (uint8_t*)out_q[p] : nullptr;
    a.out_scale[p] = out_scale ? (float*)out_scale[p] : nullptr;
    a.ready[p] = (uint32_t*)ready[p];
  }
  a.count = (uint32_t*)count;
  int* status = nullptr;
  cudaGetSymbolAddress((void**)&status, g_comm_status);
  a.status = status;
  a.plane = plane; a.ld = ld; a.rank = rank; a.nranks = nranks; a.flag_stride = flag_stride; a.hidden = hidden;
  a.rs_seq = rs_seq; a.ag_seq = ag_seq; a.eps = eps; a.w_offset = plus_one ? 1.f : 0.f;
  a.wait_ns = (unsigned long long)wait_us * 1000ull;
  if (dtype == MSGL_BF16) return launch_rs<__nv_bfloat16>(a, owned_rows, quant != 0, stream);
  if (dtype == MSGL_F16) return launch_rs<__half>(a, owned_rows, quant != 0, stream);
  return MSGL_BAD_ARG;
}

// pairs / flags: arrays of `nranks` peer-mapped region bases; seq: local [max_rows] counters.
MSGL_API int msgl_argmax_exchange(const void* logits, long long ld, int rows, int len, int start, void* out,
                                  void* const* pairs, void* const* flags, void* seq, int rank, int nranks,
                                  int max_rows, long long wait_us, cudaStream_t stream) {
  if (rows == 0) return MSGL_OK;
  if (nranks > kMaxRanks || rows > max_rows || len < 0) {
    msgl_set_error_text("argmax_exchange: unsupported shape");
    return MSGL_BAD_ARG;
  }
  ArgmaxArgs a;
  a.logits = (const float*)logits; a.ld = ld; a.len = len; a.start = start; a.out = (int32_t*)out;
  for (int p = 0; p < nranks; ++p) { a.pairs[p] = (uint2*)pairs[p]; a.flags[p] = (uint32_t*)flags[p]; }
  a.seq = (uint32_t*)seq;
  int* status = nullptr;
  cudaGetSymbolAddress((void**)&status, g_comm_status);
  a.status = status;
  a.rank = rank; a.nranks = nranks; a.max_rows = max_rows;
  a.wait_ns = (unsigned long long)wait_us * 1000ull;
  msgl_launch(argmax_exchange_kernel, dim3(rows), dim3(256), 0, stream, a);
  MSGL_CHECK_LAUNCH("argmax_exchange");
  return MSGL_OK;
}

MSGL_API int msgl_wait_flags(const void* flags, int n, unsigned int seq, long long wait_us, cudaStream_t stream) {
  if (n <= 0) return MSGL_OK;
  int* status = nullptr;
  cudaGetSymbolAddress((void**)&status, g_comm_status);
  msgl_launch(wait_flags_kernel, dim3(1), dim3(256), 0, stream, (const uint32_t*)flags, n, seq, (unsigned long long)wait_us * 1000ull,
                                           status);
  MSGL_CHECK_LAUNCH("wait_flags");
  return MSGL_OK;
}

MSGL_API int msgl_comm_status(int reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_comm_status, sizeof(int));
  if (reset && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_comm_status, &z, sizeof(int));
  }
  return v;
}
