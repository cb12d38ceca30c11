// Causal prefill / extend attention on the tcgen05 tensor cores (head_dim 128, even GQA group).
//
// The reference's prefill kernels (flash_prefill, flash_prefill_paged[_fp8];
// python/minisgl/attention/hip.py:670-792, python/minisgl/attention/rdna4.py:419-503) walk the
// page table inside the attention loop. Here a step is two launches:
//
//   1. kv_gather_kernel copies the K and V rows that this step's requests can see out of the
//      paged pool into a dense 16-bit scratch: K as [Hk][T][128], V transposed as [Hk][128][T],
//      every request starting on a multiple of 128 tokens, rows past a request's length zeroed.
//      fp8 pools are widened here (e4m3 -> 16 bit is exact; the per-head descales are applied
//      to the fp32 scores / output, not to the data). The copy moves a few bytes per token while
//      attention does ~hundreds of FLOP per byte, so it is noise next to the main kernel, and it
//      leaves the main kernel with plain 2-D tensor maps and K-major operands only.
//   2. attn_prefill_tc_kernel: one CTA per (128 query positions of one request, two query heads
//      of one KV head). S = Q K^T and O += P_j V_j are tcgen05.mma (kind::f16, M = N = 128) with
//      S and the output accumulator in tensor memory (2 x 128 + 2 x 128 columns); warp 0 is the
//      TMA producer (Q once, then a 3-slot ring of K_j / V_j tiles), warp 1 issues the MMAs, and
//      two groups of four warps (warps 4-7, 8-11) own one head each: they pull a block of S into
//      registers with tcgen05.ld (which frees S for the next QK^T at once), keep the online-
//      softmax state, rescale O in tensor memory when the running maximum has to move
//      (tcgen05.ld / st, rare), and hand P_j to the MMA through shared memory in the swizzled
//      K-major layout it reads. The two heads alternate on the tensor pipe, so one group's
//      softmax overlaps the other's MMAs. setmaxnreg moves the idle warps' registers to the
//      softmax groups.
//
// A row's result does not depend on which other rows share its tile or on how a prompt was
// chunked: KV blocks are absolute (0, 128, ...), visited in ascending order, and a block that
// is fully masked for a row changes nothing (alpha = 1, P = 0).
#include "common.cuh"
#include "ptx.cuh"

#include <string>

using namespace msgl;
using namespace msgl::ptx;

namespace {

constexpr int kD = 128;            // head dim
constexpr int kTile = 128;         // query rows per head tile, KV rows per block
constexpr int kPanel = 16384;      // 128 rows x 128 bytes (64 16-bit columns), 128B-swizzled
constexpr int kTcThreads = 384;   // warps 0-3: TMA / MMA / two idle; warps 4-7, 8-11: one head each
constexpr float kLog2eTc = 1.4426950408889634f;

struct TcItem {        // one per (request, block of 128 query positions); eight int32
  int q_row0;          // first row of the tile in the packed q / out tensors
  int q_rows;          // valid rows (<= 128)
  int q_pos0;          // absolute position of the first row
  int kv_off;          // first scratch row of the request (multiple of 128)
  int n_blocks;        // KV blocks of 128 the tile can see
  int req, pad0, pad1;
};

struct TcArgs {
  const TcItem* items;
  int n_items, pairs;  // pairs = Hq / 2
  int Hq, Hk;
  long long t_cap;     // scratch rows per KV head
  void* out;
  const float* k_scale;
  const float* v_scale;
  float scale;
  int* status;
};

__device__ int g_attn_tc_status = 0;

struct TcSmem {
  static constexpr int off_q = 0;                       // [2 heads][2 panels]
  static constexpr int off_p = 4 * kPanel;              // [2 heads][2 panels]
  static constexpr int off_kv = 8 * kPanel;             // [3 slots][2 panels]
  static constexpr int off_bar = 14 * kPanel;
  static constexpr int n_bars = 1 + 3 + 3 + 2 * 5;
  static constexpr int bytes = off_bar + 256 + 1024;    // + slack to align the base to 1024
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <typename T> __device__ __forceinline__ uint32_t pack2_tc(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2_tc<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2_tc<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T> struct TcFmt;
template <> struct TcFmt<__half> { static constexpr uint32_t fmt = 0; };
template <> struct TcFmt<__nv_bfloat16> { static constexpr uint32_t fmt = 1; };

// ------------------------------------------------------------------------------------------
// 1. Pool -> dense scratch. grid (scratch rows / 64, Hk), 256 threads.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t e4m3x2_to_h2(uint32_t x) {
  uint32_t r;
  asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(r) : "r"(x));
  return r;
}
template <typename T> __device__ __forceinline__ uint32_t widen2(uint32_t two_bytes) {
  const uint32_t h = e4m3x2_to_h2(two_bytes);
  if constexpr (sizeof(T) == 2 && TcFmt<T>::fmt == 0) {
    return h;
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
    return pack2_tc<__nv_bfloat16>(f.x, f.y);
  }
}
template <typename T> __device__ __forceinline__ uint4 widen8(uint2 b) {
  uint4 o;
  o.x = widen2<T>(b.x & 0xFFFFu);
  o.y = widen2<T>(b.x >> 16);
  o.z = widen2<T>(b.y & 0xFFFFu);
  o.w = widen2<T>(b.y >> 16);
  return o;
}

template <typename T, bool KV8>
__global__ void __launch_bounds__(256)
kv_gather_kernel(const void* __restrict__ k_pool, const void* __restrict__ v_pool, T* __restrict__ kc,
                 T* __restrict__ vt, const int* __restrict__ blk_req, const int* __restrict__ req_info,
                 const int* __restrict__ block_table, int bt_stride, int Hk, int page_size, long long t_cap) {
  pdl_enter();
  __shared__ __align__(16) T vs[64][kD + 8];
  const int t0 = blockIdx.x * 64, h = blockIdx.y;
  const int req = blk_req[t0 >> 7];
  const int kv_off = req_info[2 * req], kv_len = req_info[2 * req + 1];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int id = threadIdx.x + i * 256;
    const int tt = id >> 4, c = id & 15;
    const int tok = t0 + tt - kv_off;
    uint4 kq = make_uint4(0, 0, 0, 0), vq = make_uint4(0, 0, 0, 0);
    if (tok >= 0 && tok < kv_len) {
      const int page = block_table[(long long)req * bt_stride + tok / page_size];
      const long long src = (((long long)page * Hk + h) * page_size + tok % page_size) * kD + c * 8;
      if constexpr (KV8) {
        kq = widen8<T>(*reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(k_pool) + src));
        vq = widen8<T>(*reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(v_pool) + src));
      } else {
        kq = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(k_pool) + src);
        vq = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(v_pool) + src);
      }
    }
    *reinterpret_cast<uint4*>(kc + ((long long)h * t_cap + t0 + tt) * kD + c * 8) = kq;
    *reinterpret_cast<uint4*>(&vs[tt][c * 8]) = vq;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int id = threadIdx.x + i * 256;
    const int d = id >> 3, ch = id & 7;
    const uint16_t* col = reinterpret_cast<const uint16_t*>(&vs[ch * 8][d]);
    constexpr int rs = kD + 8;
    uint4 o;
    o.x = (uint32_t)col[0 * rs] | ((uint32_t)col[1 * rs] << 16);
    o.y = (uint32_t)col[2 * rs] | ((uint32_t)col[3 * rs] << 16);
    o.z = (uint32_t)col[4 * rs] | ((uint32_t)col[5 * rs] << 16);
    o.w = (uint32_t)col[6 * rs] | ((uint32_t)col[7 * rs] << 16);
    *reinterpret_cast<uint4*>(vt + ((long long)h * kD + d) * t_cap + t0 + ch * 8) = o;
  }
}

// ------------------------------------------------------------------------------------------
// 2. The attention kernel. grid = items x head pairs (heaviest items first), 320 threads.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kTcThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                       const __grid_constant__ CUtensorMap tma_v, const TcArgs args) {
  pdl_enter();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t s_base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (s_base - raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int item_idx = blockIdx.x / args.pairs, pair = blockIdx.x - item_idx * args.pairs;
  const TcItem it = args.items[item_idx];
  const int head0 = pair * 2;
  const int hk = head0 / (args.Hq / args.Hk);
  const int nb = it.n_blocks;

  const uint32_t q_s = s_base + TcSmem::off_q, p_s = s_base + TcSmem::off_p, kv_s = s_base + TcSmem::off_kv;
  const uint32_t bars = s_base + TcSmem::off_bar;
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
  auto q_full = [&]() { return bar(0); };
  auto kv_full = [&](int s) { return bar(1 + s); };
  auto kv_empty = [&](int s) { return bar(4 + s); };
  auto s_full = [&](int t) { return bar(7 + 5 * t); };
  auto s_free = [&](int t) { return bar(8 + 5 * t); };
  auto p_full = [&](int t) { return bar(9 + 5 * t); };
  auto o_full = [&](int t) { return bar(10 + 5 * t); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + TcSmem::off_bar + 8 * TcSmem::n_bars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + TcSmem::off_bar + 8 * TcSmem::n_bars + 8);

  if (threadIdx.x == 0) {
    mbar_init(q_full(), 1);
    for (int s = 0; s < 3; ++s) { mbar_init(kv_full(s), 1); mbar_init(kv_empty(s), 1); }
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(s_free(t), 128);
      mbar_init(p_full(t), 128);
      mbar_init(o_full(t), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_q);
    prefetch_tensormap(&tma_k);
    prefetch_tensormap(&tma_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The two softmax groups keep a 128-float output row per thread; the first warpgroup gives
  // them its registers (3 warps per scheduler: 56 + 2 x 224 registers x 32 lanes fit 16384).
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full(), 4 * kPanel);
      for (int t = 0; t < 2; ++t)
        for (int p = 0; p < 2; ++p)
          tma_load_3d(q_s + (t * 2 + p) * kPanel, &tma_q, q_full(), 64 * p, head0 + t, it.q_row0);
      const int k_row0 = (int)((long long)hk * args.t_cap) + it.kv_off;
      for (int i = 0; i < 2 * nb && !*abort_flag; ++i) {
        const int slot = i % 3, n = i / 3, j = i >> 1;
        if (!mbar_wait(kv_empty(slot), (uint32_t)((n & 1) ^ 1), abort_flag, args.status, 201)) break;
        mbar_expect_tx(kv_full(slot), 2 * kPanel);
        const uint32_t dst = kv_s + slot * 2 * kPanel;
        if ((i & 1) == 0) {
          tma_load_2d(dst, &tma_k, kv_full(slot), 0, k_row0 + j * kTile);
          tma_load_2d(dst + kPanel, &tma_k, kv_full(slot), 64, k_row0 + j * kTile);
        } else {
          tma_load_2d(dst, &tma_v, kv_full(slot), it.kv_off + j * kTile, hk * kD);
          tma_load_2d(dst + kPanel, &tma_v, kv_full(slot), it.kv_off + j * kTile + 64, hk * kD);
        }
      }
      if (*abort_flag) {  // let copies that are still in flight land before the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_dense(TcFmt<T>::fmt, TcFmt<T>::fmt, 128, 128);
      auto issue_s = [&](int t, uint32_t k_tile) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          mma_f16(tmem_base + t * 128, smem_desc_sw128(q_s + (t * 2 + (kk >> 2)) * kPanel + (kk & 3) * 32),
                  smem_desc_sw128(k_tile + (kk >> 2) * kPanel + (kk & 3) * 32), idesc, kk > 0 ? 1u : 0u);
      };
      auto issue_pv = [&](int t, uint32_t v_tile, bool first) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          mma_f16(tmem_base + 256 + t * 128, smem_desc_sw128(p_s + (t * 2 + (kk >> 2)) * kPanel + (kk & 3) * 32),
                  smem_desc_sw128(v_tile + (kk >> 2) * kPanel + (kk & 3) * 32), idesc, (kk > 0 || !first) ? 1u : 0u);
      };
      bool ok = mbar_wait(q_full(), 0, abort_flag, args.status, 202) &&
                mbar_wait(kv_full(0), 0, abort_flag, args.status, 203);
      if (ok) {
        tc_fence_after();
        issue_s(0, kv_s);
        tc_commit(s_full(0));
        issue_s(1, kv_s);
        tc_commit(s_full(1));
        tc_commit(kv_empty(0));
      }
      for (int j = 0; ok && j < nb; ++j) {
        const bool next = j + 1 < nb;
        const int iv = 2 * j + 1, ik = 2 * j + 2;
        if (next && !mbar_wait(kv_full(ik % 3), (uint32_t)((ik / 3) & 1), abort_flag, args.status, 204)) break;
        if (!mbar_wait(kv_full(iv % 3), (uint32_t)((iv / 3) & 1), abort_flag, args.status, 205)) break;
        for (int t = 0; t < 2; ++t) {
          if (next) {
            if (!mbar_wait(s_free(t), (uint32_t)(j & 1), abort_flag, args.status, 206)) { ok = false; break; }
            tc_fence_after();
            issue_s(t, kv_s + (ik % 3) * 2 * kPanel);
            tc_commit(s_full(t));
          }
          if (!mbar_wait(p_full(t), (uint32_t)(j & 1), abort_flag, args.status, 207)) { ok = false; break; }
          tc_fence_after();
          issue_pv(t, kv_s + (iv % 3) * 2 * kPanel, j == 0);
          tc_commit(o_full(t));
        }
        if (!ok) break;
        if (next) tc_commit(kv_empty(ik % 3));
        tc_commit(kv_empty(iv % 3));
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ---------------------------------------------------------------- softmax / output groups
    const int t = (warp - 4) >> 2;               // head of the pair
    const int quarter = warp & 3;                // tensor-memory lanes this warp may read
    const int row = quarter * 32 + lane;
    const int head = head0 + t;
    const int q_pos = it.q_pos0 + row;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_base + t * 128, o_addr = lane_base + 256 + t * 128;
    const uint32_t p_row = p_s + t * 2 * kPanel + row * 128;
    const uint32_t swz = (uint32_t)(row & 7);
    const float sl2 = args.scale * kLog2eTc * (args.k_scale != nullptr ? args.k_scale[hk] : 1.f);

    // The output row accumulates in tensor memory across KV blocks. The running maximum is only
    // raised when a block exceeds it by more than 2^8 (probabilities then stay below 256, exact
    // enough in 16 bits and harmless in the fp32 row sum), so rescaling the accumulator - read,
    // multiply, write back - is rare after the first blocks. The decision depends on the row's
    // own history over absolute KV blocks only.
    float m = -INFINITY, l = 0.f;
    uint32_t s[4][32];
    bool ok = true;
    for (int j = 0; j < nb; ++j) {
      const int kv0 = j * kTile;
      const bool masked = kv0 + kTile - 1 > it.q_pos0;   // the block reaches past some row's position
      if (!mbar_wait(s_full(t), (uint32_t)(j & 1), abort_flag, args.status, 209)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(s_addr + c * 32, s[c]);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(s_free(t));                             // S is in registers: the next QK^T may start
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (masked && kv0 + c * 32 + i > q_pos) s[c][i] = 0xFF800000u;   // -inf
          mx = fmaxf(mx, __uint_as_float(s[c][i]));
        }
      }
      const bool grow = (mx - m) * sl2 > 8.f;             // false when both are -inf (NaN compares false)
      float alpha = 1.f;
      if (grow) {
        alpha = ex2f((m - mx) * sl2);                     // m = -inf on the first block: 0
        m = mx;
        l *= alpha;
      }
      if (j > 0) {
        // P V of the previous block is complete: the P buffer is free and O may be rescaled
        if (!mbar_wait(o_full(t), (uint32_t)((j - 1) & 1), abort_flag, args.status, 210)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xFFFFFFFFu, grow)) {
          uint32_t r[32];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tmem_ld_32x32b_x32(o_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x32(o_addr + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      // probabilities -> shared memory (K-major, 128-byte swizzle), row sum
      const float mb = (m == -INFINITY ? 0.f : m) * sl2;
      float l_blk = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t panel = p_row + (uint32_t)(c >> 1) * kPanel;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = g * 8 + e * 2;
            const float p0 = ex2f(fmaf(__uint_as_float(s[c][i]), sl2, -mb));
            const float p1 = ex2f(fmaf(__uint_as_float(s[c][i + 1]), sl2, -mb));
            l_blk += p0 + p1;
            pk[e] = pack2_tc<T>(p0, p1);
          }
          const uint32_t u = (uint32_t)((c & 1) * 4 + g);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(panel + ((u ^ swz) << 4)), "r"(pk[0]),
                       "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                       : "memory");
        }
      }
      l += l_blk;
      tc_fence_before();
      fence_proxy_async();
      mbar_arrive(p_full(t));
    }
    if (ok && nb > 0 && mbar_wait(o_full(t), (uint32_t)((nb - 1) & 1), abort_flag, args.status, 211)) {
      tc_fence_after();
      const float inv = (l > 0.f ? 1.f / l : 0.f) * (args.v_scale != nullptr ? args.v_scale[hk] : 1.f);
      T* dst = reinterpret_cast<T*>(args.out) + ((long long)(it.q_row0 + row) * args.Hq + head) * kD;
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(o_addr + c * 32, s[c]);
      tmem_ld_wait();
      if (row < it.q_rows) {
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const uint32_t* o = &s[c >> 2][(c & 3) * 8];
          uint4 v;
          v.x = pack2_tc<T>(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv);
          v.y = pack2_tc<T>(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv);
          v.z = pack2_tc<T>(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv);
          v.w = pack2_tc<T>(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv);
          *reinterpret_cast<uint4*>(dst + 8 * c) = v;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

bool encode_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                const cuuint32_t* box, const char* what) {
  msgl_encode_tiled_fn enc = msgl_get_encode_tiled();
  if (enc == nullptr) return false;
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    msgl_set_error_text((std::string("prefill attention: cuTensorMapEncodeTiled(") + what + ") failed with code " +
                         std::to_string((int)r)).c_str());
    return false;
  }
  return true;
}

template <typename T>
int launch_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const TcArgs& a,
              cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TcSmem::bytes);
    if (e != cudaSuccess) { msgl_set_error("prefill attention smem attribute", e); return MSGL_CUDA_ERROR; }
    configured = true;
  }
  msgl_launch(attn_prefill_tc_kernel<T>, dim3(a.n_items * a.pairs), dim3(kTcThreads), TcSmem::bytes, stream, mq, mk, mv, a);
  MSGL_CHECK_LAUNCH("attn_prefill_tc");
  return MSGL_OK;
}

}  // namespace

// Causal prefill / extend attention for one layer. `kc` / `vt` are scratch buffers of
// hk * t_cap * 128 16-bit elements each; `items` (n_items x 8 int32), `blk_req` (t_pad / 128
// int32) and `req_info` (B x 2 int32: scratch offset, KV length) describe the step and are
// built once per step by the caller. q and out are [total_q, hq, 128] with rows
// `q_row_stride` / hq * 128 elements apart.
MSGL_API int msgl_attn_prefill_tc(const void* q, long long q_row_stride, void* out, const void* k_pool,
                                  const void* v_pool, void* kc, void* vt, long long t_cap, int t_pad,
                                  const void* items, int n_items, const void* blk_req, const void* req_info,
                                  const void* block_table, int bt_stride, const void* k_scale, const void* v_scale,
                                  int total_q, int hq, int hk, int page_size, int kv_fp8, float scale, int dtype,
                                  cudaStream_t stream) {
  if (n_items == 0 || total_q == 0) return MSGL_OK;
  if (hq % hk || (hq / hk) % 2 || t_cap % 128 || t_pad % 128 || t_pad > t_cap || (q_row_stride % 8) ||
      (dtype != MSGL_BF16 && dtype != MSGL_F16)) {
    msgl_set_error_text("prefill attention: needs head_dim 128, an even GQA group, 16-bit q and a scratch of whole blocks");
    return MSGL_BAD_ARG;
  }
  CUtensorMap mq, mk, mv;
  {
    cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)hq, (cuuint64_t)total_q};
    cuuint64_t strides[2] = {(cuuint64_t)kD * 2, (cuuint64_t)q_row_stride * 2};
    cuuint32_t box[3] = {64, 1, 128};
    if (!encode_map(&mq, q, 3, dims, strides, box, "q")) return MSGL_CUDA_ERROR;
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)kD, (cuuint64_t)hk * (cuuint64_t)t_cap};
    cuuint64_t strides[1] = {(cuuint64_t)kD * 2};
    cuuint32_t box[2] = {64, 128};
    if (!encode_map(&mk, kc, 2, dims, strides, box, "k")) return MSGL_CUDA_ERROR;
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)t_cap, (cuuint64_t)hk * kD};
    cuuint64_t strides[1] = {(cuuint64_t)t_cap * 2};
    cuuint32_t box[2] = {64, 128};
    if (!encode_map(&mv, vt, 2, dims, strides, box, "v")) return MSGL_CUDA_ERROR;
  }
  int* status = nullptr;
  cudaGetSymbolAddress((void**)&status, g_attn_tc_status);
  const dim3 ggrid(t_pad / 64, hk);
#define GATHER(T, F8)                                                                                              \
  msgl_launch(kv_gather_kernel<T, F8>, dim3(ggrid), dim3(256), 0, stream, k_pool, v_pool, (T*)kc, (T*)vt, (const int*)blk_req,          \
                                                     (const int*)req_info, (const int*)block_table, bt_stride, hk, \
                                                     page_size, t_cap)
  if (dtype == MSGL_BF16) { if (kv_fp8) GATHER(__nv_bfloat16, true); else GATHER(__nv_bfloat16, false); }
  else { if (kv_fp8) GATHER(__half, true); else GATHER(__half, false); }
#undef GATHER
  MSGL_CHECK_LAUNCH("kv_gather");
  TcArgs a;
  a.items = (const TcItem*)items; a.n_items = n_items; a.pairs = hq / 2; a.Hq = hq; a.Hk = hk; a.t_cap = t_cap;
  a.out = out; a.k_scale = (const float*)k_scale; a.v_scale = (const float*)v_scale; a.scale = scale;
  a.status = status;
  if (dtype == MSGL_BF16) return launch_tc<__nv_bfloat16>(mq, mk, mv, a, stream);
  return launch_tc<__half>(mq, mk, mv, a, stream);
}

MSGL_API int msgl_attn_tc_status(int reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_attn_tc_status, sizeof(int));
  if (reset && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_attn_tc_status, &z, sizeof(int));
  }
  return v;
}
