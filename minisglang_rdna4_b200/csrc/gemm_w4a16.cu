// GEMM with 4-bit weights that stay 4-bit in HBM: C[M, N] = A[M, K] * dequant(Wq)[N, K]^T.
//
// Serves the group-quantised integer formats (AWQ, GPTQ, compressed-tensors int4: a code 0..15,
// a scale and a zero point per group of K) and NVFP4 (an e2m1 code, an e4m3 scale per 16 elements
// and a per-channel fp32 factor). The reference runs these through its fp8_wmma package with the
// weights expanded in registers (mmq_fp8_gemm with w_zeros / NVFP4 global, mmq_regdirect_w4a16_*;
// python/minisgl/quant/kernels.py:1125-1180,1686-1731, python/minisgl/quant/nvfp4.py:81-179).
//
// Numerics: W4A16. Four "expander" warps turn every packed weight tile into 16-bit values in shared
// memory, w = (code - zero) * scale (or e2m1(code) * scale * channel factor), computed in fp32 and
// rounded once to the activation type; the tensor core then multiplies 16-bit activations with
// 16-bit weights (tcgen05.mma kind::f16) and accumulates in fp32 over K in ascending order. The
// result equals a GEMM on the fully expanded weight matrix bit for bit, but HBM holds and streams
// only the 4-bit codes and their group parameters. Block-scaled tensor-core kinds are not used
// because they take power-of-two (UE8M0) scales per 32 elements, which neither format has.
//
// Pipeline per CTA (persistent, one 128 x 128 output tile at a time, K blocks of 64):
//   warp 0       TMA producer: one or two A tiles (128 x 64, 128-byte swizzle) and the raw packed
//                weight tile (128 rows x 32 bytes) per stage
//   warp 1       MMA issuer, owner of tensor memory (two accumulator buffers)
//   warps 2-5    epilogue (tcgen05.ld, convert, store)
//   warps 6-13   expanders: two threads per weight row of the tile, group parameters fetched one
//                K block ahead
// With more than 128 rows, two activation tiles are multiplied from each expanded weight tile.
// All waits are bounded; a wait that runs out sets a status word and the CTA unwinds.
#include "common.cuh"
#include "ptx.cuh"

#include <mutex>
#include <string>
#include <unordered_map>

using namespace msgl;
using namespace msgl::ptx;

namespace {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int kThreads = 448;              // TMA, MMA, 4 epilogue warps, 8 expander warps
constexpr int kExpandWarp0 = 6, kExpandWarps = 8;
constexpr int A_BYTES = BM * BK * 2;       // 16 KB per 128-row activation tile
constexpr int B_BYTES = BN * BK * 2;       // 16 KB, written by the expanders
constexpr int RAW_BYTES = BN * BK / 2;     // 4 KB packed codes

// MT = activation tiles (of 128 rows) that share one expanded weight tile: with 129..256 rows both
// tiles of a column block are multiplied from one expansion.
template <int MT> struct Cfg {
  static constexpr int STAGES = MT == 1 ? 5 : 4;
  static constexpr int STAGE_A = MT * A_BYTES;
  static constexpr int off_a = 0;
  static constexpr int off_b = off_a + STAGES * STAGE_A;
  static constexpr int off_raw = off_b + STAGES * B_BYTES;
  static constexpr int off_bar = off_raw + STAGES * RAW_BYTES;
  static constexpr int n_bars = 3 * STAGES + 4;   // loaded / expanded / empty per stage, tfull / tempty per buffer
  static constexpr int smem_total = off_bar + n_bars * 8 + 16;
  static constexpr int NCOLS = 2 * MT * BN;       // two accumulator buffers of MT tiles
};

enum W4Format : int { W4_INT = 0, W4_NVFP4 = 1 };

struct W4Args {
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  int group;                 // K elements per scale: 16 or a multiple of 32
  int fmt;
  const void* scales;        // [K / group, N]: fp32 (int formats) or e4m3 bytes (NVFP4)
  const float* zeros;        // [K / group, N] fp32 (int formats)
  const float* channel;      // [N] fp32 per-channel factor (NVFP4) or nullptr
  const void* bias;          // [N] in the activation dtype or nullptr
  void* c;
  long long ldc;
  int out_dtype;             // MSGL_BF16 / MSGL_F16 / MSGL_F32
  int act_bf16;              // activation (and expanded weight) type: 1 bf16, 0 f16
  int* status;
};

__device__ int g_w4_status = 0;

// e2m1 code -> value {0, .5, 1, 1.5, 2, 3, 4, 6} with sign, built from the float's bit fields
__device__ __forceinline__ float e2m1_value(uint32_t nib) {
  const uint32_t e = (nib >> 1) & 3u, m = nib & 1u;
  const uint32_t normal = ((126u + e) << 23) | (m << 22);
  const uint32_t sub = m ? 0x3F000000u : 0u;
  return __uint_as_float((e ? normal : sub) | ((nib & 8u) << 28));
}

// integer code 0..15 as a float without an int->float conversion: 2^23 + code, minus 2^23 (exact)
__device__ __forceinline__ float code_value(uint32_t nib) { return __uint_as_float(0x4B000000u | nib) - 8388608.0f; }

__device__ __forceinline__ uint32_t pack2(bool bf16, float a, float b) {
  if (bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// MT: activation tiles per weight tile; INT: integer codes with zero points (else NVFP4); BF: bf16
// activations (else f16). Format and type are compile-time so that the expanders' inner loop holds
// one conversion only.
template <int MT, bool INT, bool BF>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_w,
                  const W4Args args) {
  using C = Cfg<MT>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ __align__(1024) uint8_t smem_raw_[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar_base = s_base + C::off_bar;
  auto loaded_bar = [&](int s) { return bar_base + 8u * s; };
  auto expanded_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto empty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (3 * STAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (3 * STAGES + 2 + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::off_bar + C::n_bars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::off_bar + C::n_bars * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_groups = (args.m_tiles + MT - 1) / MT;
  const int total_units = m_groups * args.n_tiles;    // unit = one weight tile x MT activation tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(loaded_bar(s), 1);
      mbar_init(expanded_bar(s), kExpandWarps);   // one arrival per expander warp
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_w);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::NCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_enter();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int unit = blockIdx.x; unit < total_units && !*abort_flag; unit += gridDim.x) {
        const int m_group = unit % m_groups, n_tile = unit / m_groups;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, args.status, 131)) break;
          mbar_expect_tx(loaded_bar(stage), MT * A_BYTES + RAW_BYTES);
          tma_load_2d(s_base + C::off_raw + stage * RAW_BYTES, &tma_w, loaded_bar(stage), kb * (BK / 2), n_tile * BN);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)   // rows past M read as zeros
            tma_load_2d(s_base + C::off_a + stage * C::STAGE_A + mt * A_BYTES, &tma_a, loaded_bar(stage), kb * BK,
                        (m_group * MT + mt) * BM);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      const uint32_t idesc = BF ? idesc_dense(1, 1, BM, BN) : idesc_dense(0, 0, BM, BN);
      for (int unit = blockIdx.x; unit < total_units && ok && !*abort_flag; unit += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, args.status, 132)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * (MT * BN);
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(expanded_bar(stage), phase, abort_flag, args.status, 133)) { ok = false; break; }
          tc_fence_after();
          const uint32_t b_s = s_base + C::off_b + stage * B_BYTES;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint32_t a_s = s_base + C::off_a + stage * C::STAGE_A + mt * A_BYTES;
#pragma unroll
            for (int k = 0; k < 4; ++k)   // four K = 16 steps of 32 bytes inside the 128-byte rows
              mma_f16(d_tmem + mt * BN, smem_desc_sw128(a_s + k * 32), smem_desc_sw128(b_s + k * 32), idesc,
                      (kb != 0 || k != 0) ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp < kExpandWarp0) {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
      const int m_group = unit % m_groups, n_tile = unit / m_groups;
      const int colbase = n_tile * BN;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, args.status, 134)) break;
      tc_fence_after();
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int row = (m_group * MT + mt) * BM + q * 32 + lane;
        const bool row_ok = row < args.M;
        const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * (MT * BN) + mt * BN);
#pragma unroll 1
        for (int cblk = 0; cblk < BN / 32; ++cblk) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + cblk * 32, r);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = colbase + cblk * 32 + g * 8;
              if (col < args.N) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  float x = __uint_as_float(r[g * 8 + e]);
                  if (args.bias != nullptr)
                    x += BF ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(args.bias)[col + e])
                            : __half2float(reinterpret_cast<const __half*>(args.bias)[col + e]);
                  o[e] = x;
                }
                if (args.out_dtype == MSGL_F32) {
                  float* cp = reinterpret_cast<float*>(args.c) + (size_t)row * args.ldc + col;
                  *reinterpret_cast<float4*>(cp) = make_float4(o[0], o[1], o[2], o[3]);
                  *reinterpret_cast<float4*>(cp + 4) = make_float4(o[4], o[5], o[6], o[7]);
                } else {
                  const bool bf = args.out_dtype == MSGL_BF16;
                  uint16_t* cp = reinterpret_cast<uint16_t*>(args.c) + (size_t)row * args.ldc + col;
                  *reinterpret_cast<uint4*>(cp) = make_uint4(pack2(bf, o[0], o[1]), pack2(bf, o[2], o[3]),
                                                             pack2(bf, o[4], o[5]), pack2(bf, o[6], o[7]));
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  } else {
    // ------------------------------------------------------------------ expanders (warps 6..13)
    // Two threads per weight row: thread (r, half) expands k = 32 half .. 32 half + 31 of each K block.
    // The group parameters of the NEXT K block are fetched before this one's codes are awaited, so
    // their global-memory latency hides behind the expansion of the current block.
    const int et = threadIdx.x - kExpandWarp0 * 32;
    const int r = et & 127, half = et >> 7;
    constexpr bool bf = BF;
    constexpr bool is_int = INT;
    const int per = args.group == 16 ? 2 : 1;            // scales per 32 consecutive k
    struct Params { float sc0, sc1, zp0, zp1, chan; };
    auto fetch = [&](int unit, int kb, Params& p) {
      const int n = (unit / m_groups) * BN + r;
      p.sc0 = p.sc1 = p.zp0 = p.zp1 = 0.f;
      p.chan = 1.f;
      if (n >= args.N) return;
      const int gi = (kb * BK + half * 32) / args.group;
      const size_t at = (size_t)gi * args.N + n;
      if (is_int) {
        p.sc0 = __ldg(reinterpret_cast<const float*>(args.scales) + at);
        p.zp0 = __ldg(args.zeros + at);
        if (per == 2) {
          p.sc1 = __ldg(reinterpret_cast<const float*>(args.scales) + at + args.N);
          p.zp1 = __ldg(args.zeros + at + args.N);
        }
      } else {
        p.sc0 = e4m3_to_float(__ldg(reinterpret_cast<const uint8_t*>(args.scales) + at));
        if (per == 2) p.sc1 = e4m3_to_float(__ldg(reinterpret_cast<const uint8_t*>(args.scales) + at + args.N));
        if (args.channel != nullptr) p.chan = __ldg(args.channel + n);
      }
    };
    int stage = 0;
    uint32_t phase = 0;
    int unit = blockIdx.x, kb = 0;
    Params cur, nxt;
    if (unit < total_units) fetch(unit, 0, cur);
    while (unit < total_units) {
      int n_unit = unit, n_kb = kb + 1;
      if (n_kb == args.k_blocks) { n_kb = 0; n_unit += gridDim.x; }
      if (n_unit < total_units) fetch(n_unit, n_kb, nxt);
      if (!mbar_wait(loaded_bar(stage), phase, abort_flag, args.status, 135)) break;
      const uint4 raw = *reinterpret_cast<const uint4*>(smem + C::off_raw + stage * RAW_BYTES + r * (BK / 2) + half * 16);
      const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};   // byte b holds k = 2b (low nibble) and 2b + 1
      uint8_t* brow = smem + C::off_b + stage * B_BYTES + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {             // chunk: 8 consecutive k
        const bool second = per == 2 && c >= 2;
        const float sc = second ? cur.sc1 : cur.sc0, zp = second ? cur.zp1 : cur.zp0;
        const uint32_t w = words[c];
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t nib = (w >> (4 * e)) & 0xFu;
          // e2m1 x e4m3 is exact in fp32; the channel factor is the one rounding, as in a load-time expansion
          v[e] = is_int ? (code_value(nib) - zp) * sc : (e2m1_value(nib) * sc) * cur.chan;
        }
        // 128-byte swizzle: 16-byte chunk ch of row r lives at chunk position ch ^ (r & 7)
        const int ch = half * 4 + c;
        *reinterpret_cast<uint4*>(brow + ((ch ^ (r & 7)) << 4)) =
            make_uint4(pack2(bf, v[0], v[1]), pack2(bf, v[2], v[3]), pack2(bf, v[4], v[5]), pack2(bf, v[6], v[7]));
      }
      fence_proxy_async();   // generic-proxy stores become visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(expanded_bar(stage));
      if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      cur = nxt;
      unit = n_unit;
      kb = n_kb;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::NCOLS);
  }
}

// Whole-matrix expansion for steps with many rows (prefill): the tile-by-tile expansion above would
// repeat for every M tile, so the weights are expanded once into a reusable 16-bit scratch matrix
// and the ordinary tcgen05 GEMM runs on that. One thread per 8 consecutive k of one row.
template <typename T>
__global__ void w4_expand_kernel(const uint8_t* __restrict__ wq, const void* __restrict__ scales,
                                 const float* __restrict__ zeros, const float* __restrict__ channel,
                                 T* __restrict__ out, int N, int K, int group, int fmt) {
  pdl_enter();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int chunks = K / 8;
  if (idx >= (size_t)N * chunks) return;
  // consecutive threads walk along N so that the scale reads ([K / group, N]) coalesce
  const int n = (int)(idx % N), ch = (int)(idx / N);
  const int k0 = ch * 8, gi = k0 / group;
  const uint32_t w = *reinterpret_cast<const uint32_t*>(wq + (size_t)n * (K / 2) + ch * 4);
  float sc, zp = 0.f, chan = 1.f;
  if (fmt == W4_INT) {
    sc = reinterpret_cast<const float*>(scales)[(size_t)gi * N + n];
    zp = zeros[(size_t)gi * N + n];
  } else {
    sc = e4m3_to_float(reinterpret_cast<const uint8_t*>(scales)[(size_t)gi * N + n]);
    chan = channel != nullptr ? channel[n] : 1.f;
  }
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t nib = (w >> (4 * e)) & 0xFu;
    v[e] = fmt == W4_INT ? ((float)nib - zp) * sc : (e2m1_value(nib) * sc) * chan;
  }
  store8(out + (size_t)n * K + k0, v);
}

struct MapKey {
  const void* ptr;
  uint64_t inner, rows, stride;
  int kind;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && inner == o.inner && rows == o.rows && stride == o.stride && kind == o.kind;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h ^= std::hash<uint64_t>()(k.inner * 1315423911ull + k.rows * 2654435761ull + k.stride) + (h << 6) + (h >> 2);
    return h ^ (size_t)k.kind;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_mutex;

int make_map(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, uint64_t inner, uint64_t rows,
             uint64_t row_bytes, uint32_t box_inner, uint32_t box_rows, bool swizzle, bool cache) {
  MapKey key{ptr, inner, rows, row_bytes, (int)dt * 2 + (swizzle ? 1 : 0)};
  if (cache) {
    std::lock_guard<std::mutex> g(g_maps_mutex);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return MSGL_OK; }
  }
  msgl_encode_tiled_fn enc = msgl_get_encode_tiled();
  if (enc == nullptr) return MSGL_CUDA_ERROR;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    msgl_set_error_text(("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r)).c_str());
    return MSGL_CUDA_ERROR;
  }
  if (cache) {
    std::lock_guard<std::mutex> g(g_maps_mutex);
    if (g_maps.size() > 8192) g_maps.clear();
    g_maps[key] = *out;
  }
  return MSGL_OK;
}

}  // namespace

// a [M, K] bf16 / f16 (row stride lda elements); wq [N, K / 2] bytes (low nibble = even k);
// fmt 0: scales fp32 [K / group, N], zeros fp32 [K / group, N]; fmt 1 (NVFP4): scales e4m3 bytes
// [K / 16, N], channel fp32 [N]. c [M, N] (ldc elements) of out_dtype.
MSGL_API int msgl_gemm_w4a16(const void* a, long long lda, const void* wq, const void* scales, const void* zeros,
                             const void* channel, const void* bias, void* c, long long ldc, int M, int N, int K,
                             int group, int fmt, int act_dtype, int out_dtype, cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || N % 8 || K % 64 || (group != 16 && (group < 32 || group % 32)) || K % group ||
      lda % 8) {
    msgl_set_error_text("gemm_w4a16: needs N % 8 == 0, K % 64 == 0, group 16 or a multiple of 32 that divides K");
    return MSGL_BAD_ARG;
  }
  if (fmt != W4_INT && fmt != W4_NVFP4) return MSGL_BAD_ARG;
  if (fmt == W4_INT && zeros == nullptr) return MSGL_BAD_ARG;
  if (act_dtype != MSGL_BF16 && act_dtype != MSGL_F16) return MSGL_BAD_ARG;
  if (M == 0) return MSGL_OK;
  W4Args args;
  args.M = M; args.N = N; args.K = K;
  args.m_tiles = (M + BM - 1) / BM;
  args.n_tiles = (N + BN - 1) / BN;
  args.k_blocks = K / BK;
  args.group = group;
  args.fmt = fmt;
  args.scales = scales;
  args.zeros = (const float*)zeros;
  args.channel = (const float*)channel;
  args.bias = bias;
  args.c = c;
  args.ldc = ldc;
  args.out_dtype = out_dtype;
  args.act_bf16 = act_dtype == MSGL_BF16 ? 1 : 0;
  int* status = nullptr;
  cudaGetSymbolAddress((void**)&status, g_w4_status);
  args.status = status;
  CUtensorMap ma, mw;
  int rc = make_map(&ma, a, act_dtype == MSGL_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                    (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, true, false);
  if (rc) return rc;
  rc = make_map(&mw, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, BK / 2, BN, false,
                true);
  if (rc) return rc;
  constexpr int smem1 = Cfg<1>::smem_total + 1024, smem2 = Cfg<2>::smem_total + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaSuccess;
#define MSGL_W4_ATTR(MT_, SMEM_)                                                                                    \
  for (int v = 0; v < 4 && e == cudaSuccess; ++v)                                                                  \
    e = cudaFuncSetAttribute(v == 0   ? gemm_w4a16_kernel<MT_, true, true>                                         \
                             : v == 1 ? gemm_w4a16_kernel<MT_, true, false>                                        \
                             : v == 2 ? gemm_w4a16_kernel<MT_, false, true>                                        \
                                      : gemm_w4a16_kernel<MT_, false, false>,                                      \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_);
    MSGL_W4_ATTR(1, smem1)
    MSGL_W4_ATTR(2, smem2)
#undef MSGL_W4_ATTR
    if (e != cudaSuccess) { msgl_set_error("w4a16 gemm smem attribute", e); return MSGL_CUDA_ERROR; }
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  // pairs of activation tiles share one weight expansion whenever there is more than one tile
  const bool pair = args.m_tiles > 1;
  int grid = ((args.m_tiles + (pair ? 1 : 0)) / (pair ? 2 : 1)) * args.n_tiles;
  if (grid > sms) grid = sms;
  void (*kernel)(const CUtensorMap, const CUtensorMap, const W4Args) = nullptr;
  const bool is_int = fmt == W4_INT, bf = act_dtype == MSGL_BF16;
#define MSGL_W4_PICK(MT_)                                                                                   \
  (is_int ? (bf ? gemm_w4a16_kernel<MT_, true, true> : gemm_w4a16_kernel<MT_, true, false>)                 \
          : (bf ? gemm_w4a16_kernel<MT_, false, true> : gemm_w4a16_kernel<MT_, false, false>))
  kernel = pair ? MSGL_W4_PICK(2) : MSGL_W4_PICK(1);
#undef MSGL_W4_PICK
  cudaError_t e = msgl_launch(kernel, dim3(grid), dim3(kThreads), pair ? smem2 : smem1, stream, ma, mw, args);
  if (e != cudaSuccess) { msgl_set_error("gemm_w4a16 launch", e); return MSGL_CUDA_ERROR; }
  return MSGL_OK;
}

// dense [N, K] 16-bit expansion of the packed weights (same arithmetic as the in-kernel expansion)
MSGL_API int msgl_w4_expand(const void* wq, const void* scales, const void* zeros, const void* channel, void* out,
                            int N, int K, int group, int fmt, int dtype, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || K % 8 || group % 8) return MSGL_BAD_ARG;
  const size_t total = (size_t)N * (K / 8);
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == MSGL_BF16)
    msgl_launch(w4_expand_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const uint8_t*)wq, scales,
                (const float*)zeros, (const float*)channel, (__nv_bfloat16*)out, N, K, group, fmt);
  else if (dtype == MSGL_F16)
    msgl_launch(w4_expand_kernel<__half>, dim3(blocks), dim3(256), 0, stream, (const uint8_t*)wq, scales,
                (const float*)zeros, (const float*)channel, (__half*)out, N, K, group, fmt);
  else
    return MSGL_BAD_ARG;
  MSGL_CHECK_LAUNCH("w4_expand");
  return MSGL_OK;
}

// 0 when no bounded wait of this GEMM has run out since the last reset; else 131 producer / 132
// accumulator / 133 expanded stage / 134 epilogue / 135 expander wait.
MSGL_API int msgl_gemm_w4a16_status(int reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_w4_status, sizeof(int));
  if (reset && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_w4_status, &z, sizeof(int));
  }
  return v;
}
