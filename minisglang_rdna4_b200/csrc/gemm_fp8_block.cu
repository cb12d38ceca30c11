// Block-scaled fp8 GEMM (W8A8 with 128 x 128 weight blocks and 1 x 128 activation groups), dense
// and grouped (mixture of experts):
//
//   C[m, n] = sum over K blocks kb of  a_s[m, kb] * w_s[n / 128, kb] * ( Aq[m, kb] . Bq[n, kb] )
//
// with Aq / Bq e4m3, a_s fp32 [M, K/128] and w_s fp32 [N/128, K/128] (grouped: [E, N/128, K/128]).
// This is the checkpoint format "block fp8" (DeepSeek / compressed-tensors `strategy: block`,
// `block_structure [128, 128]`) that the reference serves through its Fp8Block linear method and
// its w8a8 expert kernels (python/minisgl/quant/method.py:846-897,
// python/minisgl/quant/kernels.py:1181-1331).
//
// The scales change every 128 elements of K and are arbitrary fp32 numbers, so they cannot ride
// on the block-scaled MMA kinds (those take power-of-two UE8M0 scales). Instead every K block
// (= one pipeline stage, four tcgen05.mma kind::f8f6f4 of K = 32) is accumulated on its own
// into one of two 128-column tensor-memory buffers; the four promotion warps pull a finished
// block out with tcgen05.ld, multiply by the block's scale product and add it to a 128-float
// register accumulator per row while the tensor core already works on the next block in the
// other buffer. Every row's sum runs over K in ascending order and does not depend on M.
//
// Structure as in gemm_tcgen05.cu: persistent CTAs, warp 0 = TMA producer, warp 1 = MMA issuer
// and tensor-memory owner, warps 2-5 = promotion + store. All waits are bounded.
#include "common.cuh"
#include "ptx.cuh"

#include <mutex>
#include <string>
#include <unordered_map>

using namespace msgl;
using namespace msgl::ptx;

int msgl_b_static_level();   // gemm_tcgen05.cu: level set by msgl_gemm_static_weights

namespace {

constexpr int BM = 128, BN = 128, BK = 128;
constexpr int kThreads = 192;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK;
constexpr int off_a = 0;
constexpr int off_b = off_a + STAGES * A_BYTES;
constexpr int off_bar = off_b + STAGES * B_BYTES;
constexpr int n_bars = 2 * STAGES + 4;  // full / empty per stage, pfull / pempty per partial buffer
constexpr int smem_total = off_bar + n_bars * 8 + 16;
constexpr int NCOLS = 256;

struct BlockArgs {
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  const float* a_scale;   // [M, k_blocks]
  const float* w_scale;   // [experts, n_tiles, k_blocks]
  void* c;
  long long ldc;
  int out_dtype;
  const int32_t* tile_expert;  // grouped: expert of M tile m (negative: tile past the live rows)
  int l2_ahead;                // request a work item's weight stream into L2 one item ahead
  int* status;
};

__device__ int g_block_status = 0;

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const BlockArgs args) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar_base = s_base + off_bar;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto pfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto pempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + off_bar + n_bars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + off_bar + n_bars * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = args.m_tiles * args.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(pfull_bar(s), 1);
      mbar_init(pempty_bar(s), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), NCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_enter();  // nothing above touched global memory

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      // A weight tile that only one or two row tiles use (grouped experts, decode-sized dense calls) is
      // streamed once: its whole K range is requested into L2 one work item ahead, so the ring in
      // shared memory covers L2 latency instead of HBM latency.
      const bool l2_ahead = args.l2_ahead && (args.tile_expert != nullptr || args.m_tiles <= 2);
      auto prefetch_item = [&](int tile) {
        const int m_tile = tile % args.m_tiles, n_tile = tile / args.m_tiles;
        const int expert = args.tile_expert != nullptr ? args.tile_expert[m_tile] : 0;
        if (expert < 0) return;
        for (int kb = 0; kb < args.k_blocks; ++kb) tma_prefetch_2d(&tma_b, kb * BK, expert * args.N + n_tile * BN);
      };
      if (l2_ahead && (int)blockIdx.x < total_tiles) prefetch_item(blockIdx.x);
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        const int m_tile = tile % args.m_tiles, n_tile = tile / args.m_tiles;
        if (l2_ahead && tile + (int)gridDim.x < total_tiles) prefetch_item(tile + gridDim.x);
        int expert = 0;
        if (args.tile_expert != nullptr) {
          expert = args.tile_expert[m_tile];
          if (expert < 0) continue;
        }
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, args.status, 121)) break;
          mbar_expect_tx(full_bar(stage), A_BYTES + B_BYTES);
          tma_load_2d(s_base + off_a + stage * A_BYTES, &tma_a, full_bar(stage), kb * BK, m_tile * BM);
          tma_load_2d(s_base + off_b + stage * B_BYTES, &tma_b, full_bar(stage), kb * BK,
                      expert * args.N + n_tile * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (*abort_flag) {  // give copies that are still in flight time to land before the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0, pb = 0;
      uint32_t phase = 0, pphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok && !*abort_flag; tile += gridDim.x) {
        if (args.tile_expert != nullptr && args.tile_expert[tile % args.m_tiles] < 0) continue;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, args.status, 123)) { ok = false; break; }
          if (!mbar_wait(pempty_bar(pb), pphase ^ 1u, abort_flag, args.status, 122)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_s = s_base + off_a + stage * A_BYTES;
          const uint32_t b_s = s_base + off_b + stage * B_BYTES;
          const uint32_t d_tmem = tmem_base + pb * BN;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_f8f6f4(d_tmem, smem_desc_sw128(a_s + k * 32), smem_desc_sw128(b_s + k * 32),
                       idesc_dense(0, 0, BM, BN), k != 0 ? 1u : 0u);
          tc_commit(empty_bar(stage));  // the stage is free once these MMAs have read it
          tc_commit(pfull_bar(pb));     // and this K block's partial sums are complete
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          if (++pb == 2) { pb = 0; pphase ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ promotion + store (warps 2..5)
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    int pb = 0;
    uint32_t pphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int m_tile = tile % args.m_tiles, n_tile = tile / args.m_tiles;
      int expert = 0;
      if (args.tile_expert != nullptr) {
        expert = args.tile_expert[m_tile];
        if (expert < 0) continue;
      }
      const int row = m_tile * BM + q * 32 + lane;
      const bool row_ok = row < args.M;
      const float* as_row = args.a_scale + (size_t)(row_ok ? row : 0) * args.k_blocks;
      const float* ws_row = args.w_scale + ((size_t)expert * args.n_tiles + n_tile) * args.k_blocks;
      float acc[BN];
#pragma unroll
      for (int e = 0; e < BN; ++e) acc[e] = 0.f;
      float s_next = row_ok ? __ldg(as_row) * __ldg(ws_row) : 0.f;
      for (int kb = 0; kb < args.k_blocks; ++kb) {
        const float s = s_next;
        if (kb + 1 < args.k_blocks) s_next = row_ok ? __ldg(as_row + kb + 1) * __ldg(ws_row + kb + 1) : 0.f;
        if (!mbar_wait(pfull_bar(pb), pphase, abort_flag, args.status, 124)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(pb * BN);
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) acc[c * 32 + e] = fmaf(__uint_as_float(r[e]), s, acc[c * 32 + e]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pempty_bar(pb));
        if (++pb == 2) { pb = 0; pphase ^= 1u; }
      }
      if (!ok) break;
      if (row_ok) {
        const int colbase = n_tile * BN;
        if (args.out_dtype == MSGL_F32) {
          float* crow = reinterpret_cast<float*>(args.c) + (size_t)row * args.ldc + colbase;
#pragma unroll
          for (int g = 0; g < BN / 4; ++g)
            if (colbase + g * 4 < args.N)
              *reinterpret_cast<float4*>(crow + g * 4) =
                  make_float4(acc[g * 4], acc[g * 4 + 1], acc[g * 4 + 2], acc[g * 4 + 3]);
        } else {
          uint16_t* crow = reinterpret_cast<uint16_t*>(args.c) + (size_t)row * args.ldc + colbase;
          const bool bf = args.out_dtype == MSGL_BF16;
#pragma unroll
          for (int g = 0; g < BN / 8; ++g) {
            if (colbase + g * 8 < args.N) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (bf) {
                  __nv_bfloat162 v = __floats2bfloat162_rn(acc[g * 8 + 2 * e], acc[g * 8 + 2 * e + 1]);
                  w[e] = *reinterpret_cast<uint32_t*>(&v);
                } else {
                  __half2 v = __floats2half2_rn(acc[g * 8 + 2 * e], acc[g * 8 + 2 * e + 1]);
                  w[e] = *reinterpret_cast<uint32_t*>(&v);
                }
              }
              *reinterpret_cast<uint4*>(crow + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, NCOLS);
  }
}

// ------------------------------------------------------------------------------------------
// SiLU(gate) * up followed by per-group (128 outputs) e4m3 quantisation: the producer of the second
// expert GEMM's activations. One warp per (row, group).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_quant_group_kernel(const T* __restrict__ x, uint8_t* __restrict__ out_q,
                                            float* __restrict__ out_scale, int inter, int groups_per_row,
                                            size_t total_groups) {
  pdl_enter();
  const size_t gidx = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gidx >= total_groups) return;
  const int lane = threadIdx.x & 31;
  const size_t row = gidx / groups_per_row;
  const int g0 = (int)(gidx % groups_per_row) * 128;
  const int i = g0 + lane * 4;
  const T* gp = x + row * 2 * inter;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  float amax = 0.f;
  if (i < inter) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float g = to_float(gp[i + e]), u = to_float(gp[inter + i + e]);
      const float h = 0.5f * g;
      float t;
      asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
      v[e] = to_float(from_float<T>(fmaf(h, t, h) * u));
      amax = fmaxf(amax, fabsf(v[e]));
    }
  }
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-8f) / kFp8Max;
  if (lane == 0) out_scale[gidx] = scale;
  if (i < inter) {
    const float inv = 1.0f / scale;
    const uint32_t w = (uint32_t)float2_to_e4m3x2(v[0] * inv, v[1] * inv) |
                       ((uint32_t)float2_to_e4m3x2(v[2] * inv, v[3] * inv) << 16);
    *reinterpret_cast<uint32_t*>(out_q + row * inter + i) = w;
  }
}

struct MapKey {
  const void* ptr;
  uint64_t inner, rows;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && inner == o.inner && rows == o.rows && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    h ^= std::hash<uint64_t>()(k.inner * 1315423911ull + k.rows) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    return h ^ k.box_rows;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_mutex;

// K-major e4m3 matrix [rows, inner] with contiguous rows of `row_bytes`; box 128 x box_rows, 128B swizzle
int make_map(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
             bool cache) {
  MapKey key{ptr, inner, rows, box_rows};
  if (cache) {
    std::lock_guard<std::mutex> g(g_maps_mutex);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return MSGL_OK; }
  }
  msgl_encode_tiled_fn enc = msgl_get_encode_tiled();
  if (enc == nullptr) return MSGL_CUDA_ERROR;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
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

// a [M, K] e4m3 (row stride lda bytes), b [experts * N, K] e4m3, a_scale [M, ceil(K/128)] fp32,
// w_scale [experts, ceil(N/128), ceil(K/128)] fp32, c [M, N] (ldc elements) of out_dtype.
// tile_expert == nullptr: dense (experts = 1). Grouped: M % 128 == 0 and tile_expert[M / 128].
MSGL_API int msgl_gemm_fp8_block(const void* a, long long lda, const void* b, void* c, long long ldc, int M, int N,
                                 int K, const void* a_scale, const void* w_scale, const void* tile_expert,
                                 int num_experts, int out_dtype, cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || N % 8 || K % 16 || lda % 16 || a_scale == nullptr || w_scale == nullptr)
    return MSGL_BAD_ARG;
  if (out_dtype != MSGL_BF16 && out_dtype != MSGL_F16 && out_dtype != MSGL_F32) return MSGL_BAD_ARG;
  if (tile_expert != nullptr && (M % 128 || num_experts <= 0)) return MSGL_BAD_ARG;
  if (tile_expert != nullptr && N % 128) return MSGL_BAD_ARG;  // a tile must not straddle two experts' rows
  if (M == 0) return MSGL_OK;
  BlockArgs args;
  args.M = M; args.N = N; args.K = K;
  args.m_tiles = (M + BM - 1) / BM;
  args.n_tiles = (N + BN - 1) / BN;
  args.k_blocks = (K + BK - 1) / BK;
  args.a_scale = (const float*)a_scale;
  args.w_scale = (const float*)w_scale;
  args.c = c;
  args.ldc = ldc;
  args.out_dtype = out_dtype;
  args.tile_expert = (const int32_t*)tile_expert;
  args.l2_ahead = msgl_b_static_level() >= 2 ? 1 : 0;
  int* status = nullptr;
  cudaGetSymbolAddress((void**)&status, g_block_status);
  args.status = status;
  const uint64_t b_rows = (uint64_t)N * (uint64_t)(tile_expert != nullptr ? num_experts : 1);
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BM, false);
  if (rc) return rc;
  rc = make_map(&mb, b, (uint64_t)K, b_rows, (uint64_t)K, BN, true);
  if (rc) return rc;
  constexpr int smem = smem_total + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { msgl_set_error("fp8 block gemm smem attribute", e); return MSGL_CUDA_ERROR; }
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  int grid = args.m_tiles * args.n_tiles;
  if (grid > sms) grid = sms;
  cudaError_t e = msgl_launch(gemm_fp8_block_kernel, dim3(grid), dim3(kThreads), smem, stream, ma, mb, args);
  if (e != cudaSuccess) { msgl_set_error("gemm_fp8_block launch", e); return MSGL_CUDA_ERROR; }
  return MSGL_OK;
}

// 0 when no bounded wait of the block-fp8 GEMM has run out since the last reset; else 121 producer /
// 122 partial buffer / 123 stage / 124 promotion wait.
MSGL_API int msgl_gemm_fp8_block_status(int reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_block_status, sizeof(int));
  if (reset && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_block_status, &z, sizeof(int));
  }
  return v;
}

// x [rows, 2 * inter] (gate columns then up columns) -> e4m3 [rows, inter] + fp32 scales [rows, inter / 128]
MSGL_API int msgl_silu_mul_quant_group(const void* x, void* out_q, void* out_scale, int rows, int inter, int dtype,
                                       cudaStream_t stream) {
  if (inter % 128 || rows < 0) return MSGL_BAD_ARG;
  if (rows == 0) return MSGL_OK;
  const int gpr = inter / 128;
  const size_t total = (size_t)rows * gpr;
  const int warps = 8;
  const unsigned blocks = (unsigned)((total + warps - 1) / warps);
  cudaError_t e;
  if (dtype == MSGL_BF16)
    e = msgl_launch(silu_mul_quant_group_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), 0, stream,
                    (const __nv_bfloat16*)x, (uint8_t*)out_q, (float*)out_scale, inter, gpr, total);
  else if (dtype == MSGL_F16)
    e = msgl_launch(silu_mul_quant_group_kernel<__half>, dim3(blocks), dim3(warps * 32), 0, stream, (const __half*)x,
                    (uint8_t*)out_q, (float*)out_scale, inter, gpr, total);
  else
    return MSGL_BAD_ARG;
  if (e != cudaSuccess) { msgl_set_error("silu_mul_quant_group", e); return MSGL_CUDA_ERROR; }
  return MSGL_OK;
}
