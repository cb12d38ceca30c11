// Dense GEMM family on the 5th-generation tensor cores: C[M,N] = A[M,K] * B[N,K]^T with fp32
// accumulation in tensor memory.
//
//   kind 0/1  f16 / bf16 operands                       (tcgen05.mma.kind::f16)
//   kind 2    e4m3 x e4m3, per-token x per-channel scales in the epilogue (W8A8)
//             (tcgen05.mma.kind::f8f6f4)
//   kind 3    e4m3 activations x packed e2m1 weights with a UE8M0 scale per 32 K elements
//             (W4A8 MXFP4; tcgen05.mma.kind::mxf8f6f4.block_scale), per-token scale in the
//             epilogue. The weights stay 4-bit in HBM; TMA expands them to the padded
//             one-element-per-byte shared-memory form the instruction wants.
//
// Replaces the reference's fp8_wmma / dense_gemm packages (mmq_fp8_gemm, mmq_w8a8_gemm,
// dense_gemm*, dense_bf16_gemv; python/minisgl/quant/kernels.py:1686-1830,
// python/minisgl/layers/minv.py:223-398) and its cuBLAS calls.
//
// Structure: persistent CTAs (one per SM), 6 warps. Warp 0 drives TMA into a ring of
// 128-byte-swizzled stages; warp 1 issues the MMAs and owns tensor memory; warps 2-5 drain
// the accumulator (two accumulator buffers, so the epilogue of tile i overlaps the main loop
// of tile i+1). Full K per output tile, no split-K: a row's result does not depend on M, so a
// verify batch (M = K+1) reproduces the decode result (M = 1) bit for bit.
#include "common.cuh"
#include "ptx.cuh"

#include <mutex>
#include <string>
#include <unordered_map>

using namespace msgl;
using namespace msgl::ptx;

namespace {

constexpr int BM = 128;
constexpr int kThreads = 192;

enum GemmKind : int { KIND_F16 = 0, KIND_BF16 = 1, KIND_F8 = 2, KIND_MXF4 = 3 };

struct GemmArgs {
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  const float* a_scale;    // [M] or nullptr
  const float* b_scale;    // [N] or nullptr
  const void* bias;        // [N] in the compute dtype, or nullptr
  void* c;
  long long ldc;
  int out_dtype;           // MSGL_BF16 / MSGL_F16 / MSGL_F32
  int bias_dtype;
  const uint8_t* sfb;      // scale-factor atoms [n_atoms][k_atoms][512] (kind 3)
  int sf_k_atoms;
  // grouped (mixture-of-experts) mode: B is [experts * N, K]; M tile m multiplies with the
  // weights of expert tile_expert[m]; a negative id marks a tile past the live rows
  const int32_t* tile_expert;
  int sf_n_atoms;          // scale-factor atoms along N per expert
  int* status;
  int b_static;            // B and its scale atoms were written before the kernels now in flight
  // ---- tensor-parallel fusion (CTA-pair kernel only) -------------------------------------
  // Row-parallel GEMM -> reduce-scatter: instead of writing C locally, the epilogue stores each
  // partial row into the slot of the rank that owns that row (peer memory, plain st.global).
  // When the last warp of a 128-row block has stored, that rank's flag for (this rank, block)
  // is set to rs_seq.
  // 128-row block b of M belongs to rank b % world and is that rank's local block b / world.
  void* rs_slots[8];        // rs_slots[o]: owner o's region [src][local block][128][rs_ld] (16-bit)
  uint32_t* rs_flags[8];    // rs_flags[o]: owner o's flags [src][rs_flag_stride]
  uint32_t* rs_count;       // local self-resetting arrival counters, one per 128-row block of M
  long long rs_plane;       // elements between source planes of a slot region
  int rs_world, rs_rank, rs_flag_stride, rs_ld;
  uint32_t rs_seq, rs_arrivals;  // arrivals per block = 8 warps x N tiles
  // All-gather -> column-parallel GEMM: A rows arrive from their owners; a_ready[b] reaches
  // a_ready_seq once 128-row block b is complete in local memory.
  const uint32_t* a_ready;
  uint32_t a_ready_seq;
  unsigned long long comm_wait_ns;
  int tile_order;           // 0: M fastest; w > 1: N fastest with M tiles interleaved over w owners
  // ---- split-K (single-CTA kernel, small M): a work item is (tile, K range). Every item stores
  // its raw fp32 accumulators; the item that arrives last at the tile's counter adds the ranges
  // in ascending order and writes the result, so the sum does not depend on arrival order.
  int splits;               // 1: off
  int kb_per_split;
  float* splitk_ws;         // [splits][m_tiles * 128][n_tiles * BN] fp32
  uint32_t* splitk_count;   // [m_tiles * n_tiles], zero between calls
};

__device__ int g_gemm_status = 0;

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// tile index -> (m_tile, n_tile). order 0: M fastest (weights reused across a wave). order 1:
// N fastest, so that 128-row blocks complete (and are needed) one after the other; row blocks
// belong to the ranks round-robin, so consecutive M tiles also alternate between owners.
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int order, int& m_tile,
                                            int& n_tile) {
  if (order <= 0) {
    m_tile = tile % m_tiles;
    n_tile = tile / m_tiles;
  } else {
    m_tile = tile / n_tiles;
    n_tile = tile % n_tiles;
  }
}

// One epilogue warp's 32 rows x 128 columns of 128-row block `blk` have landed in the owner's
// slots. The warp that completes the block raises the owner's flag; the local counter resets
// itself for the next call.
__device__ __forceinline__ void rs_signal(const GemmArgs& args, int blk) {
  // the tensor stores of this warp are complete (bulk group waited for); order them, made by
  // the async proxy, before the generic-proxy release below
  asm volatile("fence.proxy.async.global;" ::: "memory");
  // release / acquire at GPU scope chains the warps of the block (a system-scope fence per warp
  // measured ~10 us each); the release store of the last one publishes system-wide
  uint32_t seen;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(seen) : "l"(args.rs_count + blk), "r"(1u) : "memory");
  if (seen + 1u == args.rs_arrivals) {
    args.rs_count[blk] = 0u;
    const int owner = blk % args.rs_world;
    st_release_sys_u32(args.rs_flags[owner] + (size_t)args.rs_rank * args.rs_flag_stride + blk / args.rs_world,
                       args.rs_seq);
  }
}

template <int KIND> struct KindTraits;
template <> struct KindTraits<KIND_F16> { static constexpr int BKE = 64; };
template <> struct KindTraits<KIND_BF16> { static constexpr int BKE = 64; };
template <> struct KindTraits<KIND_F8> { static constexpr int BKE = 128; };
template <> struct KindTraits<KIND_MXF4> { static constexpr int BKE = 128; };

template <int KIND, int BN> struct TmemCols {
  static constexpr int need = 2 * BN + (KIND == KIND_MXF4 ? 8 : 0);
  static constexpr int value = need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
};

template <int BN, int STAGES> struct SmemLayout {
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int SF_BYTES = 512;
  static constexpr int off_a = 0;
  static constexpr int off_b = off_a + STAGES * A_BYTES;
  static constexpr int off_sf = off_b + STAGES * B_BYTES;
  static constexpr int off_sfa = off_sf + STAGES * SF_BYTES;
  static constexpr int off_colv = off_sfa + 512;  // 4 epilogue warps x (BN scales + BN biases) fp32
  static constexpr int off_bar = off_colv + 4 * 2 * BN * 4;
  static constexpr int total = off_bar + (2 * STAGES + 4) * 8 + 16;
};

__device__ __forceinline__ uint32_t pack2_out(int out_dtype, float x0, float x1) {
  if (out_dtype == MSGL_BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(x0, x1);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(x0, x1);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int KIND, int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const GemmArgs args) {
  using L = SmemLayout<BN, STAGES>;
  using KT = KindTraits<KIND>;
  constexpr int NCOLS = TmemCols<KIND, BN>::value;
  // TMA counts the packed source bytes of a 4-bit tile (64 per row), not its padded
  // one-element-per-byte footprint in shared memory (128 per row)
  constexpr uint32_t STAGE_TX =
      KIND == KIND_MXF4 ? L::A_BYTES + L::B_BYTES / 2 + L::SF_BYTES : L::A_BYTES + L::B_BYTES;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // the dynamic segment is only guaranteed 16-byte aligned: round up to the swizzle period
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar_base = s_base + L::off_bar;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::off_bar + (2 * STAGES + 4) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::off_bar + (2 * STAGES + 4) * 8 + 4);
  volatile int* splitk_last = reinterpret_cast<volatile int*>(smem + L::off_bar + (2 * STAGES + 4) * 8 + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int splits = args.splits;
  const int total_tiles = args.m_tiles * args.n_tiles * splits;  // work items: (tile, K range)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
  }
  if (KIND == KIND_MXF4) {
    // activation block scales are all 2^0: the per-token fp32 scale is applied in the epilogue
    for (int i = threadIdx.x; i < 128; i += blockDim.x)
      reinterpret_cast<uint32_t*>(smem + L::off_sfa)[i] = 0x7F7F7F7Fu;
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), NCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Everything above touched no global memory. The weights (B, scale atoms) are not written by
  // any kernel of the stream either, so the producer puts the first stages' weight tiles in
  // flight before it waits for the kernels ahead of this one; the activations (A), their scales
  // and the expert table of the grouped mode are only read after the wait.
  if (!(warp == 0 && lane == 0)) pdl_enter();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int pre = 0;  // leading stages of the first work item whose weight tile is already in flight
      const bool l2_ahead = args.b_static >= 2 && args.tile_expert == nullptr && args.m_tiles <= 2;
      // grouped (expert) calls: every weight tile serves the rows of one expert only; same treatment,
      // one work item ahead, once the expert table may be read
      const bool l2_grouped = args.b_static >= 2 && args.tile_expert != nullptr;
      auto prefetch_weights = [&](int item, int skip) {
        const int tile = item / splits, split = item - tile * splits;
        const int n0 = (tile / args.m_tiles) * BN;
        int expert = 0;
        if (args.tile_expert != nullptr) {
          expert = args.tile_expert[tile % args.m_tiles];
          if (expert < 0) return;
        }
        const int kb0 = split * args.kb_per_split;
        const int kb1 = min(args.k_blocks, kb0 + args.kb_per_split);
        for (int kb = kb0 + skip; kb < kb1; ++kb) tma_prefetch_2d(&tma_b, kb * KT::BKE, expert * args.N + n0);
        if (KIND == KIND_MXF4 && kb1 > kb0 + skip)
          bulk_prefetch_l2(args.sfb + ((size_t)(expert * args.sf_n_atoms + n0 / 128) * args.sf_k_atoms + kb0 + skip) * 512,
                           (uint32_t)(kb1 - kb0 - skip) * 512u);
      };
      if (args.b_static && args.tile_expert == nullptr && (int)blockIdx.x < total_tiles) {
        const int tile = (int)blockIdx.x / splits, split = (int)blockIdx.x - tile * splits;
        const int n0 = (tile / args.m_tiles) * BN;
        const int kb0 = split * args.kb_per_split;
        const int kb1 = min(args.k_blocks, kb0 + args.kb_per_split);
        pre = min(STAGES, kb1 - kb0);
        for (int s = 0; s < pre; ++s) {
          const int kb = kb0 + s;
          mbar_expect_tx(full_bar(s), STAGE_TX);
          tma_load_2d(s_base + L::off_b + s * L::B_BYTES, &tma_b, full_bar(s), kb * KT::BKE, n0);
          if (KIND == KIND_MXF4) {
            const uint8_t* src = args.sfb + ((size_t)(n0 / 128) * args.sf_k_atoms + kb) * 512;
            bulk_load(s_base + L::off_sf + s * L::SF_BYTES, src, 512, full_bar(s));
          }
        }
        // decode-sized calls: the rest of this item's weight stream is requested into L2 now, so the
        // ring only has to cover L2 latency once the kernels ahead have finished
        if (l2_ahead) prefetch_weights(blockIdx.x, pre);
      }
      pdl_enter();
      if (l2_grouped && (int)blockIdx.x < total_tiles) prefetch_weights(blockIdx.x, 0);
      for (int item = blockIdx.x; item < total_tiles && !*abort_flag; item += gridDim.x) {
        const int tile = item / splits, split = item - tile * splits;
        const int m_tile = tile % args.m_tiles, n_tile = tile / args.m_tiles;
        const int n0 = n_tile * BN;
        if ((l2_ahead || l2_grouped) && item + (int)gridDim.x < total_tiles) prefetch_weights(item + gridDim.x, 0);
        int expert = 0;
        if (args.tile_expert != nullptr) {
          expert = args.tile_expert[m_tile];
          if (expert < 0) continue;
        }
        const int kb0 = split * args.kb_per_split;
        const int kb1 = min(args.k_blocks, kb0 + args.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          const bool have_b = pre > 0;
          if (have_b) {
            --pre;  // fresh stage: nothing to wait for, the weight tile and the byte count are posted
          } else {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, args.status, 101)) break;
            mbar_expect_tx(full_bar(stage), STAGE_TX);
          }
          tma_load_2d(s_base + L::off_a + stage * L::A_BYTES, &tma_a, full_bar(stage), kb * KT::BKE, m_tile * BM);
          if (!have_b) {
            tma_load_2d(s_base + L::off_b + stage * L::B_BYTES, &tma_b, full_bar(stage), kb * KT::BKE,
                        expert * args.N + n0);
            if (KIND == KIND_MXF4) {
              const uint8_t* src =
                  args.sfb + ((size_t)(expert * args.sf_n_atoms + n0 / 128) * args.sf_k_atoms + kb) * 512;
              bulk_load(s_base + L::off_sf + stage * L::SF_BYTES, src, 512, full_bar(stage));
            }
          }
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
      const uint32_t sfa_tmem = tmem_base + 2 * BN;
      const uint32_t sfb_tmem = tmem_base + 2 * BN + 4;
      if (KIND == KIND_MXF4) tmem_cp_32x128b_warpx4(sfa_tmem, smem_desc_sf(s_base + L::off_sfa));
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int item = blockIdx.x; item < total_tiles && !*abort_flag; item += gridDim.x) {
        const int tile = item / splits, split = item - tile * splits;
        const int n0 = (tile / args.m_tiles) * BN;
        if (args.tile_expert != nullptr && args.tile_expert[tile % args.m_tiles] < 0) continue;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, args.status, 102)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        const int kb0 = split * args.kb_per_split;
        const int kb1 = min(args.k_blocks, kb0 + args.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, args.status, 103)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_s = s_base + L::off_a + stage * L::A_BYTES;
          const uint32_t b_s = s_base + L::off_b + stage * L::B_BYTES;
          if (KIND == KIND_MXF4)
            tmem_cp_32x128b_warpx4(sfb_tmem, smem_desc_sf(s_base + L::off_sf + stage * L::SF_BYTES));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t a_desc = smem_desc_sw128(a_s + k * 32);
            const uint64_t b_desc = smem_desc_sw128(b_s + k * 32);
            const uint32_t accum = (kb != kb0 || k != 0) ? 1u : 0u;
            const uint32_t d_k = d_tmem;
            if (KIND == KIND_F16) {
              mma_f16(d_k, a_desc, b_desc, idesc_dense(0, 0, BM, BN), accum);
            } else if (KIND == KIND_BF16) {
              mma_f16(d_k, a_desc, b_desc, idesc_dense(1, 1, BM, BN), accum);
            } else if (KIND == KIND_F8) {
              mma_f8f6f4(d_k, a_desc, b_desc, idesc_dense(0, 0, BM, BN), accum);
            } else {
              mma_mxf8f6f4(d_k, a_desc, b_desc, idesc_block_scaled(0, 5, BM, BN, 0, (uint32_t)k), accum,
                           sfa_tmem, sfb_tmem + (uint32_t)((n0 & 127) >> 5));
            }
          }
          tc_commit(empty_bar(stage));  // the stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    // per-warp staging of the tile's column scales and bias: [0,BN) scale, [BN,2BN) bias
    float* colv = reinterpret_cast<float*>(smem + L::off_colv) + (warp - 2) * 2 * BN;
    const bool has_colv = args.b_scale != nullptr || args.bias != nullptr;
    for (int item = blockIdx.x; item < total_tiles; item += gridDim.x) {
      const int tile = item / splits, split = item - tile * splits;
      const int m_tile = tile % args.m_tiles, n_tile = tile / args.m_tiles;
      int expert = 0;
      if (args.tile_expert != nullptr) {
        expert = args.tile_expert[m_tile];
        if (expert < 0) continue;
      }
      const int row = m_tile * BM + q * 32 + lane;
      const bool row_ok = row < args.M;
      const int colbase = n_tile * BN;
      // everything that does not depend on the accumulator is fetched before waiting for it
      const float a_s = (args.a_scale != nullptr && row_ok) ? __ldg(args.a_scale + row) : 1.f;
      if (has_colv) {
        __syncwarp();
        for (int i = lane; i < BN; i += 32) {
          const int col = colbase + i;
          float sc = 1.f, bi = 0.f;
          if (col < args.N) {
            if (args.b_scale != nullptr) sc = __ldg(args.b_scale + (size_t)expert * args.N + col);  // [experts][N]
            if (args.bias != nullptr && (split == 0 || args.splitk_count != nullptr))
              bi = args.bias_dtype == MSGL_BF16
                       ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(args.bias)[col])
                       : (args.bias_dtype == MSGL_F16 ? __half2float(reinterpret_cast<const __half*>(args.bias)[col])
                                                      : reinterpret_cast<const float*>(args.bias)[col]);
          }
          colv[i] = sc;
          colv[BN + i] = bi;
        }
        __syncwarp();
      }
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, args.status, 104)) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
      if (splits > 1 && args.splitk_count != nullptr) {
        // raw partial sums of this K range -> workspace; the last range to arrive finishes the tile
        const int ws_ld = args.n_tiles * BN;
        const size_t ws_plane = (size_t)args.m_tiles * BM * ws_ld;
        float* wrow = args.splitk_ws + (size_t)split * ws_plane + (size_t)row * ws_ld + colbase;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 8; ++g)
            *reinterpret_cast<uint4*>(wrow + c * 32 + g * 4) = make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        // the four epilogue warps meet, one thread takes the tile's ticket
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          uint32_t seen;
          asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(seen) : "l"(args.splitk_count + tile), "r"(1u) : "memory");
          *splitk_last = seen + 1u == (uint32_t)splits ? 1 : 0;
          if (seen + 1u == (uint32_t)splits) args.splitk_count[tile] = 0u;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*splitk_last) {
          __threadfence();
          const float* srow = args.splitk_ws + (size_t)row * ws_ld + colbase;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            float accv[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) accv[e] = 0.f;
            for (int sp = 0; sp < splits; ++sp) {  // ascending K ranges: the order never changes
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(srow + (size_t)sp * ws_plane + c * 32 + g * 4));
                accv[g * 4] += v.x; accv[g * 4 + 1] += v.y; accv[g * 4 + 2] += v.z; accv[g * 4 + 3] += v.w;
              }
            }
            if (row_ok) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const int lc = c * 32 + g * 8;
                if (colbase + lc < args.N) {
                  float o[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    float x = accv[g * 8 + e] * a_s;
                    if (has_colv) x = fmaf(x, colv[lc + e], colv[BN + lc + e]);
                    o[e] = x;
                  }
                  if (args.out_dtype == MSGL_F32) {
                    float* cp = reinterpret_cast<float*>(args.c) + (size_t)row * args.ldc + colbase + lc;
                    *reinterpret_cast<float4*>(cp) = make_float4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<float4*>(cp + 4) = make_float4(o[4], o[5], o[6], o[7]);
                  } else {
                    uint16_t* cp = reinterpret_cast<uint16_t*>(args.c) + (size_t)row * args.ldc + colbase + lc;
                    *reinterpret_cast<uint4*>(cp) =
                        make_uint4(pack2_out(args.out_dtype, o[0], o[1]), pack2_out(args.out_dtype, o[2], o[3]),
                                   pack2_out(args.out_dtype, o[4], o[5]), pack2_out(args.out_dtype, o[6], o[7]));
                  }
                }
              }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // splitk_last is reused by the next item
      } else if (args.out_dtype != MSGL_F32) {
        // pack the whole row segment, hand the accumulator back, then store in one burst
        // (stores interleaved with the conversion measured 2x slower)
        uint32_t packed[BN / 2];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int lc = c * 32 + 2 * e;
            float x0 = __uint_as_float(r[2 * e]) * a_s, x1 = __uint_as_float(r[2 * e + 1]) * a_s;
            if (has_colv) {
              x0 = fmaf(x0, colv[lc], colv[BN + lc]);
              x1 = fmaf(x1, colv[lc + 1], colv[BN + lc + 1]);
            }
            packed[c * 16 + e] = pack2_out(args.out_dtype, x0, x1);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        if (row_ok) {
          uint16_t* crow = reinterpret_cast<uint16_t*>(args.c) + (size_t)row * args.ldc;
#pragma unroll
          for (int g = 0; g < BN / 8; ++g) {
            const int col = colbase + g * 8;
            if (col < args.N)
              *reinterpret_cast<uint4*>(crow + col) =
                  make_uint4(packed[g * 4], packed[g * 4 + 1], packed[g * 4 + 2], packed[g * 4 + 3]);
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float x = __uint_as_float(r[e]) * a_s;
            if (has_colv) x = fmaf(x, colv[c * 32 + e], colv[BN + c * 32 + e]);
            r[e] = __float_as_uint(x);
          }
          if (row_ok) {
            // planes mode (splits > 1 without counters): K range `split` writes plane `split` of an
            // fp32 [splits][M][ldc] output; the consumer sums the planes in ascending order
            float* crow = reinterpret_cast<float*>(args.c) + (size_t)split * args.M * args.ldc +
                          (size_t)row * args.ldc + colbase + c * 32;
#pragma unroll
            for (int g = 0; g < 8; ++g)
              if (colbase + c * 32 + g * 4 < args.N)
                *reinterpret_cast<uint4*>(crow + g * 4) = make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
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
// CTA-pair variant for large M: a cluster of two CTAs on neighbouring SMs computes one
// 256 x 256 output tile with cta_group::2 MMAs. Each CTA stages 128 rows of A and 128 rows of B
// per K block and gets 128 x 256 of output for them, so a byte brought into shared memory feeds
// twice the math of the 128 x 128 single-CTA tile; that tile is bound by shared-memory traffic
// (tensor pipe under 30 % busy on the prefill projections), this one is not.
//
// Barriers: full[s] lives in the even CTA and counts the bytes of both CTAs' copies; empty[s],
// tfull[a] exist in both CTAs and are signalled together by a multicast commit; tempty[a] lives
// in the even CTA and collects the epilogue warps of both. 10 warps: TMA, MMA, 8 epilogue
// (two per tensor-memory lane quarter, 128 columns each). The epilogue packs its columns into
// registers, frees the accumulator, then stores, so the block-scaled kind, whose scale factors
// leave room for one 256-column accumulator only, still overlaps its stores with the next tile.
// ------------------------------------------------------------------------------------------
constexpr int kPairThreads = 320;
constexpr int kPairBN = 256;

// RS: the epilogue pushes its rows to other ranks. Stores issued by the SM's load/store path
// top out near 2.4 GB/s per SM across NVLink (few outstanding requests, microseconds of
// latency), so the rows go through a per-warp shared-memory patch and leave as TMA tensor
// stores; their completion is awaited one tile late, behind the next tile's stores. Two
// pipeline stages make room for the patches.
template <int KIND, bool RS> struct PairCfg {
  static constexpr int NACC = KIND == KIND_MXF4 ? 1 : 2;
  static constexpr int STAGES = RS ? 4 : 6;
  static constexpr int PATCH_WARP = 2 * 32 * 128;            // two 64-column halves of 32 rows, 128-byte-swizzled
  static constexpr int PATCH_BYTES = RS ? 8 * PATCH_WARP : 0;
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = 128 * 128;
  static constexpr int SF_BYTES = 1024;  // two 128-row scale atoms: every CTA needs all 256 columns' scales
  static constexpr int off_a = 0;
  static constexpr int off_b = off_a + STAGES * A_BYTES;
  static constexpr int off_sf = off_b + STAGES * B_BYTES;
  static constexpr int off_sfa = off_sf + STAGES * SF_BYTES;
  static constexpr int off_colv = off_sfa + 512;       // 8 epilogue warps x (128 scales + 128 biases) fp32
  static constexpr int off_patch = (off_colv + 8 * 256 * 4 + 1023) / 1024 * 1024;  // swizzle period
  static constexpr int off_bar = off_patch + PATCH_BYTES;
  static constexpr int n_bars = 2 * STAGES + 2 * NACC;
  static constexpr int total = off_bar + n_bars * 8 + 16;
  static constexpr uint32_t STAGE_TX =
      KIND == KIND_MXF4 ? A_BYTES + B_BYTES / 2 + SF_BYTES : A_BYTES + B_BYTES;
};

struct PairOwnerMaps {
  CUtensorMap m[8];  // m[o]: this rank's plane in owner o's slot region (RS only)
};

template <int KIND, bool RS>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_sf, const __grid_constant__ PairOwnerMaps omaps,
                 const GemmArgs args) {
  using L = PairCfg<KIND, RS>;
  using KT = KindTraits<KIND>;
  constexpr int NACC = L::NACC;
  constexpr int STAGES = L::STAGES;
  constexpr int NCOLS = 512;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar_base = s_base + L::off_bar;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + NACC + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::off_bar + L::n_bars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::off_bar + L::n_bars * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int total_tiles = args.m_tiles * args.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < NACC; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 16);  // 8 epilogue warps in each of the two CTAs
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
    if (KIND == KIND_MXF4) prefetch_tensormap(&tma_sf);
  }
  if (KIND == KIND_MXF4) {
    for (int i = threadIdx.x; i < 128; i += blockDim.x)
      reinterpret_cast<uint32_t*>(smem + L::off_sfa)[i] = 0x7F7F7F7Fu;
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), NCOLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the other CTA's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_enter();  // the prologue above touched no global memory

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = pair; tile < total_tiles && !*abort_flag; tile += num_pairs) {
        int m_tile, n_tile;
        tile_coords(tile, args.m_tiles, args.n_tiles, args.tile_order, m_tile, n_tile);
        const int m0 = m_tile * 256 + (int)rank * 128;
        const int n0 = n_tile * kPairBN + (int)rank * 128;
        if (args.a_ready != nullptr && m0 < args.M) {
          // the 128 rows this CTA stages are written by their owner rank: wait (bounded) for them
          const uint32_t* flag = args.a_ready + (m0 >> 7);
          if ((int)(ld_acquire_sys_u32(flag) - args.a_ready_seq) < 0) {
            const uint64_t t0 = globaltimer_ns();
            while ((int)(ld_acquire_sys_u32(flag) - args.a_ready_seq) < 0) {
              if (*abort_flag) break;
              if (globaltimer_ns() - t0 > args.comm_wait_ns) {
                *abort_flag = 1;
                atomicCAS(args.status, 0, 115);
                break;
              }
            }
            if (*abort_flag) break;
          }
          // rows stored by a peer through the generic proxy are about to be read by TMA
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, args.status, 111)) break;
          const uint32_t lead_full = mapa_cluster(full_bar(stage), 0);
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * L::STAGE_TX);
          tma_load_2d_pair(s_base + L::off_a + stage * L::A_BYTES, &tma_a, lead_full, kb * KT::BKE, m0);
          tma_load_2d_pair(s_base + L::off_b + stage * L::B_BYTES, &tma_b, lead_full, kb * KT::BKE, n0);
          if (KIND == KIND_MXF4) {
            const int atom0 = (n_tile * 2) * args.sf_k_atoms + kb;
            tma_load_2d_pair(s_base + L::off_sf + stage * L::SF_BYTES, &tma_sf, lead_full, 0, atom0);
            tma_load_2d_pair(s_base + L::off_sf + stage * L::SF_BYTES + 512, &tma_sf, lead_full, 0,
                             atom0 + args.sf_k_atoms);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t sfa_tmem = tmem_base + NACC * kPairBN;
      const uint32_t sfb_tmem = sfa_tmem + 4;
      if (KIND == KIND_MXF4) tmem_cp_32x128b_warpx4_pair(sfa_tmem, smem_desc_sf(s_base + L::off_sfa));
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (int tile = pair; tile < total_tiles && !*abort_flag; tile += num_pairs) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, args.status, 112)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairBN;
        bool ok = true;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, args.status, 113)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_s = s_base + L::off_a + stage * L::A_BYTES;
          const uint32_t b_s = s_base + L::off_b + stage * L::B_BYTES;
          if (KIND == KIND_MXF4) {
            const uint32_t sf_s = s_base + L::off_sf + stage * L::SF_BYTES;
            tmem_cp_32x128b_warpx4_pair(sfb_tmem, smem_desc_sf(sf_s));
            tmem_cp_32x128b_warpx4_pair(sfb_tmem + 4, smem_desc_sf(sf_s + 512));
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t a_desc = smem_desc_sw128(a_s + k * 32);
            const uint64_t b_desc = smem_desc_sw128(b_s + k * 32);
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            if (KIND == KIND_F16) {
              mma_f16_pair(d_tmem, a_desc, b_desc, idesc_dense(0, 0, 256, kPairBN), accum);
            } else if (KIND == KIND_BF16) {
              mma_f16_pair(d_tmem, a_desc, b_desc, idesc_dense(1, 1, 256, kPairBN), accum);
            } else if (KIND == KIND_F8) {
              mma_f8f6f4_pair(d_tmem, a_desc, b_desc, idesc_dense(0, 0, 256, kPairBN), accum);
            } else {
              mma_mxf8f6f4_pair(d_tmem, a_desc, b_desc, idesc_block_scaled(0, 5, 256, kPairBN, 0, (uint32_t)k),
                                accum, sfa_tmem, sfb_tmem);
            }
          }
          tc_commit_pair(empty_bar(stage), 3);  // frees this stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit_pair(tfull_bar(acc), 3);
        if (++acc == NACC) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int q = warp & 3;          // tensor-memory lane quarter this warp may read
    const int h = (warp - 2) >> 2;   // which 128 of the tile's 256 columns
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t lead_tempty0 = mapa_cluster(tempty_bar(0), 0);
    // per-warp staging of the tile's column scales and bias: [0,128) scale, [128,256) bias
    float* colv = reinterpret_cast<float*>(smem + L::off_colv) + (warp - 2) * 256;
    const bool has_colv = args.b_scale != nullptr || args.bias != nullptr;
    int pending_blk = -1;  // RS: block of the previous tile, whose stores are still in flight
    for (int tile = pair; tile < total_tiles; tile += num_pairs) {
      int m_tile, n_tile;
      tile_coords(tile, args.m_tiles, args.n_tiles, args.tile_order, m_tile, n_tile);
      const int row = m_tile * 256 + (int)rank * 128 + q * 32 + lane;
      const bool row_ok = row < args.M;
      const int colbase = n_tile * kPairBN + h * 128;
      // everything that does not depend on the accumulator is fetched before waiting for it
      // (rows that are still arriving from a peer have their scale read after the wait instead)
      float a_s = (args.a_scale != nullptr && row_ok && args.a_ready == nullptr) ? __ldg(args.a_scale + row) : 1.f;
      if (has_colv) {
        __syncwarp();  // the previous tile's readers are done with the staging rows
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = colbase + i * 32 + lane;
          float sc = 1.f, bi = 0.f;
          if (col < args.N) {
            if (args.b_scale != nullptr) sc = __ldg(args.b_scale + col);
            if (args.bias != nullptr)
              bi = args.bias_dtype == MSGL_BF16
                       ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(args.bias)[col])
                       : (args.bias_dtype == MSGL_F16 ? __half2float(reinterpret_cast<const __half*>(args.bias)[col])
                                                      : reinterpret_cast<const float*>(args.bias)[col]);
          }
          colv[i * 32 + lane] = sc;
          colv[128 + i * 32 + lane] = bi;
        }
        __syncwarp();
      }
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, args.status, 114)) break;
      tc_fence_after();
      if (args.a_ready != nullptr && args.a_scale != nullptr && row_ok)
        a_s = *reinterpret_cast<const volatile float*>(args.a_scale + row);
      const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * kPairBN + h * 128);
      // Drain two 32-column loads at a time, fold the scales in and pack to the output type, hand
      // the accumulator back, and only then store: 16 back-to-back 16-byte stores per thread
      // (256 contiguous bytes of one row). Stores interleaved with the conversion measured 2x slower.
      if (args.out_dtype != MSGL_F32) {
        uint32_t packed[64];
        uint32_t r0[32], r1[32];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          tmem_ld_32x32b_x32(t_addr + hh * 64, r0);
          tmem_ld_32x32b_x32(t_addr + hh * 64 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int c0 = hh * 64 + 2 * e, c1 = c0 + 32;
            float x0 = __uint_as_float(r0[2 * e]) * a_s, x1 = __uint_as_float(r0[2 * e + 1]) * a_s;
            float y0 = __uint_as_float(r1[2 * e]) * a_s, y1 = __uint_as_float(r1[2 * e + 1]) * a_s;
            if (has_colv) {
              x0 = fmaf(x0, colv[c0], colv[128 + c0]);
              x1 = fmaf(x1, colv[c0 + 1], colv[128 + c0 + 1]);
              y0 = fmaf(y0, colv[c1], colv[128 + c1]);
              y1 = fmaf(y1, colv[c1 + 1], colv[128 + c1 + 1]);
            }
            packed[hh * 32 + e] = pack2_out(args.out_dtype, x0, x1);
            packed[hh * 32 + 16 + e] = pack2_out(args.out_dtype, y0, y1);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8u * acc);
        if (RS) {
          uint8_t* patch = smem + L::off_patch + (warp - 2) * L::PATCH_WARP;
          const uint32_t patch_s = s_base + L::off_patch + (warp - 2) * L::PATCH_WARP;
          const int blk0 = (m_tile * 256 + (int)rank * 128) >> 7;
          const int owner = blk0 % args.rs_world;
          // the previous tile's stores must have finished reading the patch
          if (lane == 0) bulk_wait_group_read<0>();
          __syncwarp();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int u = 0; u < 8; ++u)  // 128-byte swizzle: 16-byte unit u of row r lives at unit u ^ (r & 7)
              *reinterpret_cast<uint4*>(patch + half * 4096 + lane * 128 + ((u ^ (lane & 7)) << 4)) =
                  make_uint4(packed[half * 32 + u * 4], packed[half * 32 + u * 4 + 1], packed[half * 32 + u * 4 + 2],
                             packed[half * 32 + u * 4 + 3]);
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            const int drow = (blk0 / args.rs_world) * 128 + q * 32;
            if ((blk0 << 7) < args.M) {
              tma_store_2d(&omaps.m[owner], patch_s, colbase, drow);
              tma_store_2d(&omaps.m[owner], patch_s + 4096, colbase + 64, drow);
            }
            bulk_commit_group();
            // The tile before this one has had a whole tile time to land: wait for it now (this
            // tile's group stays in flight), then count its warp as delivered. The warp that
            // completes a 128-row block tells the owner; the counter resets itself.
            if (pending_blk >= 0) {
              bulk_wait_group<1>();
              rs_signal(args, pending_blk);
            }
            pending_blk = (blk0 << 7) < args.M ? blk0 : -1;
          }
        } else if (row_ok) {
          uint16_t* crow = reinterpret_cast<uint16_t*>(args.c) + (size_t)row * args.ldc;
#pragma unroll
          for (int g = 0; g < 16; ++g) {
            const int col = colbase + g * 8;
            if (col < args.N)
              *reinterpret_cast<uint4*>(crow + col) =
                  make_uint4(packed[g * 4], packed[g * 4 + 1], packed[g * 4 + 2], packed[g * 4 + 3]);
          }
        }
      } else {
        // fp32 output (logits): all 128 columns stay in registers until the burst of stores
        uint32_t r0[32], r1[32], r2[32], r3[32];
        tmem_ld_32x32b_x32(t_addr, r0);
        tmem_ld_32x32b_x32(t_addr + 32, r1);
        tmem_ld_32x32b_x32(t_addr + 64, r2);
        tmem_ld_32x32b_x32(t_addr + 96, r3);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8u * acc);
        auto scale_in_place = [&](uint32_t (&r)[32], int c) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float x = __uint_as_float(r[e]) * a_s;
            if (has_colv) x = fmaf(x, colv[c * 32 + e], colv[128 + c * 32 + e]);
            r[e] = __float_as_uint(x);
          }
        };
        scale_in_place(r0, 0);
        scale_in_place(r1, 1);
        scale_in_place(r2, 2);
        scale_in_place(r3, 3);
        if (row_ok) {
          float* crow = reinterpret_cast<float*>(args.c) + (size_t)row * args.ldc + colbase;
          auto burst = [&](const uint32_t (&r)[32], int c) {
#pragma unroll
            for (int g = 0; g < 8; ++g)
              if (colbase + c * 32 + g * 4 < args.N)
                *reinterpret_cast<uint4*>(crow + c * 32 + g * 4) =
                    make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
          };
          burst(r0, 0);
          burst(r1, 1);
          burst(r2, 2);
          burst(r3, 3);
        }
      }
      if (++acc == NACC) { acc = 0; acc_phase ^= 1u; }
    }
    if (RS && lane == 0) {
      bulk_wait_group<0>();
      if (pending_blk >= 0) rs_signal(args, pending_blk);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory or exits while the other may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, NCOLS);
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
struct MapKey {
  const void* ptr;
  uint64_t d0, d1, stride;
  uint32_t b0, b1;
  int dtype;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && stride == o.stride && b0 == o.b0 && b1 == o.b1 &&
           dtype == o.dtype;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    auto mix = [&](uint64_t v) { h ^= std::hash<uint64_t>()(v) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.d0); mix(k.d1); mix(k.stride); mix(k.b0); mix(k.b1); mix((uint64_t)k.dtype);
    return h;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;
std::mutex g_map_mutex;

// 2-D K-major tensor map: dims {inner (elements), rows}, box {box_inner, box_rows}, 128B swizzle
int make_map_2d(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, uint64_t inner, uint64_t rows,
                uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows, bool cache,
                bool swizzle = true) {
  MapKey key{ptr, inner, rows, row_stride_bytes, box_inner, box_rows, (int)dt + (swizzle ? 0 : 1000)};
  if (cache) {
    std::lock_guard<std::mutex> g(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) { *out = it->second; return MSGL_OK; }
  }
  msgl_encode_tiled_fn enc = msgl_get_encode_tiled();
  if (enc == nullptr) return MSGL_CUDA_ERROR;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    msgl_set_error_text(("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r)).c_str());
    return MSGL_CUDA_ERROR;
  }
  if (cache) {
    std::lock_guard<std::mutex> g(g_map_mutex);
    if (g_map_cache.size() > 16384) g_map_cache.clear();
    g_map_cache[key] = *out;
  }
  return MSGL_OK;
}

int g_b_static = 0;
int g_num_sms = 0;
int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int KIND, int BN, int STAGES>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, GemmArgs& args, int max_ctas, cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  constexpr int smem = L::total + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<KIND, BN, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { msgl_set_error("gemm smem attribute", e); return MSGL_CUDA_ERROR; }
    configured = true;
  }
  int total = args.m_tiles * args.n_tiles * args.splits;
  int grid = total < max_ctas ? total : max_ctas;
  msgl_launch(gemm_tcgen05_kernel<KIND, BN, STAGES>, dim3(grid), dim3(kThreads), smem, stream, ma, mb, args);
  MSGL_CHECK_LAUNCH("gemm_tcgen05");
  return MSGL_OK;
}

template <int KIND>
int dispatch_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, GemmArgs& args, int max_ctas,
                cudaStream_t stream) {
  switch (bn) {
    case 128: return launch<KIND, 128, 6>(ma, mb, args, max_ctas, stream);
    case 64: return launch<KIND, 64, 8>(ma, mb, args, max_ctas, stream);
    case 32: return launch<KIND, 32, 8>(ma, mb, args, max_ctas, stream);
    default: return MSGL_BAD_ARG;
  }
}

// Launch the CTA-pair kernel: clusters of two, one cluster per pair of SMs, persistent over tiles.
template <int KIND, bool RS>
int launch_pair_impl(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& msf, const PairOwnerMaps& omaps,
                     GemmArgs& args, int max_ctas, cudaStream_t stream) {
  using L = PairCfg<KIND, RS>;
  constexpr int smem = L::total + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(gemm_pair_kernel<KIND, RS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { msgl_set_error("pair gemm smem attribute", e); return MSGL_CUDA_ERROR; }
    configured = true;
  }
  const int total = args.m_tiles * args.n_tiles;
  int pairs = max_ctas / 2;
  if (pairs > total) pairs = total;
  if (pairs < 1) pairs = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2] = {};
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = msgl_pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<KIND, RS>, ma, mb, msf, omaps, args);
  if (e != cudaSuccess) { msgl_set_error("gemm_pair launch", e); return MSGL_CUDA_ERROR; }
  return MSGL_OK;
}

int make_map_2d(CUtensorMap* out, const void* ptr, CUtensorMapDataType dt, uint64_t inner, uint64_t rows,
                uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows, bool cache, bool swizzle);

template <int KIND>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& msf, GemmArgs& args, int max_ctas,
                cudaStream_t stream) {
  static PairOwnerMaps omaps;  // contents only matter to the RS instantiation
  if (args.rs_world > 0) {
    // store maps: this rank's plane in every owner's slot region, 64-column x 32-row boxes
    for (int o = 0; o < args.rs_world; ++o) {
      const uint16_t* base = reinterpret_cast<const uint16_t*>(args.rs_slots[o]) + (size_t)args.rs_rank * args.rs_plane;
      const uint64_t rows = (uint64_t)(args.rs_plane / args.rs_ld);
      int rc = make_map_2d(&omaps.m[o], base, CU_TENSOR_MAP_DATA_TYPE_UINT16, (uint64_t)args.rs_ld, rows,
                           (uint64_t)args.rs_ld * 2, 64, 32, true, true);
      if (rc) return rc;
    }
    return launch_pair_impl<KIND, true>(ma, mb, msf, omaps, args, max_ctas, stream);
  }
  return launch_pair_impl<KIND, false>(ma, mb, msf, omaps, args, max_ctas, stream);
}

int g_pair_mode = 0;  // 0 = by size, 1 = never, 2 = whenever the arguments allow

}  // namespace

msgl_encode_tiled_fn msgl_get_encode_tiled() {
  static msgl_encode_tiled_fn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<msgl_encode_tiled_fn>(p);
    else msgl_set_error_text("cuTensorMapEncodeTiled is not available from the driver");
  }
  return fn;
}

// Pick the N tile so that the grid fills the GPU when the problem allows it.
// Pick the N tile that minimises (waves over the SMs) x (bytes a CTA stages per K block): a tile
// twice as wide costs 1.2-1.5x the bytes per K block but halves the tile count, so it wins
// whenever the narrower tile would need an extra wave.
static int choose_bn(int m_tiles, int n, int sms, int smallest, int b_row_bytes) {
  const int cands[3] = {128, 64, 32};
  int best = smallest;
  long long best_cost = -1;
  for (int i = 0; i < 3; ++i) {
    const int bn = cands[i];
    if (bn < smallest) continue;
    const long long tiles = (long long)m_tiles * ((n + bn - 1) / bn);
    const long long waves = (tiles + sms - 1) / sms;
    const long long cost = waves * (128 * 128 + (long long)bn * b_row_bytes);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
  }
  return best;
}

// Tensor-parallel fusion arguments of msgl_gemm_tp (mirrored by a ctypes.Structure).
struct MsglGemmTp {
  void* rs_slots[8];       // per owner rank: slot region base for this call's parity (peer-mapped)
  void* rs_flags[8];       // per owner rank: flag region base
  void* rs_count;          // local arrival counters [M / 128], zero between calls
  long long rs_plane;      // elements between source planes
  int rs_world;            // 0: write C locally; > 0: push row blocks to their owners (block b -> rank b % world)
  int rs_rank, rs_flag_stride, rs_ld;
  unsigned int rs_seq;
  unsigned int a_ready_seq;
  const void* a_ready;     // nullptr: A is local and complete
  long long wait_us;       // bound of the device-side flag waits
  int order_world;         // > 1: N-fastest tile walk (row blocks complete / are needed in order)
};

// a: [M, K] (kind 0/1: 16-bit, kind 2/3: e4m3 bytes), row stride lda elements
// b: [N, K] (kind 0/1: 16-bit, kind 2: e4m3 bytes, kind 3: packed e2m1 [N, ceil(K/128)*64], zero codes
//    past K)
// c: [M, N] out_dtype, row stride ldc elements
// bn_override: 0 = automatic, else 32 / 64 / 128; max_ctas: 0 = one per SM
static int gemm_impl(int kind, const void* a, long long lda, const void* b, void* c, long long ldc, int M, int N,
                     int K, const void* a_scale, const void* b_scale, const void* bias, int bias_dtype,
                     const void* sf_atoms, int out_dtype, int bn_override, int max_ctas, const void* tile_expert,
                     int num_experts, cudaStream_t stream, const MsglGemmTp* tp = nullptr, int splits = 1,
                     void* splitk_ws = nullptr, void* splitk_count = nullptr) {
  if (M <= 0 || N <= 0 || K <= 0) return M == 0 ? MSGL_OK : MSGL_BAD_ARG;
  if (tp != nullptr) {
    if (tile_expert != nullptr || M % 128 || (tp->rs_world > 0 && out_dtype == MSGL_F32)) {
      msgl_set_error_text("gemm_tp: needs M a multiple of 128, 16-bit output and ungrouped operands");
      return MSGL_BAD_ARG;
    }
    bn_override = 256;
  }
  if (N % 8) { msgl_set_error_text("gemm: N must be a multiple of 8"); return MSGL_BAD_ARG; }
  const int esize_a = (kind == KIND_F16 || kind == KIND_BF16) ? 2 : 1;
  if ((lda * esize_a) % 16 || (uintptr_t)a % 16 || (uintptr_t)b % 16 || (uintptr_t)c % 16) {
    msgl_set_error_text("gemm: operands must be 16-byte aligned with 16-byte row strides");
    return MSGL_BAD_ARG;
  }
  if (kind == KIND_MXF4 && (K % 32 || sf_atoms == nullptr || (uintptr_t)b % 32)) {
    msgl_set_error_text("gemm: MXFP4 needs K % 32 == 0, 32-byte aligned weights and scale atoms");
    return MSGL_BAD_ARG;
  }
  if ((kind == KIND_F16 || kind == KIND_BF16) ? (K % 8) : (K % 16)) {
    msgl_set_error_text("gemm: K row bytes must be a multiple of 16");
    return MSGL_BAD_ARG;
  }
  const int sms = num_sms();
  if (max_ctas <= 0 || max_ctas > sms) max_ctas = sms;
  const int bke = (kind == KIND_F16 || kind == KIND_BF16) ? 64 : 128;
  GemmArgs args;
  args.M = M; args.N = N; args.K = K;
  args.m_tiles = (M + BM - 1) / BM;
  // The block-scaled instruction takes its weight scale factors from tensor-memory columns in
  // steps of 64 rows (two columns), so the MXFP4 kind has no 32-wide N tile.
  // Above 256 rows the CTA-pair kernel (256 x 256 tiles) takes over; below, a pair tile would be
  // mostly padding and too few tiles would exist to fill the GPU.
  const bool pair_ok = tile_expert == nullptr && (uintptr_t)sf_atoms % 16 == 0;
  const bool use_pair =
      pair_ok && (bn_override == 256 || (bn_override == 0 && g_pair_mode != 1 && (M > 256 || g_pair_mode == 2)));
  if (bn_override == 256 && !pair_ok) {
    msgl_set_error_text("gemm: the 256-wide CTA-pair tile does not support grouped operands");
    return MSGL_BAD_ARG;
  }
  const int bn = use_pair ? 256
                 : bn_override ? bn_override
                               : choose_bn(args.m_tiles, N, sms, kind == KIND_MXF4 ? 64 : 32, kind == KIND_MXF4 ? 64 : 128);
  if (use_pair) args.m_tiles = (M + 255) / 256;
  const int b_box = use_pair ? 128 : bn;
  if (kind == KIND_MXF4 && bn == 32) {
    msgl_set_error_text("gemm: the MXFP4 kind supports N tiles of 64 and 128 only");
    return MSGL_BAD_ARG;
  }
  args.n_tiles = (N + bn - 1) / bn;
  args.k_blocks = (K + bke - 1) / bke;
  args.a_scale = (const float*)a_scale;
  args.b_scale = (const float*)b_scale;
  args.bias = bias;
  args.bias_dtype = bias_dtype;
  args.c = c;
  args.ldc = ldc;
  args.out_dtype = out_dtype;
  args.sfb = (const uint8_t*)sf_atoms;
  args.sf_k_atoms = (K + 127) / 128;
  args.sf_n_atoms = (N + 127) / 128;
  args.tile_expert = (const int32_t*)tile_expert;
  args.splits = 1;
  args.kb_per_split = args.k_blocks;
  args.splitk_ws = nullptr;
  args.splitk_count = nullptr;
  const bool planes = splits > 1 && splitk_ws == nullptr && splitk_count == nullptr && out_dtype == MSGL_F32;
  if (splits > 1 && !use_pair && tile_expert == nullptr && ((splitk_ws != nullptr && splitk_count != nullptr) || planes)) {
    args.splits = splits;
    args.kb_per_split = (args.k_blocks + splits - 1) / splits;
    args.splitk_ws = (float*)splitk_ws;
    args.splitk_count = (uint32_t*)splitk_count;
  } else if (planes) {
    msgl_set_error_text("gemm_splitk_planes: needs the single-CTA kernel (M <= 256) and ungrouped operands");
    return MSGL_BAD_ARG;
  }
  args.rs_world = 0;
  args.a_ready = nullptr;
  args.tile_order = 0;
  args.comm_wait_ns = 0;
  if (tp != nullptr) {
    for (int i = 0; i < 8; ++i) {
      args.rs_slots[i] = tp->rs_slots[i];
      args.rs_flags[i] = (uint32_t*)tp->rs_flags[i];
    }
    args.rs_count = (uint32_t*)tp->rs_count;
    args.rs_plane = tp->rs_plane;
    args.rs_world = tp->rs_world;
    args.rs_rank = tp->rs_rank;
    args.rs_flag_stride = tp->rs_flag_stride;
    args.rs_ld = tp->rs_ld;
    args.rs_seq = tp->rs_seq;
    args.rs_arrivals = 8u * (uint32_t)((N + 255) / 256);
    args.a_ready = (const uint32_t*)tp->a_ready;
    args.a_ready_seq = tp->a_ready_seq;
    args.comm_wait_ns = (unsigned long long)(tp->wait_us > 0 ? tp->wait_us : 500000) * 1000ull;
    args.tile_order = tp->order_world > 1 ? 1 : 0;
  }
  const uint64_t b_rows = (uint64_t)N * (uint64_t)(num_experts > 0 ? num_experts : 1);
  int* status = nullptr;
  cudaGetSymbolAddress((void**)&status, g_gemm_status);
  args.status = status;
  args.b_static = g_b_static;

  CUtensorMap ma, mb;
  int rc;
  if (kind == KIND_F16 || kind == KIND_BF16) {
    CUtensorMapDataType dt = kind == KIND_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    rc = make_map_2d(&ma, a, dt, K, M, (uint64_t)lda * 2, 64, BM, false);
    if (rc) return rc;
    rc = make_map_2d(&mb, b, dt, K, b_rows, (uint64_t)K * 2, 64, b_box, true);
  } else if (kind == KIND_F8) {
    rc = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, K, M, (uint64_t)lda, 128, BM, false);
    if (rc) return rc;
    rc = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, K, b_rows, (uint64_t)K, 128, b_box, true);
  } else if (kind == KIND_MXF4) {
    rc = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, K, M, (uint64_t)lda, 128, BM, false);
    if (rc) return rc;
    // 4-bit rows are stored in whole 128-element K blocks (zero codes past K); A's last block is
    // zero-filled by TMA past its own K
    const uint64_t kb4 = ((uint64_t)K + 127) / 128 * 128;
    rc = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, kb4, b_rows, kb4 / 2, 128, b_box, true);
  } else {
    return MSGL_BAD_ARG;
  }
  if (rc) return rc;
  if (use_pair) {
    CUtensorMap msf = ma;  // placeholder for the kinds without scale atoms
    if (kind == KIND_MXF4) {
      // scale atoms as rows of 128 words: one tensor copy per 512-byte atom
      const uint64_t atoms = (uint64_t)args.sf_n_atoms * (uint64_t)args.sf_k_atoms;
      rc = make_map_2d(&msf, sf_atoms, CU_TENSOR_MAP_DATA_TYPE_UINT32, 128, atoms, 512, 128, 1, true, false);
      if (rc) return rc;
    }
    switch (kind) {
      case KIND_F16: return launch_pair<KIND_F16>(ma, mb, msf, args, max_ctas, stream);
      case KIND_BF16: return launch_pair<KIND_BF16>(ma, mb, msf, args, max_ctas, stream);
      case KIND_F8: return launch_pair<KIND_F8>(ma, mb, msf, args, max_ctas, stream);
      default: return launch_pair<KIND_MXF4>(ma, mb, msf, args, max_ctas, stream);
    }
  }
  switch (kind) {
    case KIND_F16: return dispatch_bn<KIND_F16>(bn, ma, mb, args, max_ctas, stream);
    case KIND_BF16: return dispatch_bn<KIND_BF16>(bn, ma, mb, args, max_ctas, stream);
    case KIND_F8: return dispatch_bn<KIND_F8>(bn, ma, mb, args, max_ctas, stream);
    default: return dispatch_bn<KIND_MXF4>(bn, ma, mb, args, max_ctas, stream);
  }
}

MSGL_API int msgl_gemm(int kind, const void* a, long long lda, const void* b, void* c, long long ldc, int M, int N,
                       int K, const void* a_scale, const void* b_scale, const void* bias, int bias_dtype,
                       const void* sf_atoms, int out_dtype, int bn_override, int max_ctas, cudaStream_t stream) {
  return gemm_impl(kind, a, lda, b, c, ldc, M, N, K, a_scale, b_scale, bias, bias_dtype, sf_atoms, out_dtype,
                   bn_override, max_ctas, nullptr, 0, stream);
}

// Split-K plan for small M: the number of K ranges depends on (kind, N, K) only, never on M, so a
// row's result is the same at every batch size this applies to (M <= 256). Returns 1 when the
// 128-wide tiles of two M tiles already fill half the GPU or K is short.
MSGL_API int msgl_gemm_splitk_plan(int kind, int N, int K) {
  const int bke = (kind == KIND_F16 || kind == KIND_BF16) ? 64 : 128;
  const int n_tiles = (N + 127) / 128, kbs = (K + bke - 1) / bke;
  int s = num_sms() / (2 * n_tiles);
  if (s > kbs / 8) s = kbs / 8;
  if (s > 8) s = 8;
  return s < 2 ? 1 : s;
}

// msgl_gemm for M <= 256 with `splits` K ranges per tile (msgl_gemm_splitk_plan). ws: fp32
// [splits][ceil(M/128)*128][ceil(N/128)*128]; counters: uint32 [ceil(M/128) * ceil(N/128)], zero on
// entry and zero again on exit.
MSGL_API int msgl_gemm_splitk(int kind, const void* a, long long lda, const void* b, void* c, long long ldc, int M,
                              int N, int K, const void* a_scale, const void* b_scale, const void* bias,
                              int bias_dtype, const void* sf_atoms, int out_dtype, int splits, void* ws,
                              void* counters, cudaStream_t stream) {
  if (M > 256 || splits < 2 || ws == nullptr || counters == nullptr) return MSGL_BAD_ARG;
  return gemm_impl(kind, a, lda, b, c, ldc, M, N, K, a_scale, b_scale, bias, bias_dtype, sf_atoms, out_dtype, 128, 0,
                   nullptr, 0, stream, nullptr, splits, ws, counters);
}

// Split-K without a reduction inside the GEMM: K range s of every tile writes its scaled partial
// sums to plane s of the fp32 output [splits][M][N] (ldc = N); the bias goes to plane 0. The
// consumer (msgl_rms_norm_planes) adds the planes in ascending order, so the result does not depend
// on scheduling. For M <= 256, where a projection with few N tiles would otherwise leave most
// SMs idle while a few walk a long K loop.
MSGL_API int msgl_gemm_splitk_planes(int kind, const void* a, long long lda, const void* b, void* planes, int M, int N,
                                     int K, const void* a_scale, const void* b_scale, const void* bias,
                                     int bias_dtype, const void* sf_atoms, int splits, cudaStream_t stream) {
  if (M > 256 || splits < 2 || planes == nullptr) return MSGL_BAD_ARG;
  return gemm_impl(kind, a, lda, b, planes, N, M, N, K, a_scale, b_scale, bias, bias_dtype, sf_atoms, MSGL_F32, 128, 0,
                   nullptr, 0, stream, nullptr, splits, nullptr, nullptr);
}

// msgl_gemm with the tensor-parallel fusions of the CTA-pair kernel: the epilogue can push its
// partial rows to the ranks that own them (GEMM -> reduce-scatter), and the producer can wait
// for A row blocks that other ranks are still delivering (all-gather -> GEMM).
MSGL_API int msgl_gemm_tp(int kind, const void* a, long long lda, const void* b, void* c, long long ldc, int M, int N,
                          int K, const void* a_scale, const void* b_scale, const void* bias, int bias_dtype,
                          const void* sf_atoms, int out_dtype, const MsglGemmTp* tp, cudaStream_t stream) {
  if (tp == nullptr) return MSGL_BAD_ARG;
  return gemm_impl(kind, a, lda, b, c, ldc, M, N, K, a_scale, b_scale, bias, bias_dtype, sf_atoms, out_dtype, 256, 0,
                   nullptr, 0, stream, tp);
}

// Grouped GEMM over expert-sorted rows: a [M, K] (M a multiple of 128), b [experts * N, K],
// tile_expert [M / 128] gives the expert of every 128-row tile (-1 = skip the tile).
// In grouped mode N tiles must not straddle experts, so N must be a multiple of the N tile.
MSGL_API int msgl_gemm_grouped(int kind, const void* a, long long lda, const void* b, void* c, long long ldc, int M,
                               int N, int K, const void* tile_expert, int num_experts, const void* a_scale,
                               const void* sf_atoms, int out_dtype, int bn_override, cudaStream_t stream) {
  if (M % 128 || tile_expert == nullptr || num_experts <= 0) return MSGL_BAD_ARG;
  int bn = bn_override;
  if (bn == 0) bn = (N % 128 == 0) ? 128 : (N % 64 == 0 ? 64 : 32);
  if (N % bn) {
    msgl_set_error_text("grouped gemm: N must be a multiple of the N tile");
    return MSGL_BAD_ARG;
  }
  return gemm_impl(kind, a, lda, b, c, ldc, M, N, K, a_scale, nullptr, nullptr, 0, sf_atoms, out_dtype, bn, 0,
                   tile_expert, num_experts, stream);
}

// Grouped W8A8 (kind 2): e4m3 rows with per-row scales against e4m3 expert weights with one
// scale per (expert, output channel): b_scale [experts * N] fp32.
MSGL_API int msgl_gemm_grouped_w8a8(const void* a, long long lda, const void* b, void* c, long long ldc, int M, int N,
                                    int K, const void* tile_expert, int num_experts, const void* a_scale,
                                    const void* b_scale, int out_dtype, int bn_override, cudaStream_t stream) {
  if (M % 128 || tile_expert == nullptr || num_experts <= 0 || b_scale == nullptr) return MSGL_BAD_ARG;
  int bn = bn_override;
  if (bn == 0) bn = (N % 128 == 0) ? 128 : (N % 64 == 0 ? 64 : 32);
  if (N % bn) {
    msgl_set_error_text("grouped gemm: N must be a multiple of the N tile");
    return MSGL_BAD_ARG;
  }
  return gemm_impl(KIND_F8, a, lda, b, c, ldc, M, N, K, a_scale, b_scale, nullptr, 0, nullptr, out_dtype, bn, 0,
                   tile_expert, num_experts, stream);
}

// Promise about the B operands (weights, scale atoms) of every GEMM call from now on: 1 = they
// were written before any kernel that can still be in flight on the calling stream (model
// parameters), so a kernel may fetch them before it has waited for the kernels ahead of it;
// 0 (default) = no promise, B is only read after that wait. Returns the previous setting.
int msgl_b_static_level() { return g_b_static; }   // for the other GEMM translation units

MSGL_API int msgl_gemm_static_weights(int on) {
  const int prev = g_b_static;
  g_b_static = on < 0 ? 0 : (on > 2 ? 2 : on);   // 2: also request the rest of a decode-sized item's weights into L2
  return prev;
}

// Tile-shape policy of msgl_gemm when bn_override is 0: 0 = CTA-pair kernel above 256 rows,
// 1 = single-CTA kernel always, 2 = CTA-pair kernel always. Returns the previous value.
MSGL_API int msgl_gemm_pair_mode(int mode) {
  const int prev = g_pair_mode;
  if (mode >= 0 && mode <= 2) g_pair_mode = mode;
  return prev;
}

// 0 when no bounded wait of a GEMM kernel has run out since the last reset; else a code
// (101 producer / 102 accumulator-free / 103 stage-full / 104 epilogue wait; 111-114 the same
// four waits of the CTA-pair kernel).
MSGL_API int msgl_gemm_status(int reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int));
  if (reset && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_gemm_status, &z, sizeof(int));
  }
  return v;
}
