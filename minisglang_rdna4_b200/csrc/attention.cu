// Paged attention over the KV pool: prefill, chunked extend over a cached prefix, decode
// (split-KV) and speculative verification with an optional additive tree mask, for bf16/f16
// and fp8-e4m3 KV with per-head descales.
//
// Replaces the reference's attn_hip / attn_decode / attn_prefill_paged packages
// (flash_prefill, flash_decode_paged[_fp8], flash_prefill_paged[_fp8] with mask_bias;
// python/minisgl/attention/hip.py:137,280-283,670-792, python/minisgl/attention/rdna4.py:419-503)
// and its flashinfer / FA call sites (python/minisgl/attention/trtllm.py:53-90).
//
// One kernel: a CTA owns up to 16*NW rows of one KV head, a row being a (query position, head
// of the GQA group) pair, and one KV range (split). A producer warp streams whole pages from
// the pool [pages, Hk, page, D] into 128-byte-swizzled shared-memory stages with TMA tensor
// copies driven by the block table; NW consumer warps run QK^T, online softmax and PV on the
// warp-level tensor-core path (decode is bound by KV bytes, not by tensor throughput). fp8 KV
// is converted to f16 in registers straight from the swizzled bytes (K through a permuted
// contraction index, V through a byte-permute after a transposing matrix load), so KV crosses
// HBM as one byte per element and is never re-materialised. Partial results of a split are
// merged by a second small kernel.
#include "common.cuh"
#include "ptx.cuh"

#include <string>
#include <type_traits>

using namespace msgl;
using namespace msgl::ptx;

namespace {

constexpr int TK = 64;       // KV tokens per stage
constexpr float kLog2e = 1.4426950408889634f;

struct AttnArgs {
  const void* q;
  void* out;
  const int32_t* block_table;
  int bt_stride;
  const int32_t* cu_q;
  const int32_t* seq_lens;
  const float* k_scale;
  const float* v_scale;
  const float* mask;
  long long mask_stride;
  int mask_window;   // > 0: a mask row covers only the last mask_window KV positions of its request; the rest is visible
  float* ws_o;
  float* ws_lse;
  int B, Hq, Hk, page_size, num_pages;
  int k_coord, v_coord;     // 5th tensor-map coordinate of this layer's K and V planes
  int causal, window, splits, total_q;
  float scale;
  int* status;
};

__device__ int g_attn_status = 0;

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_16816_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two e4m3 bytes (low 16 bits of x) -> f16x2
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t x) {
  uint32_t r;
  asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(r) : "r"(x));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_f16x2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// T: query/output element type. KV8: pool holds e4m3. MMA runs in f16 when KV8 or T == half,
// in bf16 otherwise.
// NWQ consumer warps side by side along the query rows (16 rows each) times NWK consumer warps
// that take turns on the KV tiles (warp wk owns tiles wk, wk + NWK, ...) and merge their partial
// softmax states at the end. Prefill uses 4 x 1, decode 1 x 4: a decode CTA has only one 16-row
// tile of queries, so its parallelism has to come from the KV axis.
template <typename T, bool KV8, int D, int NWQ, int NWK, int STAGES>
__global__ void __launch_bounds__(32 * (NWQ * NWK + 1))
paged_attention_kernel(const __grid_constant__ CUtensorMap kv_map, const AttnArgs args) {
  pdl_enter();
  constexpr int NW = NWQ * NWK;
  constexpr int ESZ = KV8 ? 1 : 2;
  constexpr int RB = D * ESZ;                 // bytes per KV row
  constexpr int PLANES = RB / 128;            // 128-byte planes per row
  constexpr int PLANE_BYTES = TK * 128;
  constexpr int KV_BYTES = PLANES * PLANE_BYTES;   // one of K / V per stage
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  constexpr int BOX_INNER = 128 / ESZ;
  constexpr bool F16MMA = KV8 || std::is_same<T, __half>::value;
  constexpr int NDB = D / 8;                  // 8-wide output column blocks

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar_base = s_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + STAGES * STAGE_BYTES + 16 * STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = args.Hq / args.Hk;
  const int ps = args.page_size;
  const int b = blockIdx.y / args.Hk, h = blockIdx.y % args.Hk;
  const int split = blockIdx.z;
  const int q_begin = args.cu_q[b], q_len = args.cu_q[b + 1] - q_begin;
  const int kv_len = args.seq_lens[b];
  const int pos_per_tile = (16 * NWQ) / G;
  // query tiles are handed out last-first: under a causal mask the late tiles see the most keys,
  // and starting them first leaves the short ones to fill the tail of the grid
  const int q_start = (int)(gridDim.x - 1 - blockIdx.x) * pos_per_tile;
  if (q_start >= q_len) return;   // uniform for the CTA; nothing has been initialised yet
  const int q_end = min(q_start + pos_per_tile, q_len);

  // KV range of this CTA (tokens), in whole TK tiles
  const bool use_mask = args.mask != nullptr;
  int kv_hi = (args.causal && !use_mask) ? min(kv_len, kv_len - q_len + q_end) : kv_len;
  int kv_lo = 0;
  if (args.window > 0 && !use_mask) kv_lo = max(0, (kv_len - q_len + q_start) - args.window + 1);
  const int tile_lo = kv_lo / TK;
  const int n_tiles_all = kv_hi > kv_lo ? (kv_hi + TK - 1) / TK - tile_lo : 0;
  const int per_split = (n_tiles_all + args.splits - 1) / args.splits;
  const int t_begin = tile_lo + split * per_split;
  const int t_end = min(tile_lo + n_tiles_all, t_begin + per_split);
  const int n_tiles = max(t_end - t_begin, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), NWQ);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&kv_map);
  }
  __syncthreads();

  if (warp == NW) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const int pages_per_tile = TK / ps;
      const int32_t* bt = args.block_table + (size_t)b * args.bt_stride;
      int stage = 0;
      uint32_t phase = 0;
      for (int t = 0; t < n_tiles; ++t) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, args.status, 201)) break;
        mbar_expect_tx(full_bar(stage), STAGE_BYTES);
        const int first_page = (t_begin + t) * pages_per_tile;
        const uint32_t k_s = s_base + stage * STAGE_BYTES, v_s = k_s + KV_BYTES;
        for (int p = 0; p < pages_per_tile; ++p) {
          int col = first_page + p;
          col = col < args.bt_stride ? col : args.bt_stride - 1;
          int page = bt[col];
          (void)MSGL_OOB(page, args.num_pages + 1);
          page = page < 0 ? 0 : (page > args.num_pages ? args.num_pages : page);
#pragma unroll
          for (int pl = 0; pl < PLANES; ++pl) {
            const uint32_t off = pl * PLANE_BYTES + p * ps * 128;
            tma_load_5d(k_s + off, &kv_map, full_bar(stage), pl * BOX_INNER, 0, h, page, args.k_coord);
            tma_load_5d(v_s + off, &kv_map, full_bar(stage), pl * BOX_INNER, 0, h, page, args.v_coord);
          }
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  const int j = lane & 3, r0 = lane >> 2;
  const int wq = warp / NWK, wk = warp % NWK;
  const int row_a = wq * 16 + r0, row_b = row_a + 8;            // rows of this thread in the tile
  const int qi_a = q_start + row_a / G, qi_b = q_start + row_b / G;
  const bool ok_a = qi_a < q_end, ok_b = qi_b < q_end;
  const int head_a = h * G + row_a % G, head_b = h * G + row_b % G;
  const size_t qoff_a = ((size_t)(q_begin + (ok_a ? qi_a : q_start)) * args.Hq + head_a) * D;
  const size_t qoff_b = ((size_t)(q_begin + (ok_b ? qi_b : q_start)) * args.Hq + head_b) * D;

  // ---- Q fragments (A operand), converted once
  uint32_t qf[D / 16][4];
  {
    const T* qa = reinterpret_cast<const T*>(args.q) + qoff_a;
    const T* qb = reinterpret_cast<const T*>(args.q) + qoff_b;
#pragma unroll
    for (int c = 0; c < D / 16; ++c) {
      float xa[4], xb[4];
      if (KV8) {
        // fp8 K arrives with four consecutive d per thread: a0/a1 take d+0,1 and a2/a3 d+2,3
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          xa[e] = to_float(qa[c * 16 + 4 * j + e]);
          xb[e] = to_float(qb[c * 16 + 4 * j + e]);
        }
      } else {
        xa[0] = to_float(qa[c * 16 + 2 * j]);     xa[1] = to_float(qa[c * 16 + 2 * j + 1]);
        xa[2] = to_float(qa[c * 16 + 8 + 2 * j]); xa[3] = to_float(qa[c * 16 + 8 + 2 * j + 1]);
        xb[0] = to_float(qb[c * 16 + 2 * j]);     xb[1] = to_float(qb[c * 16 + 2 * j + 1]);
        xb[2] = to_float(qb[c * 16 + 8 + 2 * j]); xb[3] = to_float(qb[c * 16 + 8 + 2 * j + 1]);
      }
      if (F16MMA) {
        qf[c][0] = pack_f16x2(xa[0], xa[1]); qf[c][1] = pack_f16x2(xb[0], xb[1]);
        qf[c][2] = pack_f16x2(xa[2], xa[3]); qf[c][3] = pack_f16x2(xb[2], xb[3]);
      } else {
        qf[c][0] = pack_bf16x2(xa[0], xa[1]); qf[c][1] = pack_bf16x2(xb[0], xb[1]);
        qf[c][2] = pack_bf16x2(xa[2], xa[3]); qf[c][3] = pack_bf16x2(xb[2], xb[3]);
      }
    }
  }

  const float k_sc = args.k_scale != nullptr ? args.k_scale[h] : 1.f;
  const float v_sc = args.v_scale != nullptr ? args.v_scale[h] : 1.f;
  const float sm_scale = args.scale * k_sc * kLog2e;
  // per-row visible KV interval [lo, hi)
  const int pos_a = kv_len - q_len + qi_a, pos_b = kv_len - q_len + qi_b;
  int hi_a = kv_len, hi_b = kv_len, lo_a = 0, lo_b = 0;
  if (!use_mask) {
    if (args.causal) { hi_a = min(kv_len, pos_a + 1); hi_b = min(kv_len, pos_b + 1); }
    if (args.window > 0) { lo_a = max(0, pos_a - args.window + 1); lo_b = max(0, pos_b - args.window + 1); }
  }
  if (!ok_a) hi_a = 0;
  if (!ok_b) hi_b = 0;
  const int mask_lo = args.mask_window > 0 ? kv_len - args.mask_window : 0;   // negative for a sequence shorter than the window
  const float* mask_a = use_mask ? args.mask + (size_t)(q_begin + (ok_a ? qi_a : q_start)) * args.mask_stride : nullptr;
  const float* mask_b = use_mask ? args.mask + (size_t)(q_begin + (ok_b ? qi_b : q_start)) * args.mask_stride : nullptr;

  float o[NDB][4];
#pragma unroll
  for (int i = 0; i < NDB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

  for (int t = wk; t < n_tiles; t += NWK) {
    const int stage = t % STAGES;
    const uint32_t phase = (uint32_t)(t / STAGES) & 1u;
    if (!mbar_wait(full_bar(stage), phase, abort_flag, args.status, 202)) break;
    const uint32_t k_s = s_base + stage * STAGE_BYTES, v_s = k_s + KV_BYTES;
    const int tok0 = (t_begin + t) * TK;

    // ---- S = Q K^T
    float s[TK / 8][4];
#pragma unroll
    for (int nb = 0; nb < TK / 8; ++nb) {
      s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
      const int trow = nb * 8 + (lane & 7);
      if (KV8) {
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf) {
          const int chunk = hf * 4 + (lane >> 3);
          uint32_t kr[4];
          ldmatrix_x4(k_s + (chunk >> 3) * PLANE_BYTES + trow * 128 + (((chunk & 7) ^ (trow & 7)) << 4), kr);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            mma_16816_f16(s[nb], qf[hf * 4 + i], e4m3x2_to_f16x2(kr[i]), e4m3x2_to_f16x2(kr[i] >> 16));
        }
      } else {
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          const int chunk = cc * 4 + (lane >> 3);   // 16-byte chunk of the 2*D-byte row
          uint32_t kr[4];
          ldmatrix_x4(k_s + (chunk >> 3) * PLANE_BYTES + trow * 128 + (((chunk & 7) ^ (trow & 7)) << 4), kr);
          if (F16MMA) {
            mma_16816_f16(s[nb], qf[2 * cc], kr[0], kr[1]);
            mma_16816_f16(s[nb], qf[2 * cc + 1], kr[2], kr[3]);
          } else {
            mma_16816_bf16(s[nb], qf[2 * cc], kr[0], kr[1]);
            mma_16816_bf16(s[nb], qf[2 * cc + 1], kr[2], kr[3]);
          }
        }
      }
    }

    // ---- scale, mask, online softmax (base-2)
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < TK / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int tok = tok0 + nb * 8 + 2 * j + e;
        float va = s[nb][e] * sm_scale, vb = s[nb][2 + e] * sm_scale;
        if (use_mask) {
          const int mt = tok - mask_lo;   // negative: ahead of the masked window, visible to every row
          va = (tok < hi_a) ? (mt >= 0 ? va + mask_a[mt] * kLog2e : va) : -INFINITY;
          vb = (tok < hi_b) ? (mt >= 0 ? vb + mask_b[mt] * kLog2e : vb) : -INFINITY;
        } else {
          if (tok >= hi_a || tok < lo_a) va = -INFINITY;
          if (tok >= hi_b || tok < lo_b) vb = -INFINITY;
        }
        s[nb][e] = va;
        s[nb][2 + e] = vb;
        mx_a = fmaxf(mx_a, va);
        mx_b = fmaxf(mx_b, vb);
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float ms_a = mn_a == -INFINITY ? 0.f : mn_a, ms_b = mn_b == -INFINITY ? 0.f : mn_b;
    const float al_a = fast_exp2(m_a - ms_a), al_b = fast_exp2(m_b - ms_b);   // exp2(-inf) = 0
    m_a = mn_a;
    m_b = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int nb = 0; nb < TK / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float pa = fast_exp2(s[nb][e] - ms_a), pb = fast_exp2(s[nb][2 + e] - ms_b);
        s[nb][e] = pa;
        s[nb][2 + e] = pb;
        sum_a += pa;
        sum_b += pb;
      }
    }
    l_a = l_a * al_a + sum_a;
    l_b = l_b * al_b + sum_b;
#pragma unroll
    for (int i = 0; i < NDB; ++i) {
      o[i][0] *= al_a; o[i][1] *= al_a;
      o[i][2] *= al_b; o[i][3] *= al_b;
    }

    // ---- O += P V
#pragma unroll
    for (int ks = 0; ks < TK / 16; ++ks) {
      uint32_t pa[4];
      if (F16MMA) {
        pa[0] = pack_f16x2(s[2 * ks][0], s[2 * ks][1]);         pa[1] = pack_f16x2(s[2 * ks][2], s[2 * ks][3]);
        pa[2] = pack_f16x2(s[2 * ks + 1][0], s[2 * ks + 1][1]); pa[3] = pack_f16x2(s[2 * ks + 1][2], s[2 * ks + 1][3]);
      } else {
        pa[0] = pack_bf16x2(s[2 * ks][0], s[2 * ks][1]);         pa[1] = pack_bf16x2(s[2 * ks][2], s[2 * ks][3]);
        pa[2] = pack_bf16x2(s[2 * ks + 1][0], s[2 * ks + 1][1]); pa[3] = pack_bf16x2(s[2 * ks + 1][2], s[2 * ks + 1][3]);
      }
      const int mi = lane >> 3;
      const int trow = ks * 16 + (mi & 1) * 8 + (lane & 7);
      if (KV8) {
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          const int chunk = 2 * cc + (mi >> 1);
          uint32_t vr[4];
          ldmatrix_x4_trans(v_s + (chunk >> 3) * PLANE_BYTES + trow * 128 + (((chunk & 7) ^ (trow & 7)) << 4), vr);
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            const uint32_t we = __byte_perm(vr[2 * c2], vr[2 * c2 + 1], 0x6420);
            const uint32_t wo = __byte_perm(vr[2 * c2], vr[2 * c2 + 1], 0x7531);
            mma_16816_f16(o[4 * cc + 2 * c2], pa, e4m3x2_to_f16x2(we), e4m3x2_to_f16x2(we >> 16));
            mma_16816_f16(o[4 * cc + 2 * c2 + 1], pa, e4m3x2_to_f16x2(wo), e4m3x2_to_f16x2(wo >> 16));
          }
        }
      } else {
#pragma unroll
        for (int cc = 0; cc < D / 16; ++cc) {
          const int chunk = 2 * cc + (mi >> 1);
          uint32_t vr[4];
          ldmatrix_x4_trans(v_s + (chunk >> 3) * PLANE_BYTES + trow * 128 + (((chunk & 7) ^ (trow & 7)) << 4), vr);
          if (F16MMA) {
            mma_16816_f16(o[2 * cc], pa, vr[0], vr[1]);
            mma_16816_f16(o[2 * cc + 1], pa, vr[2], vr[3]);
          } else {
            mma_16816_bf16(o[2 * cc], pa, vr[0], vr[1]);
            mma_16816_bf16(o[2 * cc + 1], pa, vr[2], vr[3]);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(stage));
  }

  // ---- finalise
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  if (NWK > 1) {
    // Merge the NWK partial states of each query tile. Every warp parks its accumulator
    // fragments in shared memory in register order ([reg][lane], so the same thread index of
    // another warp holds the same matrix element); warp wk == 0 then folds them in.
    constexpr int REGS = NDB * 4 + 4;
    float* park = reinterpret_cast<float*>(smem);   // the KV stages are dead by now
    asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
    if (wk != 0) {
      float* mine = park + (size_t)((wq * (NWK - 1) + (wk - 1)) * REGS) * 32 + lane;
#pragma unroll
      for (int i = 0; i < NDB; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) mine[(i * 4 + e) * 32] = o[i][e];
      }
      mine[(NDB * 4 + 0) * 32] = m_a;
      mine[(NDB * 4 + 1) * 32] = m_b;
      mine[(NDB * 4 + 2) * 32] = l_a;
      mine[(NDB * 4 + 3) * 32] = l_b;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(NW * 32) : "memory");
    if (wk != 0) return;
#pragma unroll 1
    for (int other = 0; other < NWK - 1; ++other) {
      const float* src = park + (size_t)((wq * (NWK - 1) + other) * REGS) * 32 + lane;
      const float om_a = src[(NDB * 4 + 0) * 32], om_b = src[(NDB * 4 + 1) * 32];
      const float ol_a = src[(NDB * 4 + 2) * 32], ol_b = src[(NDB * 4 + 3) * 32];
      const float nm_a = fmaxf(m_a, om_a), nm_b = fmaxf(m_b, om_b);
      const float sa = nm_a == -INFINITY ? 0.f : nm_a, sb = nm_b == -INFINITY ? 0.f : nm_b;
      const float f_a = fast_exp2(m_a - sa), g_a = fast_exp2(om_a - sa);
      const float f_b = fast_exp2(m_b - sb), g_b = fast_exp2(om_b - sb);
#pragma unroll
      for (int i = 0; i < NDB; ++i) {
        o[i][0] = o[i][0] * f_a + src[(i * 4 + 0) * 32] * g_a;
        o[i][1] = o[i][1] * f_a + src[(i * 4 + 1) * 32] * g_a;
        o[i][2] = o[i][2] * f_b + src[(i * 4 + 2) * 32] * g_b;
        o[i][3] = o[i][3] * f_b + src[(i * 4 + 3) * 32] * g_b;
      }
      l_a = l_a * f_a + ol_a * g_a;
      l_b = l_b * f_b + ol_b * g_b;
      m_a = nm_a;
      m_b = nm_b;
    }
  }
  const float inv_a = l_a > 0.f ? v_sc / l_a : 0.f, inv_b = l_b > 0.f ? v_sc / l_b : 0.f;

  // column of accumulator element (block i, e) for this thread
  auto col_of = [&](int i, int e) -> int {
    if (KV8) return (i >> 1) * 16 + 4 * j + 2 * e + (i & 1);
    return i * 8 + 2 * j + e;
  };
  if (args.splits == 1) {
    T* oa = reinterpret_cast<T*>(args.out) + qoff_a;
    T* ob = reinterpret_cast<T*>(args.out) + qoff_b;
    if (KV8) {
#pragma unroll
      for (int c = 0; c < D / 16; ++c) {
        // four consecutive d per thread: blocks 2c (even d) and 2c+1 (odd d)
        if (ok_a) {
          typename Pack2<T>::type lo = Pack2<T>::make(o[2 * c][0] * inv_a, o[2 * c + 1][0] * inv_a);
          typename Pack2<T>::type hi = Pack2<T>::make(o[2 * c][1] * inv_a, o[2 * c + 1][1] * inv_a);
          *reinterpret_cast<uint2*>(oa + c * 16 + 4 * j) =
              make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
        if (ok_b) {
          typename Pack2<T>::type lo = Pack2<T>::make(o[2 * c][2] * inv_b, o[2 * c + 1][2] * inv_b);
          typename Pack2<T>::type hi = Pack2<T>::make(o[2 * c][3] * inv_b, o[2 * c + 1][3] * inv_b);
          *reinterpret_cast<uint2*>(ob + c * 16 + 4 * j) =
              make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < NDB; ++i) {
        if (ok_a) *reinterpret_cast<typename Pack2<T>::type*>(oa + i * 8 + 2 * j) = Pack2<T>::make(o[i][0] * inv_a, o[i][1] * inv_a);
        if (ok_b) *reinterpret_cast<typename Pack2<T>::type*>(ob + i * 8 + 2 * j) = Pack2<T>::make(o[i][2] * inv_b, o[i][3] * inv_b);
      }
    }
  } else {
    const size_t plane = (size_t)args.total_q * args.Hq;
    float* wa = args.ws_o + ((size_t)split * plane + (size_t)(q_begin + qi_a) * args.Hq + head_a) * D;
    float* wb = args.ws_o + ((size_t)split * plane + (size_t)(q_begin + qi_b) * args.Hq + head_b) * D;
#pragma unroll
    for (int i = 0; i < NDB; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (ok_a) wa[col_of(i, e)] = o[i][e] * inv_a;
        if (ok_b) wb[col_of(i, e)] = o[i][2 + e] * inv_b;
      }
    }
    if (j == 0) {
      if (ok_a) args.ws_lse[(size_t)split * plane + (size_t)(q_begin + qi_a) * args.Hq + head_a] =
          l_a > 0.f ? m_a + log2f(l_a) : -INFINITY;
      if (ok_b) args.ws_lse[(size_t)split * plane + (size_t)(q_begin + qi_b) * args.Hq + head_b] =
          l_b > 0.f ? m_b + log2f(l_b) : -INFINITY;
    }
  }
}

// merge split partials: one warp per (query row, head)
template <typename T, int D>
__global__ void attn_combine_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_lse,
                                    T* __restrict__ out, int rows_heads, int splits,
                                    const int32_t* __restrict__ cu_q, int B, int hq) {
  pdl_enter();
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (idx >= rows_heads) return;
  const int lane = threadIdx.x & 31;
  // rows past cu_q[B] belong to no request (padding of a captured batch): the split kernels wrote
  // no partials for them, so they are zero-filled instead of merged from whatever the workspace holds
  if (idx >= cu_q[B] * hq) {
    T* pad = out + (size_t)idx * D + lane * (D / 32);
#pragma unroll
    for (int i = 0; i < D / 32; ++i) pad[i] = from_float<T>(0.f);
    return;
  }
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, ws_lse[(size_t)s * rows_heads + idx]);
  constexpr int PER = D / 32;
  float acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  float wsum = 0.f;
  if (mx > -INFINITY) {
    for (int s = 0; s < splits; ++s) {
      const float w = exp2f(ws_lse[(size_t)s * rows_heads + idx] - mx);
      if (w == 0.f) continue;
      wsum += w;
      const float* src = ws_o + ((size_t)s * rows_heads + idx) * D + lane * PER;
#pragma unroll
      for (int i = 0; i < PER; ++i) acc[i] += w * src[i];
    }
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  T* dst = out + (size_t)idx * D + lane * PER;
#pragma unroll
  for (int i = 0; i < PER; ++i) dst[i] = from_float<T>(acc[i] * inv);
}

// ------------------------------------------------------------------------------------------
// Decode (one query position per request). The problem is transposed so that the 16-row side of
// the warp MMA is filled with KV tokens and the 8-column side with the (up to 8) query heads of
// one GQA group: S^T = K Q^T and O^T = V^T P^T. Compared with putting the heads on the 16-row
// side this halves the MMA and softmax work per token, halves the accumulator registers (so
// several times more CTAs fit on an SM, which is what hides the latency of the dependent
// ldmatrix -> convert -> mma chains) and wastes nothing when the group has 8 heads.
// P is transposed between the two products with movmatrix.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

template <typename T, bool KV8, int D, int STAGES>
__global__ void __launch_bounds__(64)
paged_decode_kernel(const __grid_constant__ CUtensorMap kv_map, const AttnArgs args) {
  // This kernel starts once the kernel ahead of it (the one that writes this step's q and the
  // newest token's K / V) has begun, which is after everything before THAT kernel has finished.
  // So the step's tables and all older KV may be read at once; only q and the tile that holds
  // position kv_len - 1 wait for pdl_wait().
  constexpr int ESZ = KV8 ? 1 : 2;
  constexpr int RB = D * ESZ;
  constexpr int PLANES = RB / 128;
  constexpr int PLANE_BYTES = TK * 128;
  constexpr int KV_BYTES = PLANES * PLANE_BYTES;
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  constexpr int BOX_INNER = 128 / ESZ;
  constexpr bool F16MMA = KV8 || std::is_same<T, __half>::value;
  constexpr int NMB = D / 16;   // 16-row blocks of O^T

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bar_base = s_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + STAGES * STAGE_BYTES + 16 * STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = args.Hq / args.Hk;
  const int ps = args.page_size;
  const int b = blockIdx.y / args.Hk, h = blockIdx.y % args.Hk;
  const int split = blockIdx.z;
  const int q_row = args.cu_q[b];
  const int kv_len = args.seq_lens[b];
  const int kv_hi = kv_len;
  const int kv_lo = args.window > 0 ? max(0, kv_len - args.window) : 0;
  const int tile_lo = kv_lo / TK;
  const int n_tiles_all = kv_hi > kv_lo ? (kv_hi + TK - 1) / TK - tile_lo : 0;
  const int per_split = (n_tiles_all + args.splits - 1) / args.splits;
  const int t_begin = tile_lo + split * per_split;
  const int t_end = min(tile_lo + n_tiles_all, t_begin + per_split);
  const int n_tiles = max(t_end - t_begin, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&kv_map);
  }
  __syncthreads();

  if (warp == 1) {
    if (lane == 0) {
      const int pages_per_tile = TK / ps;
      const int32_t* bt = args.block_table + (size_t)b * args.bt_stride;
      int stage = 0;
      uint32_t phase = 0;
      const int newest_tile = kv_len > 0 ? (kv_len - 1) / TK : 0;
      bool waited = false;
      for (int t = 0; t < n_tiles; ++t) {
        if (!waited && t_begin + t >= newest_tile) {
          pdl_wait();
          waited = true;
        }
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, args.status, 211)) break;
        mbar_expect_tx(full_bar(stage), STAGE_BYTES);
        const int first_page = (t_begin + t) * pages_per_tile;
        const uint32_t k_s = s_base + stage * STAGE_BYTES, v_s = k_s + KV_BYTES;
        for (int p = 0; p < pages_per_tile; ++p) {
          int col = first_page + p;
          col = col < args.bt_stride ? col : args.bt_stride - 1;
          int page = bt[col];
          (void)MSGL_OOB(page, args.num_pages + 1);
          page = page < 0 ? 0 : (page > args.num_pages ? args.num_pages : page);
#pragma unroll
          for (int pl = 0; pl < PLANES; ++pl) {
            const uint32_t off = pl * PLANE_BYTES + p * ps * 128;
            tma_load_5d(k_s + off, &kv_map, full_bar(stage), pl * BOX_INNER, 0, h, page, args.k_coord);
            tma_load_5d(v_s + off, &kv_map, full_bar(stage), pl * BOX_INNER, 0, h, page, args.v_coord);
          }
        }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
    return;
  }

  // ---------------------------------------------------------------------- consumer warp
  pdl_enter();
  const int j = lane & 3, g = lane >> 2;
  const int mi = lane >> 3;
  // Q^T fragments (B operand): column n = g is head h*G + g
  uint32_t qb[NMB][2];
  {
    const bool head_ok = g < G;
    const T* qp = reinterpret_cast<const T*>(args.q) + ((size_t)q_row * args.Hq + h * G + (head_ok ? g : 0)) * D;
#pragma unroll
    for (int c = 0; c < NMB; ++c) {
      float x[4];
      if (KV8) {
#pragma unroll
        for (int e = 0; e < 4; ++e) x[e] = head_ok ? to_float(qp[c * 16 + 4 * j + e]) : 0.f;
      } else {
        x[0] = head_ok ? to_float(qp[c * 16 + 2 * j]) : 0.f;
        x[1] = head_ok ? to_float(qp[c * 16 + 2 * j + 1]) : 0.f;
        x[2] = head_ok ? to_float(qp[c * 16 + 8 + 2 * j]) : 0.f;
        x[3] = head_ok ? to_float(qp[c * 16 + 8 + 2 * j + 1]) : 0.f;
      }
      qb[c][0] = F16MMA ? pack_f16x2(x[0], x[1]) : pack_bf16x2(x[0], x[1]);
      qb[c][1] = F16MMA ? pack_f16x2(x[2], x[3]) : pack_bf16x2(x[2], x[3]);
    }
  }
  const float k_sc = args.k_scale != nullptr ? args.k_scale[h] : 1.f;
  const float v_sc = args.v_scale != nullptr ? args.v_scale[h] : 1.f;
  const float sm_scale = args.scale * k_sc * kLog2e;

  float ot[NMB][4];
#pragma unroll
  for (int i = 0; i < NMB; ++i) { ot[i][0] = ot[i][1] = ot[i][2] = ot[i][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // heads 2j and 2j+1

  int stage = 0;
  uint32_t phase = 0;
  for (int t = 0; t < n_tiles; ++t) {
    if (!mbar_wait(full_bar(stage), phase, abort_flag, args.status, 212)) break;
    const uint32_t k_s = s_base + stage * STAGE_BYTES, v_s = k_s + KV_BYTES;
    const int tok0 = (t_begin + t) * TK;

    // ---- S^T = K Q^T : four blocks of 16 tokens x 8 heads
    float st[TK / 16][4];
#pragma unroll
    for (int tb = 0; tb < TK / 16; ++tb) {
      st[tb][0] = st[tb][1] = st[tb][2] = st[tb][3] = 0.f;
      const int trow = tb * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
      for (int cp = 0; cp < RB / 32; ++cp) {
        const int chunk = 2 * cp + (mi >> 1);
        uint32_t r[4];
        ldmatrix_x4(k_s + (chunk >> 3) * PLANE_BYTES + trow * 128 + (((chunk & 7) ^ (trow & 7)) << 4), r);
        if (KV8) {
          // one 16-byte chunk = 16 d = one k-step; the pair of chunks gives two k-steps
          uint32_t a[4] = {e4m3x2_to_f16x2(r[0]), e4m3x2_to_f16x2(r[1]), e4m3x2_to_f16x2(r[0] >> 16),
                           e4m3x2_to_f16x2(r[1] >> 16)};
          mma_16816_f16(st[tb], a, qb[2 * cp][0], qb[2 * cp][1]);
          uint32_t a2[4] = {e4m3x2_to_f16x2(r[2]), e4m3x2_to_f16x2(r[3]), e4m3x2_to_f16x2(r[2] >> 16),
                            e4m3x2_to_f16x2(r[3] >> 16)};
          mma_16816_f16(st[tb], a2, qb[2 * cp + 1][0], qb[2 * cp + 1][1]);
        } else {
          // two 16-byte chunks = 16 d = one k-step
          if (F16MMA) mma_16816_f16(st[tb], r, qb[cp][0], qb[cp][1]);
          else mma_16816_bf16(st[tb], r, qb[cp][0], qb[cp][1]);
        }
      }
    }

    // ---- scale, mask, online softmax over the token axis (per head column)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int tb = 0; tb < TK / 16; ++tb) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int tok = tok0 + tb * 16 + g + 8 * hf;
        const bool ok = tok >= kv_lo && tok < kv_hi;
        const float a0 = ok ? st[tb][2 * hf] * sm_scale : -INFINITY;
        const float a1 = ok ? st[tb][2 * hf + 1] * sm_scale : -INFINITY;
        st[tb][2 * hf] = a0;
        st[tb][2 * hf + 1] = a1;
        mx0 = fmaxf(mx0, a0);
        mx1 = fmaxf(mx1, a1);
      }
    }
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
    const float al0 = fast_exp2(m0 - ms0), al1 = fast_exp2(m1 - ms1);
    m0 = mn0;
    m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int tb = 0; tb < TK / 16; ++tb) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const float p0 = fast_exp2(st[tb][2 * hf] - ms0), p1 = fast_exp2(st[tb][2 * hf + 1] - ms1);
        st[tb][2 * hf] = p0;
        st[tb][2 * hf + 1] = p1;
        sum0 += p0;
        sum1 += p1;
      }
    }
    l0 = l0 * al0 + sum0;
    l1 = l1 * al1 + sum1;
#pragma unroll
    for (int i = 0; i < NMB; ++i) {
      ot[i][0] *= al0; ot[i][1] *= al1;
      ot[i][2] *= al0; ot[i][3] *= al1;
    }

    // ---- O^T += V^T P^T
#pragma unroll
    for (int tb = 0; tb < TK / 16; ++tb) {
      uint32_t p01, p23;
      if (F16MMA) { p01 = pack_f16x2(st[tb][0], st[tb][1]); p23 = pack_f16x2(st[tb][2], st[tb][3]); }
      else { p01 = pack_bf16x2(st[tb][0], st[tb][1]); p23 = pack_bf16x2(st[tb][2], st[tb][3]); }
      const uint32_t pb0 = movmatrix_trans(p01), pb1 = movmatrix_trans(p23);
      if (KV8) {
        const int trow = tb * 16 + (mi & 1) * 8 + (lane & 7);
#pragma unroll
        for (int cp = 0; cp < D / 32; ++cp) {
          const int chunk = 2 * cp + (mi >> 1);
          uint32_t r[4];
          ldmatrix_x4_trans(v_s + (chunk >> 3) * PLANE_BYTES + trow * 128 + (((chunk & 7) ^ (trow & 7)) << 4), r);
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            // rows 0..7 of the block are the even d of the chunk, rows 8..15 the odd d
            const uint32_t we = __byte_perm(r[2 * c2], r[2 * c2 + 1], 0x6420);
            const uint32_t wo = __byte_perm(r[2 * c2], r[2 * c2 + 1], 0x7531);
            uint32_t a[4] = {e4m3x2_to_f16x2(we), e4m3x2_to_f16x2(wo), e4m3x2_to_f16x2(we >> 16),
                             e4m3x2_to_f16x2(wo >> 16)};
            mma_16816_f16(ot[2 * cp + c2], a, pb0, pb1);
          }
        }
      } else {
        const int trow = tb * 16 + (mi >> 1) * 8 + (lane & 7);
#pragma unroll
        for (int mb = 0; mb < NMB; ++mb) {
          const int chunk = 2 * mb + (mi & 1);
          uint32_t r[4];
          ldmatrix_x4_trans(v_s + (chunk >> 3) * PLANE_BYTES + trow * 128 + (((chunk & 7) ^ (trow & 7)) << 4), r);
          if (F16MMA) mma_16816_f16(ot[mb], r, pb0, pb1);
          else mma_16816_bf16(ot[mb], r, pb0, pb1);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(stage));
    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
  }

  // ---- finalise: sums over the token lanes, then write heads 2j and 2j+1
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, o);
    l1 += __shfl_xor_sync(0xffffffffu, l1, o);
  }
  const float inv0 = l0 > 0.f ? v_sc / l0 : 0.f, inv1 = l1 > 0.f ? v_sc / l1 : 0.f;
  const bool ok0 = 2 * j < G, ok1 = 2 * j + 1 < G;
  const int head0 = h * G + 2 * j, head1 = head0 + 1;
  if (args.splits == 1) {
    T* o0 = reinterpret_cast<T*>(args.out) + ((size_t)q_row * args.Hq + head0) * D;
    T* o1 = reinterpret_cast<T*>(args.out) + ((size_t)q_row * args.Hq + head1) * D;
#pragma unroll
    for (int c = 0; c < NMB; ++c) {
      if (KV8) {
        // this thread holds d = 16c + 2g and 16c + 2g + 1 of both heads
        if (ok0) *reinterpret_cast<typename Pack2<T>::type*>(o0 + c * 16 + 2 * g) = Pack2<T>::make(ot[c][0] * inv0, ot[c][2] * inv0);
        if (ok1) *reinterpret_cast<typename Pack2<T>::type*>(o1 + c * 16 + 2 * g) = Pack2<T>::make(ot[c][1] * inv1, ot[c][3] * inv1);
      } else {
        if (ok0) { o0[c * 16 + g] = from_float<T>(ot[c][0] * inv0); o0[c * 16 + 8 + g] = from_float<T>(ot[c][2] * inv0); }
        if (ok1) { o1[c * 16 + g] = from_float<T>(ot[c][1] * inv1); o1[c * 16 + 8 + g] = from_float<T>(ot[c][3] * inv1); }
      }
    }
  } else {
    const size_t plane = (size_t)args.total_q * args.Hq;
    float* w0 = args.ws_o + ((size_t)split * plane + (size_t)q_row * args.Hq + head0) * D;
    float* w1 = args.ws_o + ((size_t)split * plane + (size_t)q_row * args.Hq + head1) * D;
#pragma unroll
    for (int c = 0; c < NMB; ++c) {
      const int d0 = KV8 ? c * 16 + 2 * g : c * 16 + g;
      const int d1 = KV8 ? d0 + 1 : d0 + 8;
      if (ok0) { w0[d0] = ot[c][0] * inv0; w0[d1] = ot[c][2] * inv0; }
      if (ok1) { w1[d0] = ot[c][1] * inv1; w1[d1] = ot[c][3] * inv1; }
    }
    if (g == 0) {
      if (ok0) args.ws_lse[(size_t)split * plane + (size_t)q_row * args.Hq + head0] = l0 > 0.f ? m0 + log2f(l0) : -INFINITY;
      if (ok1) args.ws_lse[(size_t)split * plane + (size_t)q_row * args.Hq + head1] = l1 > 0.f ? m1 + log2f(l1) : -INFINITY;
    }
  }
}

template <typename T, bool KV8, int D, int STAGES>
int launch_decode(const CUtensorMap& map, const AttnArgs& a, cudaStream_t stream) {
  constexpr int ESZ = KV8 ? 1 : 2;
  constexpr int smem = STAGES * 2 * (D * ESZ / 128) * TK * 128 + 16 * STAGES + 64 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_kernel<T, KV8, D, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { msgl_set_error("decode attention smem attribute", e); return MSGL_CUDA_ERROR; }
    configured = true;
  }
  dim3 grid(1, a.B * a.Hk, a.splits);
  msgl_launch(paged_decode_kernel<T, KV8, D, STAGES>, dim3(grid), dim3(64), smem, stream, map, a);
  MSGL_CHECK_LAUNCH("paged_decode");
  return MSGL_OK;
}

template <typename T, bool KV8, int D, int NWQ, int NWK, int STAGES>
int launch_attn(const CUtensorMap& map, const AttnArgs& a, int q_tiles, cudaStream_t stream) {
  constexpr int ESZ = KV8 ? 1 : 2;
  constexpr int NW = NWQ * NWK;
  constexpr int smem = STAGES * 2 * (D * ESZ / 128) * TK * 128 + 16 * STAGES + 64 + 1024;
  static_assert(NWK == 1 || NWQ * (NWK - 1) * (D / 8 * 4 + 4) * 32 * 4 <= STAGES * 2 * (D * ESZ / 128) * TK * 128,
                "merge buffer must fit in the stage memory");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(paged_attention_kernel<T, KV8, D, NWQ, NWK, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { msgl_set_error("attention smem attribute", e); return MSGL_CUDA_ERROR; }
    configured = true;
  }
  dim3 grid(q_tiles, a.B * a.Hk, a.splits);
  msgl_launch(paged_attention_kernel<T, KV8, D, NWQ, NWK, STAGES>, dim3(grid), dim3(32 * (NW + 1)), smem, stream, map, a);
  MSGL_CHECK_LAUNCH("paged_attention");
  return MSGL_OK;
}

bool g_force_general_decode = false;
int g_decode_stages = 2;   // shared-memory stages of the fp8 decode kernel (2, 3 or 4)

template <typename T>
int dispatch_attn(const CUtensorMap& map, const AttnArgs& a, bool kv8, int d, int max_q, cudaStream_t stream) {
  const int G = a.Hq / a.Hk;
  if (max_q == 1 && G <= 8 && a.mask == nullptr && !g_force_general_decode) {
    if (d == 128) {
      if (kv8) {
        if (g_decode_stages == 3) return launch_decode<T, true, 128, 3>(map, a, stream);
        if (g_decode_stages == 4) return launch_decode<T, true, 128, 4>(map, a, stream);
        return launch_decode<T, true, 128, 2>(map, a, stream);
      }
      return launch_decode<T, false, 128, 2>(map, a, stream);
    }
    if (d == 64 && !kv8) return launch_decode<T, false, 64, 3>(map, a, stream);
  }
  const bool small = max_q * G <= 16;
  const int rows = small ? 16 : 64;
  const int q_tiles = (max_q + rows / G - 1) / (rows / G);
  if (d == 128) {
    // Decode (one 16-row query tile per CTA): measured on B200 at batch 8..256, four small
    // CTAs per SM with one consumer warp each beat one CTA whose four warps split the KV axis
    // (198 us vs 309 us at batch 256, context 1400), so the KV-split form is not dispatched.
    if (kv8) return small ? launch_attn<T, true, 128, 1, 1, 3>(map, a, q_tiles, stream)
                          : launch_attn<T, true, 128, 4, 1, 4>(map, a, q_tiles, stream);
    return small ? launch_attn<T, false, 128, 1, 1, 3>(map, a, q_tiles, stream)
                 : launch_attn<T, false, 128, 4, 1, 3>(map, a, q_tiles, stream);
  }
  if (d == 64 && !kv8)
    return small ? launch_attn<T, false, 64, 1, 1, 3>(map, a, q_tiles, stream)
                 : launch_attn<T, false, 64, 4, 1, 4>(map, a, q_tiles, stream);
  if (d == 256 && !kv8)   // Qwen3.5-style 256-wide heads: two stages of 64 tokens fit beside the 4 query warps
    return small ? launch_attn<T, false, 256, 1, 1, 2>(map, a, q_tiles, stream)
                 : launch_attn<T, false, 256, 4, 1, 2>(map, a, q_tiles, stream);
  msgl_set_error_text("attention: unsupported head_dim / KV dtype combination");
  return MSGL_BAD_ARG;
}

}  // namespace

// Tensor map over the whole pool buffer [2*L, pages, Hk, page, D]; `out_map` receives 128 bytes.
MSGL_API int msgl_attn_make_kv_map(void* out_map, const void* pool, int elem_bytes, int head_dim, int page_size,
                                   int hk, long long pages_total, int planes_2l) {
  msgl_encode_tiled_fn enc = msgl_get_encode_tiled();
  if (enc == nullptr) return MSGL_CUDA_ERROR;
  if (page_size < 8 || TK % page_size || (head_dim * elem_bytes) % 128) {
    msgl_set_error_text("attention: page_size must be 8, 16, 32 or 64 and a KV row a multiple of 128 bytes");
    return MSGL_BAD_ARG;
  }
  cuuint64_t dims[5] = {(cuuint64_t)head_dim, (cuuint64_t)page_size, (cuuint64_t)hk, (cuuint64_t)pages_total,
                        (cuuint64_t)planes_2l};
  cuuint64_t row = (cuuint64_t)head_dim * elem_bytes;
  cuuint64_t strides[4] = {row, row * page_size, row * page_size * hk, row * page_size * hk * pages_total};
  cuuint32_t box[5] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)page_size, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(reinterpret_cast<CUtensorMap*>(out_map),
                   elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 5,
                   const_cast<void*>(pool), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    msgl_set_error_text(("attention: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r)).c_str());
    return MSGL_CUDA_ERROR;
  }
  return MSGL_OK;
}

// Workspace sizes (floats) for `splits` partials of `total_q` rows.
MSGL_API long long msgl_attn_workspace_floats(int total_q, int hq, int head_dim, int splits) {
  return (long long)splits * total_q * hq * (head_dim + 1);
}

MSGL_API int msgl_paged_attention(const void* kv_map, const void* q, void* out, const void* block_table,
                                  int bt_stride, const void* cu_q, const void* seq_lens, const void* k_scale,
                                  const void* v_scale, const void* mask, long long mask_stride, void* workspace,
                                  int B, int total_q, int max_q, int hq, int hk, int head_dim, int page_size,
                                  int num_pages, int layer, int num_layers, int kv_fp8, int causal, int window,
                                  int splits, float scale, int dtype, cudaStream_t stream) {
  if (B == 0 || total_q == 0) return MSGL_OK;
  if (hq % hk || 16 % (hq / hk)) {
    msgl_set_error_text("attention: the GQA group size must divide 16");
    return MSGL_BAD_ARG;
  }
  if (splits < 1) splits = 1;
  if (splits > 1 && workspace == nullptr) return MSGL_BAD_ARG;
  AttnArgs a;
  a.q = q; a.out = out;
  a.block_table = (const int32_t*)block_table; a.bt_stride = bt_stride;
  a.cu_q = (const int32_t*)cu_q; a.seq_lens = (const int32_t*)seq_lens;
  a.k_scale = (const float*)k_scale; a.v_scale = (const float*)v_scale;
  // a negative stride selects the windowed form: rows of -mask_stride floats for the last -mask_stride KV positions
  a.mask = (const float*)mask;
  a.mask_window = mask_stride < 0 ? (int)(-mask_stride) : 0;
  a.mask_stride = mask_stride < 0 ? -mask_stride : mask_stride;
  a.ws_o = (float*)workspace;
  a.ws_lse = a.ws_o != nullptr ? a.ws_o + (size_t)splits * total_q * hq * head_dim : nullptr;
  a.B = B; a.Hq = hq; a.Hk = hk; a.page_size = page_size; a.num_pages = num_pages;
  a.k_coord = layer; a.v_coord = num_layers + layer;
  a.causal = causal; a.window = window; a.splits = splits; a.total_q = total_q;
  a.scale = scale;
  int* status = nullptr;
  cudaGetSymbolAddress((void**)&status, g_attn_status);
  a.status = status;
  const CUtensorMap& map = *reinterpret_cast<const CUtensorMap*>(kv_map);
  int rc;
  if (dtype == MSGL_BF16) rc = dispatch_attn<__nv_bfloat16>(map, a, kv_fp8 != 0, head_dim, max_q, stream);
  else if (dtype == MSGL_F16) rc = dispatch_attn<__half>(map, a, kv_fp8 != 0, head_dim, max_q, stream);
  else return MSGL_BAD_ARG;
  if (rc) return rc;
  if (splits > 1) {
    const int rows_heads = total_q * hq;
    const int warps = 4;
    const int blocks = (rows_heads + warps - 1) / warps;
#define COMBINE(T, D) msgl_launch(attn_combine_kernel<T, D>, dim3(blocks), dim3(warps * 32), 0, stream, a.ws_o, a.ws_lse, (T*)out, rows_heads, splits, a.cu_q, a.B, a.Hq)
    if (dtype == MSGL_BF16) {
      if (head_dim == 128) COMBINE(__nv_bfloat16, 128);
      else if (head_dim == 256) COMBINE(__nv_bfloat16, 256);
      else COMBINE(__nv_bfloat16, 64);
    } else {
      if (head_dim == 128) COMBINE(__half, 128);
      else if (head_dim == 256) COMBINE(__half, 256);
      else COMBINE(__half, 64);
    }
#undef COMBINE
    MSGL_CHECK_LAUNCH("attn_combine");
  }
  return MSGL_OK;
}

// Test hook: route decode batches through the general (prefill/verify) kernel.
MSGL_API void msgl_attn_force_general_decode(int on) { g_force_general_decode = on != 0; }
// Tuning hook: stages of the fp8 decode kernel's TMA ring (fewer, deeper CTAs per SM as it grows).
MSGL_API void msgl_attn_decode_stages(int stages) { g_decode_stages = stages < 2 ? 2 : (stages > 4 ? 4 : stages); }

MSGL_API int msgl_attn_status(int reset) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int));
  if (reset && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_attn_status, &z, sizeof(int));
  }
  return v;
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant (see no_alloc.h): the split-KV partials live in an array that is part
// of the library image instead of a caller-provided workspace.
// ------------------------------------------------------------------------------------------
#include "no_alloc.h"

// In host code this name is only a handle for the runtime; the usable device address comes from
// cudaGetSymbolAddress below. Handing the name itself to a kernel would pass a host address.
static __device__ __align__(256) unsigned char g_attn_noalloc_ws[MSGL_ATTN_NOALLOC_WS_BYTES];

namespace {
constexpr int kNoAllocMaxDevices = 64;
void* g_noalloc_ws_addr[kNoAllocMaxDevices] = {nullptr};
}  // namespace

int msgl_paged_attention_noalloc(const void* kv_map, const void* q, void* out, const void* block_table,
                                 int bt_stride, const void* cu_q, const void* seq_lens, const void* k_scale,
                                 const void* v_scale, const void* mask, long long mask_stride, int B, int total_q,
                                 int max_q, int hq, int hk, int head_dim, int page_size, int num_pages, int layer,
                                 int num_layers, int kv_fp8, int causal, int window, int splits, float scale,
                                 int dtype, cudaStream_t stream) {
  if (splits < 1) splits = 1;
  void* ws = nullptr;
  if (splits > 1) {
    const long long need = msgl_attn_workspace_floats(total_q, hq, head_dim, splits) * (long long)sizeof(float);
    if (need > (long long)MSGL_ATTN_NOALLOC_WS_BYTES) {
      msgl_set_error_text(("paged_attention_noalloc: the split partials need " + std::to_string(need) +
                           " bytes but the built-in scratch holds " + std::to_string(MSGL_ATTN_NOALLOC_WS_BYTES) +
                           "; use fewer splits or a smaller batch")
                              .c_str());
      return MSGL_BAD_ARG;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { msgl_set_error("paged_attention_noalloc: cudaGetDevice", e); return MSGL_CUDA_ERROR; }
    if (dev < 0 || dev >= kNoAllocMaxDevices) {
      msgl_set_error_text("paged_attention_noalloc: device index out of range");
      return MSGL_BAD_ARG;
    }
    if (g_noalloc_ws_addr[dev] == nullptr) {
      // once per device, with that device current: resolve the array's address on this GPU
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_attn_noalloc_ws);
      if (e != cudaSuccess || p == nullptr) {
        msgl_set_error("paged_attention_noalloc: cudaGetSymbolAddress", e);
        return MSGL_CUDA_ERROR;
      }
      g_noalloc_ws_addr[dev] = p;
    }
    ws = g_noalloc_ws_addr[dev];
  }
  return msgl_paged_attention(kv_map, q, out, block_table, bt_stride, cu_q, seq_lens, k_scale, v_scale, mask,
                              mask_stride, ws, B, total_q, max_q, hq, hk, head_dim, page_size, num_pages, layer,
                              num_layers, kv_fp8, causal, window, splits, scale, dtype, stream);
}
