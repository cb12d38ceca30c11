// CPU expert tier: mixture-of-experts SwiGLU MLPs evaluated on the host for experts whose
// weights stay in host memory as 4-bit e2m1 codes with one scale per group of K elements
// (32 for MXFP4, 16 for NVFP4; the scale arrives as fp32, whatever its stored format was).
//
// Counterpart of the reference's libcpumoe (tools/cpu_moe/cpu_moe_so.cpp:316-476 C ABI,
// tools/cpu_moe/moe_core.hpp:44-267 kernels): same job, different shape. One work item is
// (token, expert, block of output rows); a persistent pool of threads pulls items from an
// atomic counter. Two inner products are provided and chosen at run time:
//   * fp32 activations: 16 codes are decoded with one AVX-512 table permute and multiplied in
//     fp32 (portable scalar loop when the CPU has no AVX-512);
//   * int8 activations (per-group symmetric quantisation of the token): codes are decoded to
//     int8 (value x 2) with a byte shuffle and accumulated with VNNI dot products.
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

namespace {

const float kE2M1[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
const int8_t kE2M1x2[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

class Pool {
 public:
  explicit Pool(int n) : stop_(false), epoch_(0), pending_(0) {
    if (n < 1) n = 1;
    for (int i = 0; i < n - 1; ++i) workers_.emplace_back([this] { loop(); });
  }
  ~Pool() {
    {
      std::lock_guard<std::mutex> g(m_);
      stop_ = true;
      ++epoch_;
    }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
  }
  // runs fn(i) for i in [0, n) on the pool and the calling thread; returns when all are done
  void parallel_for(int n, const std::function<void(int)>& fn) {
    if (n <= 0) return;
    {
      std::lock_guard<std::mutex> g(m_);
      fn_ = &fn;
      total_ = n;
      next_.store(0);
      pending_ = (int)workers_.size();
      ++epoch_;
    }
    cv_.notify_all();
    drain();
    std::unique_lock<std::mutex> g(m_);
    done_.wait(g, [this] { return pending_ == 0; });
    fn_ = nullptr;
  }

 private:
  void drain() {
    for (;;) {
      const int i = next_.fetch_add(1);
      if (i >= total_) break;
      (*fn_)(i);
    }
  }
  void loop() {
    uint64_t seen = 0;
    for (;;) {
      {
        std::unique_lock<std::mutex> g(m_);
        cv_.wait(g, [&] { return epoch_ != seen; });
        seen = epoch_;
        if (stop_) return;
      }
      drain();
      {
        std::lock_guard<std::mutex> g(m_);
        if (--pending_ == 0) done_.notify_one();
      }
    }
  }
  std::vector<std::thread> workers_;
  std::mutex m_;
  std::condition_variable cv_, done_;
  bool stop_;
  uint64_t epoch_;
  int pending_;
  const std::function<void(int)>* fn_ = nullptr;
  int total_ = 0;
  std::atomic<int> next_{0};
};

struct Expert {
  const uint8_t* w13 = nullptr;  // [2 * inter, hidden / 2] codes, low nibble first
  const float* s13 = nullptr;    // [2 * inter, hidden / group]
  const uint8_t* w2 = nullptr;   // [hidden, inter / 2]
  const float* s2 = nullptr;     // [hidden, inter / group]
};

struct Tier {
  int experts, hidden, inter, group;
  bool has_avx512, has_vnni;
  std::vector<Expert> e;
  Pool pool;
  Tier(int ne, int h, int i, int g, int threads) : experts(ne), hidden(h), inter(i), group(g), e(ne), pool(threads) {
#if defined(__x86_64__)
    has_avx512 = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw");
    has_vnni = has_avx512 && __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512vl");
#else
    has_avx512 = has_vnni = false;
#endif
  }
};

// ---- inner products over one weight row: sum_g scale[g] * sum_{k in g} code(k) * x[k] ----------
float dot_scalar(const uint8_t* w, const float* s, const float* x, int k, int group) {
  float acc = 0.f;
  for (int g0 = 0; g0 < k; g0 += group) {
    float part = 0.f;
    for (int j = g0; j < g0 + group; j += 2) {
      const uint8_t b = w[j >> 1];
      part += kE2M1[b & 15] * x[j] + kE2M1[b >> 4] * x[j + 1];
    }
    acc += s[g0 / group] * part;
  }
  return acc;
}

#if defined(__x86_64__)
__attribute__((target("avx512f,avx512bw"))) float dot_avx512(const uint8_t* w, const float* s, const float* x, int k,
                                                              int group) {
  const __m512 lut = _mm512_loadu_ps(kE2M1);
  __m512 acc = _mm512_setzero_ps();
  for (int g0 = 0; g0 < k; g0 += group) {
    __m512 part = _mm512_setzero_ps();
    for (int j = g0; j < g0 + group; j += 16) {
      // 8 bytes = 16 codes; interleave low / high nibbles back into element order
      const __m128i bytes = _mm_loadl_epi64(reinterpret_cast<const __m128i*>(w + (j >> 1)));
      const __m128i lo = _mm_and_si128(bytes, _mm_set1_epi8(15));
      const __m128i hi = _mm_and_si128(_mm_srli_epi16(bytes, 4), _mm_set1_epi8(15));
      const __m128i codes = _mm_unpacklo_epi8(lo, hi);
      const __m512i idx = _mm512_cvtepu8_epi32(codes);
      const __m512 wv = _mm512_permutexvar_ps(idx, lut);
      part = _mm512_fmadd_ps(wv, _mm512_loadu_ps(x + j), part);
    }
    acc = _mm512_fmadd_ps(part, _mm512_set1_ps(s[g0 / group]), acc);
  }
  return _mm512_reduce_add_ps(acc);
}

// int8 activations xq (per-group scale xs), codes decoded to int8 (value x 2)
__attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni"))) float dot_vnni(const uint8_t* w, const float* s,
                                                                         const int8_t* xq, const float* xs, int k,
                                                                         int group) {
  const __m128i lut = _mm_loadu_si128(reinterpret_cast<const __m128i*>(kE2M1x2));
  float acc = 0.f;
  for (int g0 = 0; g0 < k; g0 += group) {
    __m128i sum = _mm_setzero_si128();
    for (int j = g0; j < g0 + group; j += 16) {
      const __m128i bytes = _mm_loadl_epi64(reinterpret_cast<const __m128i*>(w + (j >> 1)));
      const __m128i lo = _mm_and_si128(bytes, _mm_set1_epi8(15));
      const __m128i hi = _mm_and_si128(_mm_srli_epi16(bytes, 4), _mm_set1_epi8(15));
      const __m128i codes = _mm_unpacklo_epi8(lo, hi);
      const __m128i wv = _mm_shuffle_epi8(lut, codes);            // signed int8 weights
      const __m128i xv = _mm_loadu_si128(reinterpret_cast<const __m128i*>(xq + j));
      // dpbusd wants unsigned x signed: |w| x (x with w's sign)
      const __m128i wa = _mm_abs_epi8(wv);
      const __m128i xsg = _mm_sign_epi8(xv, wv);
      sum = _mm_dpbusd_epi32(sum, wa, xsg);
    }
    int32_t t[4];
    _mm_storeu_si128(reinterpret_cast<__m128i*>(t), sum);
    acc += s[g0 / group] * xs[g0 / group] * 0.5f * (float)(t[0] + t[1] + t[2] + t[3]);
  }
  return acc;
}
#endif

inline float silu(float v) { return v / (1.f + std::exp(-v)); }

// per-group symmetric int8 quantisation of one activation vector
void quant_groups(const float* x, int k, int group, int8_t* q, float* scale) {
  for (int g0 = 0; g0 < k; g0 += group) {
    float amax = 0.f;
    for (int j = g0; j < g0 + group; ++j) amax = std::fmax(amax, std::fabs(x[j]));
    const float sc = amax > 0.f ? amax / 127.f : 1.f;
    scale[g0 / group] = sc;
    const float inv = 1.f / sc;
    for (int j = g0; j < g0 + group; ++j) q[j] = (int8_t)std::lrint(x[j] * inv);
  }
}

}  // namespace

#define MSGL_HOST_API __attribute__((visibility("default")))

extern "C" {

MSGL_HOST_API void* msgl_cpumoe_create(int experts, int hidden, int inter, int group, int threads) {
  if (experts <= 0 || hidden <= 0 || inter <= 0 || (group != 16 && group != 32) || hidden % group || inter % group)
    return nullptr;
  if (threads <= 0) threads = (int)std::thread::hardware_concurrency();
  return new Tier(experts, hidden, inter, group, threads);
}

MSGL_HOST_API void msgl_cpumoe_destroy(void* h) { delete static_cast<Tier*>(h); }

// The tier keeps the pointers: the arrays (pinned host memory in the engine) must outlive it.
MSGL_HOST_API int msgl_cpumoe_set_expert(void* h, int expert, const void* w13, const void* s13, const void* w2, const void* s2) {
  Tier* t = static_cast<Tier*>(h);
  if (t == nullptr || expert < 0 || expert >= t->experts) return 1;
  Expert& e = t->e[expert];
  e.w13 = static_cast<const uint8_t*>(w13);
  e.s13 = static_cast<const float*>(s13);
  e.w2 = static_cast<const uint8_t*>(w2);
  e.s2 = static_cast<const float*>(s2);
  return 0;
}

// which inner product the tier uses on this machine: 0 scalar, 1 AVX-512 fp32, 2 AVX-512 VNNI int8
MSGL_HOST_API int msgl_cpumoe_isa(void* h, int int8_act) {
  Tier* t = static_cast<Tier*>(h);
  if (int8_act && t->has_vnni && t->group % 16 == 0) return 2;
  return t->has_avx512 ? 1 : 0;
}

// out[tok] = sum_j weight[tok, j] * MLP_{ids[tok, j]}(x[tok]); experts with no weights set
// (negative id, or not resident on the host) are skipped. int8_act selects the VNNI path.
MSGL_HOST_API int msgl_cpumoe_forward(void* h, const float* x, const int32_t* ids, const float* weights, float* out, int tokens,
                        int top_k, int int8_act) {
  Tier* t = static_cast<Tier*>(h);
  if (t == nullptr || tokens < 0 || top_k <= 0) return 1;
  const int H = t->hidden, I = t->inter, G = t->group;
  const int isa = msgl_cpumoe_isa(h, int8_act);
  const int pairs = tokens * top_k;
  std::vector<float> act((size_t)pairs * I);
  std::vector<int8_t> xq, aq;
  std::vector<float> xs, as;
  if (isa == 2) {
    xq.resize((size_t)tokens * H);
    xs.resize((size_t)tokens * (H / G));
    for (int tok = 0; tok < tokens; ++tok) quant_groups(x + (size_t)tok * H, H, G, &xq[(size_t)tok * H], &xs[(size_t)tok * (H / G)]);
    aq.resize((size_t)pairs * I);
    as.resize((size_t)pairs * (I / G));
  }
  auto row_dot = [&](const uint8_t* w, const float* s, const float* xf, const int8_t* xi, const float* xsc, int k) {
#if defined(__x86_64__)
    if (isa == 2) return dot_vnni(w, s, xi, xsc, k, G);
    if (isa == 1) return dot_avx512(w, s, xf, k, G);
#endif
    (void)xi; (void)xsc;
    return dot_scalar(w, s, xf, k, G);
  };
  // stage 1: act[pair, i] = silu(w1[i] . x) * (w3[i] . x), blocks of 64 rows per work item
  const int rb1 = 64, nb1 = (I + rb1 - 1) / rb1;
  t->pool.parallel_for(pairs * nb1, [&](int item) {
    const int pair = item / nb1, blk = item % nb1;
    const int tok = pair / top_k, ex = ids[pair];
    float* a = &act[(size_t)pair * I];
    const int r0 = blk * rb1, r1 = std::min(I, r0 + rb1);
    if (ex < 0 || ex >= t->experts || t->e[ex].w13 == nullptr) {
      for (int r = r0; r < r1; ++r) a[r] = 0.f;
      return;
    }
    const Expert& e = t->e[ex];
    const float* xf = x + (size_t)tok * H;
    const int8_t* xi = isa == 2 ? &xq[(size_t)tok * H] : nullptr;
    const float* xsc = isa == 2 ? &xs[(size_t)tok * (H / G)] : nullptr;
    for (int r = r0; r < r1; ++r) {
      const float g = row_dot(e.w13 + (size_t)r * (H / 2), e.s13 + (size_t)r * (H / G), xf, xi, xsc, H);
      const float u = row_dot(e.w13 + (size_t)(I + r) * (H / 2), e.s13 + (size_t)(I + r) * (H / G), xf, xi, xsc, H);
      a[r] = silu(g) * u;
    }
  });
  if (isa == 2)
    for (int p = 0; p < pairs; ++p) quant_groups(&act[(size_t)p * I], I, G, &aq[(size_t)p * I], &as[(size_t)p * (I / G)]);
  // stage 2: out[tok, r] = sum_j weight * (w2[r] . act[pair]); one item owns its output rows
  const int rb2 = 64, nb2 = (H + rb2 - 1) / rb2;
  t->pool.parallel_for(tokens * nb2, [&](int item) {
    const int tok = item / nb2, blk = item % nb2;
    const int r0 = blk * rb2, r1 = std::min(H, r0 + rb2);
    float* o = out + (size_t)tok * H;
    for (int r = r0; r < r1; ++r) o[r] = 0.f;
    for (int j = 0; j < top_k; ++j) {
      const int pair = tok * top_k + j, ex = ids[pair];
      if (ex < 0 || ex >= t->experts || t->e[ex].w2 == nullptr) continue;
      const Expert& e = t->e[ex];
      const float wgt = weights[pair];
      const float* af = &act[(size_t)pair * I];
      const int8_t* ai = isa == 2 ? &aq[(size_t)pair * I] : nullptr;
      const float* asc = isa == 2 ? &as[(size_t)pair * (I / G)] : nullptr;
      for (int r = r0; r < r1; ++r)
        o[r] += wgt * row_dot(e.w2 + (size_t)r * (I / 2), e.s2 + (size_t)r * (I / G), af, ai, asc, I);
    }
  });
  return 0;
}

}  // extern "C"
