// Device side of a speculative decode step: acceptance, EOS / length truncation, commit of the
// emitted tokens to the token pool, the draft-vocabulary map, and KV compaction after tree
// verification. Replaces the reference's torch-op acceptance (python/minisgl/spec/accept_gpu.py:
// 110-330) and keeps the host out of the step until one small record is copied back.
//
// Layout of a verify step with a fixed width W = 1 + K rows per request: request b feeds the
// tokens at positions c_b .. c_b + K (its last committed token followed by K draft tokens that sit
// in the token pool behind it); target[b * W + j] is the target model's arg-max after row j, i.e.
// its token for position c_b + j + 1. Draft j (position c_b + 1 + j) stands while
// target[b * W + j] equals it and all earlier drafts stood.
#include "common.cuh"

using namespace msgl;

namespace {

constexpr int kMaxEos = 8;

struct AcceptArgs {
  const int32_t* target;     // [B * W] arg-max ids of the verify rows
  int32_t* token_pool;       // [slots * max_seq_len]
  const int32_t* first_idx;  // [B] flat pool index of the first draft token (slot * msl + c_b + 1)
  const int32_t* num_draft;  // [B] drafts offered, 0 .. W - 1
  const int32_t* max_emit;   // [B] tokens the request may still emit (>= 1)
  const int32_t* flags;      // [B] bit 0: ignore EOS
  int32_t* record;           // [B * (W + 2)]: n, hit_eos, emitted[W]
  int32_t* sel_row;          // [B] row of the last emitted token's predecessor: b * W + n - 1
  int32_t eos[kMaxEos];
  int n_eos;
  int B, W;
};

// one thread per request (B is at most a few hundred; the work per request is W <= 17 steps)
__global__ void spec_accept_kernel(AcceptArgs a) {
  pdl_enter();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= a.B) return;
  const int W = a.W;
  const int32_t* tgt = a.target + (size_t)b * W;
  int32_t* pool = a.token_pool + a.first_idx[b];
  const int k = min(max(a.num_draft[b], 0), W - 1);
  int n = 1;
  while (n <= k && tgt[n - 1] == pool[n - 1]) ++n;   // draft j-1 stands: row j's prediction counts too
  n = min(n, max(a.max_emit[b], 1));
  int hit = 0;
  if (!(a.flags[b] & 1)) {
    for (int j = 0; j < n && !hit; ++j)
      for (int e = 0; e < a.n_eos; ++e)
        if (tgt[j] == a.eos[e]) { n = j + 1; hit = 1; break; }
  }
  int32_t* rec = a.record + (size_t)b * (W + 2);
  rec[0] = n;
  rec[1] = hit;
  for (int j = 0; j < W; ++j) rec[2 + j] = j < n ? tgt[j] : -1;
  for (int j = 0; j < n; ++j) pool[j] = tgt[j];       // commit: positions c_b + 1 .. c_b + n
  a.sel_row[b] = b * W + n - 1;
}

// Acceptance over a draft tree with a fixed shape: a best chain of K nodes (verify rows 1 .. K, K/V
// already at their sequence positions) and W - 1 sibling candidates per depth (rows K + 1 ..., K/V at
// scratch slots behind the chain). The target's prediction is followed from the root: at depth d
// it either equals the chain's draft (continue), equals a sibling (accept it, emit that sibling
// row's own prediction as the bonus token, stop: siblings have no children), or neither (stop).
struct TreeArgs {
  const int32_t* target;     // [B * R] arg-max ids of the verify rows, R = 1 + K * W
  int32_t* token_pool;
  const int32_t* first_idx;  // [B] flat pool index of position c + 1 (the chain drafts sit there)
  const int32_t* num_draft;  // [B] depth offered, 0 .. K
  const int32_t* max_emit;
  const int32_t* flags;
  const int32_t* sib_tok;    // [K][sib_stride][W - 1] sibling candidates (target vocabulary)
  const int32_t* out_loc;    // [B * R] K/V token slot of every verify row
  int32_t* record;           // [B * (K + 3)]: n, hit_eos, emitted[K + 1]
  int32_t* sel_row;          // [B] row of the draft-update batch that holds the next chain state
  int32_t* feat_row;         // [B * (K + 1)] verify row whose features feed update row j
  int32_t* moves;            // [B * 2] (src slot, dst slot) of an accepted sibling's K/V, or -1
  int32_t eos[kMaxEos];
  int n_eos;
  int B, K, W, sib_stride;
};

__global__ void spec_accept_tree_kernel(TreeArgs a) {
  pdl_enter();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= a.B) return;
  const int K = a.K, W = a.W, R = 1 + K * W;
  const int32_t* tgt = a.target + (size_t)b * R;
  int32_t* pool = a.token_pool + a.first_idx[b];
  const int k = min(max(a.num_draft[b], 0), K);
  const int limit = max(a.max_emit[b], 1);
  const bool stop_at_eos = !(a.flags[b] & 1);
  int32_t* rec = a.record + (size_t)b * (K + 3);
  int32_t* frow = a.feat_row + (size_t)b * (K + 1);
  for (int j = 0; j <= K; ++j) frow[j] = b * R + j;
  int n = 0, hit = 0, cur = 0, mv_src = -1, mv_dst = -1;
  auto is_eos = [&](int t) {
    for (int e = 0; e < a.n_eos; ++e)
      if (t == a.eos[e]) return true;
    return false;
  };
  for (int d = 1; d <= K + 1; ++d) {
    const int p = tgt[cur];                       // the token at position c + d
    rec[2 + n] = p;
    ++n;
    if (stop_at_eos && is_eos(p)) { hit = 1; break; }
    if (n >= limit || d > k) break;
    if (pool[d - 1] == p) { cur = d; continue; }  // the chain's draft stands
    int found = -1;
    const int32_t* sib = a.sib_tok + ((size_t)(d - 1) * a.sib_stride + b) * (W - 1);
    for (int s = 0; s < W - 1; ++s)
      if (sib[s] == p) { found = s; break; }
    if (found < 0) break;
    const int row = K + (d - 1) * (W - 1) + found + 1;
    mv_src = a.out_loc[(size_t)b * R + row];
    mv_dst = a.out_loc[(size_t)b * R + d];
    frow[d] = b * R + row;
    const int p2 = tgt[row];                      // bonus: the accepted sibling's own prediction
    rec[2 + n] = p2;
    ++n;
    if (stop_at_eos && is_eos(p2)) hit = 1;
    break;
  }
  rec[0] = n;
  rec[1] = hit;
  for (int j = n; j <= K; ++j) rec[2 + j] = -1;
  for (int j = 0; j < n; ++j) pool[j] = rec[2 + j];   // commit: positions c + 1 .. c + n
  a.sel_row[b] = b * (K + 1) + n - 1;
  a.moves[2 * b] = mv_src;
  a.moves[2 * b + 1] = mv_dst;
}

// token_pool[dst_idx[i]] = ids[i] + d2t[ids[i]]   (draft vocabulary -> target vocabulary)
__global__ void spec_write_draft_kernel(const int32_t* __restrict__ ids, const int64_t* __restrict__ d2t,
                                        const int32_t* __restrict__ dst_idx, int32_t* __restrict__ token_pool,
                                        int32_t* __restrict__ out_ids, int n, int draft_vocab) {
  pdl_enter();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int id = ids[i];
  (void)MSGL_OOB(id, draft_vocab);
  id = id < 0 ? 0 : (id >= draft_vocab ? draft_vocab - 1 : id);
  const int t = id + (int)d2t[id];
  if (dst_idx[i] >= 0) token_pool[dst_idx[i]] = t;
  if (out_ids != nullptr) out_ids[i] = t;
}

// Tree verification leaves the K / V of an accepted node at the slot of its node index; the
// committed sequence wants it at the slot of its depth. moves [n][2] = (src slot, dst slot) token
// slots of one pool buffer [2][layers][slots][hk][ps][d] laid out page-major: slot = page * ps + off.
// grid = (moves, 2 * layers), block = 128; element bytes esz.
__global__ void spec_kv_compact_kernel(uint8_t* __restrict__ pool, const int32_t* __restrict__ moves, int n_moves,
                                       long long plane_bytes, int hk, int ps, int row_bytes) {
  pdl_enter();
  const int m = blockIdx.x;
  if (m >= n_moves) return;
  const int src = moves[2 * m], dst = moves[2 * m + 1];
  if (src < 0 || dst < 0 || src == dst) return;
  uint8_t* plane = pool + (size_t)blockIdx.y * plane_bytes;   // one (k|v, layer) plane: [pages][hk][ps][d]
  const size_t page_bytes = (size_t)hk * ps * row_bytes;
  for (int h = 0; h < hk; ++h) {
    const uint8_t* s = plane + (size_t)(src / ps) * page_bytes + ((size_t)h * ps + src % ps) * row_bytes;
    uint8_t* d = plane + (size_t)(dst / ps) * page_bytes + ((size_t)h * ps + dst % ps) * row_bytes;
    for (int i = threadIdx.x * 16; i < row_bytes; i += blockDim.x * 16)
      *reinterpret_cast<uint4*>(d + i) = *reinterpret_cast<const uint4*>(s + i);
  }
}

}  // namespace

MSGL_API int msgl_spec_accept(const void* target, void* token_pool, const void* first_idx, const void* num_draft,
                              const void* max_emit, const void* flags, void* record, void* sel_row,
                              const int* eos_ids, int n_eos, int B, int W, cudaStream_t stream) {
  if (B <= 0 || W < 1 || W > 64 || n_eos < 0 || n_eos > kMaxEos) return MSGL_BAD_ARG;
  AcceptArgs a;
  a.target = (const int32_t*)target;
  a.token_pool = (int32_t*)token_pool;
  a.first_idx = (const int32_t*)first_idx;
  a.num_draft = (const int32_t*)num_draft;
  a.max_emit = (const int32_t*)max_emit;
  a.flags = (const int32_t*)flags;
  a.record = (int32_t*)record;
  a.sel_row = (int32_t*)sel_row;
  for (int i = 0; i < kMaxEos; ++i) a.eos[i] = i < n_eos ? eos_ids[i] : -1;
  a.n_eos = n_eos;
  a.B = B;
  a.W = W;
  msgl_launch(spec_accept_kernel, dim3((B + 63) / 64), dim3(64), 0, stream, a);
  MSGL_CHECK_LAUNCH("spec_accept");
  return MSGL_OK;
}

MSGL_API int msgl_spec_accept_tree(const void* target, void* token_pool, const void* first_idx, const void* num_draft,
                                   const void* max_emit, const void* flags, const void* sib_tok, const void* out_loc,
                                   void* record, void* sel_row, void* feat_row, void* moves, const int* eos_ids,
                                   int n_eos, int B, int K, int W, int sib_stride, cudaStream_t stream) {
  if (B <= 0 || K < 1 || K > 16 || W < 2 || W > 16 || n_eos < 0 || n_eos > kMaxEos || sib_stride < B) return MSGL_BAD_ARG;
  TreeArgs a;
  a.target = (const int32_t*)target;
  a.token_pool = (int32_t*)token_pool;
  a.first_idx = (const int32_t*)first_idx;
  a.num_draft = (const int32_t*)num_draft;
  a.max_emit = (const int32_t*)max_emit;
  a.flags = (const int32_t*)flags;
  a.sib_tok = (const int32_t*)sib_tok;
  a.out_loc = (const int32_t*)out_loc;
  a.record = (int32_t*)record;
  a.sel_row = (int32_t*)sel_row;
  a.feat_row = (int32_t*)feat_row;
  a.moves = (int32_t*)moves;
  for (int i = 0; i < kMaxEos; ++i) a.eos[i] = i < n_eos ? eos_ids[i] : -1;
  a.n_eos = n_eos;
  a.B = B; a.K = K; a.W = W; a.sib_stride = sib_stride;
  msgl_launch(spec_accept_tree_kernel, dim3((B + 63) / 64), dim3(64), 0, stream, a);
  MSGL_CHECK_LAUNCH("spec_accept_tree");
  return MSGL_OK;
}

MSGL_API int msgl_spec_write_draft(const void* ids, const void* d2t, const void* dst_idx, void* token_pool,
                                   void* out_ids, int n, int draft_vocab, cudaStream_t stream) {
  if (n <= 0) return n == 0 ? MSGL_OK : MSGL_BAD_ARG;
  msgl_launch(spec_write_draft_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, (const int32_t*)ids,
              (const int64_t*)d2t, (const int32_t*)dst_idx, (int32_t*)token_pool, (int32_t*)out_ids, n, draft_vocab);
  MSGL_CHECK_LAUNCH("spec_write_draft");
  return MSGL_OK;
}

MSGL_API int msgl_spec_kv_compact(void* pool, const void* moves, int n_moves, long long plane_bytes, int planes, int hk,
                                  int ps, int row_bytes, cudaStream_t stream) {
  if (n_moves <= 0) return n_moves == 0 ? MSGL_OK : MSGL_BAD_ARG;
  if (row_bytes % 16) return MSGL_BAD_ARG;
  msgl_launch(spec_kv_compact_kernel, dim3(n_moves, planes), dim3(128), 0, stream, (uint8_t*)pool,
              (const int32_t*)moves, n_moves, plane_bytes, hk, ps, row_bytes);
  MSGL_CHECK_LAUNCH("spec_kv_compact");
  return MSGL_OK;
}
