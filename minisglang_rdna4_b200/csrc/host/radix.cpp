// Host helpers of the scheduler, exported with C linkage for ctypes.
//
// msgl_common_prefix_i32: length of the common prefix of two int32 key arrays; the radix
// prefix cache calls it for every edge it walks. Same job as the reference's
// fast_compare_key (python/minisgl/kernel/csrc/src/radix.cpp:19-40), here with a word-at-a-
// time scan.
//
// msgl_pages_*: LIFO free list of KV page ids (the scheduler's page allocator).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {

__attribute__((visibility("default"))) int64_t msgl_common_prefix_i32(const int32_t* a, const int32_t* b,
                                                                      int64_t n) {
  int64_t i = 0;
  // compare eight bytes at a time while both halves match
  for (; i + 2 <= n; i += 2) {
    uint64_t x, y;
    std::memcpy(&x, a + i, 8);
    std::memcpy(&y, b + i, 8);
    if (x != y) break;
  }
  for (; i < n; ++i)
    if (a[i] != b[i]) return i;
  return n;
}

struct MsglPageList {
  std::vector<int32_t> free_pages;
  int64_t capacity;
};

__attribute__((visibility("default"))) void* msgl_pages_create(int64_t num_pages) {
  auto* l = new MsglPageList();
  l->capacity = num_pages;
  l->free_pages.resize(num_pages);
  for (int64_t i = 0; i < num_pages; ++i) l->free_pages[i] = (int32_t)(num_pages - 1 - i);
  return l;
}
__attribute__((visibility("default"))) void msgl_pages_destroy(void* h) { delete (MsglPageList*)h; }
__attribute__((visibility("default"))) int64_t msgl_pages_available(void* h) {
  return (int64_t)((MsglPageList*)h)->free_pages.size();
}
// pops n pages into out (lowest ids first on a fresh list); returns 0 or -1 when short
__attribute__((visibility("default"))) int msgl_pages_take(void* h, int64_t n, int32_t* out) {
  auto* l = (MsglPageList*)h;
  if ((int64_t)l->free_pages.size() < n) return -1;
  for (int64_t i = 0; i < n; ++i) {
    out[i] = l->free_pages.back();
    l->free_pages.pop_back();
  }
  return 0;
}
// returns -1 when the list would exceed its capacity (a page was freed twice)
__attribute__((visibility("default"))) int msgl_pages_give(void* h, const int32_t* pages, int64_t n) {
  auto* l = (MsglPageList*)h;
  if ((int64_t)l->free_pages.size() + n > l->capacity) return -1;
  l->free_pages.insert(l->free_pages.end(), pages, pages + n);
  return 0;
}

}  // extern "C"
