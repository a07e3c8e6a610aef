// liboxbrt: host-side runtime pieces of oxidize_b200 in C++ (plain C ABI, loaded with ctypes).
//
//  * KV block pool: free list, per-block reference counts, prefix cache keyed by a running
//    FNV-1a hash of the whole prefix up to the block end, LRU eviction of cached blocks that
//    nobody references.  Semantics (and block-id order) match engine/kv_pool.py::BlockPool, which
//    stays as the executable specification; the reference's counterpart is
//    oxidize-core/src/paged_attention/block_pool.rs + scheduler/prefix_cache.rs.
//
// Nothing here touches the GPU.
#include <cstdint>
#include <cstring>
#include <unordered_map>
#include <vector>

#define OXBRT_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr uint64_t FNV_OFFSET = 0xCBF29CE484222325ull;
constexpr uint64_t FNV_PRIME = 0x100000001B3ull;

inline uint64_t hash_tokens(const int32_t* t, int64_t n, uint64_t h) {
  for (int64_t i = 0; i < n; ++i) {
    h *= FNV_PRIME;
    h ^= (uint64_t)(int64_t)t[i];
  }
  return h;
}

struct Pool {
  int num_blocks, page;
  bool prefix;
  std::vector<int32_t> ref;
  std::vector<uint64_t> hash_of;
  std::vector<uint8_t> has_hash;
  std::vector<int32_t> free_list;  // back() is handed out next
  std::unordered_map<uint64_t, int32_t> cache;
  // LRU of cached blocks with ref == 0: intrusive doubly linked list, head = oldest
  std::vector<int32_t> prev, next;
  std::vector<uint8_t> in_lru;
  int32_t head = -1, tail = -1, lru_count = 0;
  int64_t hits = 0, misses = 0;

  void lru_push(int32_t b) {
    prev[b] = tail;
    next[b] = -1;
    if (tail >= 0) next[tail] = b;
    tail = b;
    if (head < 0) head = b;
    in_lru[b] = 1;
    ++lru_count;
  }
  void lru_remove(int32_t b) {
    if (!in_lru[b]) return;
    if (prev[b] >= 0) next[prev[b]] = next[b]; else head = next[b];
    if (next[b] >= 0) prev[next[b]] = prev[b]; else tail = prev[b];
    in_lru[b] = 0;
    --lru_count;
  }
  int32_t allocate() {
    int32_t b;
    if (!free_list.empty()) {
      b = free_list.back();
      free_list.pop_back();
    } else if (head >= 0) {
      b = head;
      lru_remove(b);
      if (has_hash[b]) {
        auto it = cache.find(hash_of[b]);
        if (it != cache.end() && it->second == b) cache.erase(it);
      }
      has_hash[b] = 0;
    } else {
      return -1;
    }
    ref[b] = 1;
    return b;
  }
  void incref(int32_t b) {
    if (ref[b] == 0) lru_remove(b);
    ++ref[b];
  }
  int release(int32_t b) {
    if (ref[b] <= 0) return -1;
    if (--ref[b] == 0) {
      bool cached = false;
      if (has_hash[b]) {
        auto it = cache.find(hash_of[b]);
        cached = it != cache.end() && it->second == b;
      }
      if (cached) {
        lru_push(b);
      } else {
        has_hash[b] = 0;
        free_list.push_back(b);
      }
    }
    return 0;
  }
  int32_t lookup(uint64_t h) {
    if (!prefix) return -1;
    auto it = cache.find(h);
    if (it == cache.end()) {
      ++misses;
      return -1;
    }
    ++hits;
    incref(it->second);
    return it->second;
  }
  void publish(int32_t b, uint64_t h) {
    if (!prefix || cache.count(h)) return;
    cache[h] = b;
    hash_of[b] = h;
    has_hash[b] = 1;
  }
};

}  // namespace

OXBRT_API int oxbrt_version() { return 1; }

OXBRT_API uint64_t oxbrt_block_hash(const int32_t* tokens, int64_t n, uint64_t h) { return hash_tokens(tokens, n, h); }

OXBRT_API void* oxbrt_pool_create(int num_blocks, int page_size, int enable_prefix_cache) {
  if (num_blocks <= 0 || page_size <= 0) return nullptr;
  Pool* p = new Pool();
  p->num_blocks = num_blocks;
  p->page = page_size;
  p->prefix = enable_prefix_cache != 0;
  p->ref.assign(num_blocks, 0);
  p->hash_of.assign(num_blocks, 0);
  p->has_hash.assign(num_blocks, 0);
  p->prev.assign(num_blocks, -1);
  p->next.assign(num_blocks, -1);
  p->in_lru.assign(num_blocks, 0);
  p->free_list.resize(num_blocks);
  for (int i = 0; i < num_blocks; ++i) p->free_list[i] = num_blocks - 1 - i;  // hands out 0, 1, 2, ...
  return p;
}
OXBRT_API void oxbrt_pool_destroy(void* h) { delete static_cast<Pool*>(h); }
OXBRT_API int oxbrt_pool_allocate(void* h) { return static_cast<Pool*>(h)->allocate(); }
OXBRT_API void oxbrt_pool_incref(void* h, int b) { static_cast<Pool*>(h)->incref(b); }
OXBRT_API int oxbrt_pool_release(void* h, int b) { return static_cast<Pool*>(h)->release(b); }
OXBRT_API int oxbrt_pool_lookup(void* h, uint64_t hash) { return static_cast<Pool*>(h)->lookup(hash); }
OXBRT_API void oxbrt_pool_publish(void* h, int b, uint64_t hash) { static_cast<Pool*>(h)->publish(b, hash); }
OXBRT_API int oxbrt_pool_ref(void* h, int b) { return static_cast<Pool*>(h)->ref[b]; }
OXBRT_API int oxbrt_pool_num_free(void* h) {
  Pool* p = static_cast<Pool*>(h);
  return (int)p->free_list.size() + p->lru_count;
}
// out: [free list length, evictable cached blocks, cache entries, hits, misses]
OXBRT_API void oxbrt_pool_stats(void* h, int64_t* out) {
  Pool* p = static_cast<Pool*>(h);
  out[0] = (int64_t)p->free_list.size();
  out[1] = p->lru_count;
  out[2] = (int64_t)p->cache.size();
  out[3] = p->hits;
  out[4] = p->misses;
}
// hash of the block published under `b`, or 0 with *has = 0
OXBRT_API uint64_t oxbrt_pool_hash_of(void* h, int b, int* has) {
  Pool* p = static_cast<Pool*>(h);
  *has = p->has_hash[b];
  return p->has_hash[b] ? p->hash_of[b] : 0;
}
// Longest run of cached full blocks covering a prefix of `tokens` (the last token is never served from
// the cache).  Takes a reference on every returned block; returns how many were written to out_blocks.
OXBRT_API int oxbrt_pool_match_prefix(void* h, const int32_t* tokens, int64_t n_tokens, int32_t* out_blocks, int max_out) {
  Pool* p = static_cast<Pool*>(h);
  if (!p->prefix || n_tokens <= 0) return 0;
  const int64_t n_full = (n_tokens - 1) / p->page;
  uint64_t hh = FNV_OFFSET;
  int n = 0;
  for (int64_t i = 0; i < n_full && n < max_out; ++i) {
    hh = hash_tokens(tokens + i * p->page, p->page, hh);
    const int32_t b = p->lookup(hh);
    if (b < 0) break;
    out_blocks[n++] = b;
  }
  return n;
}
