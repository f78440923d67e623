// Paged-KV block pool: FIFO free list + per-block reference counts (a block is shared between a running sequence and
// the prefix cache by reference).  Reference behaviour: crates/spark-runtime/src/kv_cache/paged_impl.rs
// (free_blocks + block_ref_counts: alloc -> 1, inc_ref for sharing, back to the free list at 0).
#include <deque>
#include <mutex>
#include <vector>

#include "runtime_api.h"

struct atlas_pool {
  int num_blocks, block_size;
  std::deque<int> free_list;
  std::vector<int> ref;
  mutable std::mutex mu;
};

extern "C" {

atlas_pool* atlas_pool_create(int num_blocks, int block_size) {
  if (num_blocks < 0 || block_size <= 0) return nullptr;
  auto* p = new atlas_pool();
  p->num_blocks = num_blocks;
  p->block_size = block_size;
  p->ref.assign(num_blocks, 0);
  for (int i = 0; i < num_blocks; ++i) p->free_list.push_back(i);
  return p;
}

void atlas_pool_destroy(atlas_pool* p) { delete p; }

int atlas_pool_num_free(const atlas_pool* p) {
  std::lock_guard<std::mutex> g(p->mu);
  return (int)p->free_list.size();
}

int atlas_pool_ref_count(const atlas_pool* p, int block) {
  std::lock_guard<std::mutex> g(p->mu);
  return (block < 0 || block >= p->num_blocks) ? -1 : p->ref[block];
}

int atlas_pool_alloc(atlas_pool* p, int n, int* out) {
  std::lock_guard<std::mutex> g(p->mu);
  if (n < 0 || (size_t)n > p->free_list.size()) return -1;
  for (int i = 0; i < n; ++i) {
    out[i] = p->free_list.front();
    p->free_list.pop_front();
    p->ref[out[i]] = 1;
  }
  return 0;
}

int atlas_pool_inc_ref(atlas_pool* p, const int* blocks, int n) {
  std::lock_guard<std::mutex> g(p->mu);
  for (int i = 0; i < n; ++i)
    if (blocks[i] < 0 || blocks[i] >= p->num_blocks || p->ref[blocks[i]] <= 0) return -2;
  for (int i = 0; i < n; ++i) ++p->ref[blocks[i]];
  return 0;
}

int atlas_pool_free(atlas_pool* p, const int* blocks, int n) {
  std::lock_guard<std::mutex> g(p->mu);
  int released = 0;
  for (int i = 0; i < n; ++i) {
    const int b = blocks[i];
    if (b < 0 || b >= p->num_blocks || p->ref[b] <= 0) return -2;
    if (--p->ref[b] == 0) {
      p->free_list.push_back(b);
      ++released;
    }
  }
  return released;
}

int atlas_pool_check(const atlas_pool* p) {
  std::lock_guard<std::mutex> g(p->mu);
  std::vector<char> in_free(p->num_blocks, 0);
  for (int b : p->free_list) {
    if (b < 0 || b >= p->num_blocks || in_free[b]) return -1;
    in_free[b] = 1;
  }
  for (int b = 0; b < p->num_blocks; ++b)
    if ((p->ref[b] == 0) != (in_free[b] != 0)) return -2;
  return 0;
}

}  // extern "C"

extern "C" int atlas_pool_block_size(const atlas_pool* p) { return p->block_size; }
