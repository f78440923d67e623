// Prefix-cache index: a radix tree whose edges are whole KV blocks of token ids, one tree per namespace (adapter /
// tenant).  Nodes hold one pool reference on their block; lookups pin the path so that eviction (least recently used
// unpinned leaf first) cannot take blocks out from under a running request.
// Reference behaviour: crates/spark-runtime/src/radix_tree.rs (+ inner/{evict,lru_index}.rs), prefix_cache.rs.
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <unordered_map>
#include <vector>

#include "runtime_api.h"

namespace {

struct Node {
  std::vector<int32_t> key;
  int block = -1;
  Node* parent = nullptr;
  std::map<std::vector<int32_t>, Node*> children;
  uint64_t last_access = 0;
  int pins = 0;
};

}  // namespace

struct atlas_radix {
  atlas_pool* pool;
  int bs;
  std::unordered_map<uint64_t, Node*> roots;
  uint64_t clock = 0;
  int num_nodes = 0;
  std::mutex mu;

  Node* root(uint64_t ns) {
    auto it = roots.find(ns);
    if (it != roots.end()) return it->second;
    Node* r = new Node();
    roots[ns] = r;
    return r;
  }
  static void destroy(Node* n) {
    for (auto& kv : n->children) destroy(kv.second);
    delete n;
  }
  void collect_leaves(Node* n, std::vector<Node*>& out) {
    for (auto& kv : n->children) collect_leaves(kv.second, out);
    if (n->parent && n->children.empty() && n->pins == 0) out.push_back(n);
  }
};

extern "C" {

atlas_radix* atlas_radix_create(atlas_pool* pool) {
  if (!pool) return nullptr;
  auto* r = new atlas_radix();
  r->pool = pool;
  r->bs = atlas_pool_block_size(pool);
  return r;
}

void atlas_radix_destroy(atlas_radix* r) {
  if (!r) return;
  for (auto& kv : r->roots) atlas_radix::destroy(kv.second);
  delete r;
}

int atlas_radix_match(atlas_radix* r, uint64_t ns, const int32_t* tokens, int n, int max_tokens, int* blocks_out,
                      uint64_t* nodes_out, int cap) {
  std::lock_guard<std::mutex> g(r->mu);
  int limit = n - 1;
  if (max_tokens >= 0 && max_tokens < limit) limit = max_tokens;
  Node* node = r->root(ns);
  const uint64_t now = ++r->clock;
  int i = 0, cnt = 0;
  std::vector<int32_t> key(r->bs);
  while (i + r->bs <= limit && cnt < cap) {
    std::memcpy(key.data(), tokens + i, sizeof(int32_t) * r->bs);
    auto it = node->children.find(key);
    if (it == node->children.end()) break;
    node = it->second;
    node->last_access = now;
    blocks_out[cnt] = node->block;
    nodes_out[cnt] = reinterpret_cast<uint64_t>(node);
    ++cnt;
    i += r->bs;
  }
  if (cnt) {
    atlas_pool_inc_ref(r->pool, blocks_out, cnt);
    for (int j = 0; j < cnt; ++j) ++reinterpret_cast<Node*>(nodes_out[j])->pins;
  }
  return cnt;
}

void atlas_radix_release(atlas_radix* r, const uint64_t* nodes, int n) {
  std::lock_guard<std::mutex> g(r->mu);
  for (int i = 0; i < n; ++i) {
    Node* nd = reinterpret_cast<Node*>(nodes[i]);
    if (nd->pins > 0) --nd->pins;
  }
}

int atlas_radix_insert(atlas_radix* r, uint64_t ns, const int32_t* tokens, int n, const int* blocks, int nblocks) {
  std::lock_guard<std::mutex> g(r->mu);
  Node* node = r->root(ns);
  const uint64_t now = ++r->clock;
  int nfull = n / r->bs;
  if (nblocks < nfull) nfull = nblocks;
  int created = 0;
  std::vector<int32_t> key(r->bs);
  for (int j = 0; j < nfull; ++j) {
    std::memcpy(key.data(), tokens + (size_t)j * r->bs, sizeof(int32_t) * r->bs);
    auto it = node->children.find(key);
    Node* child;
    if (it == node->children.end()) {
      child = new Node();
      child->key = key;
      child->block = blocks[j];
      child->parent = node;
      node->children.emplace(key, child);
      atlas_pool_inc_ref(r->pool, &blocks[j], 1);
      ++r->num_nodes;
      ++created;
    } else {
      child = it->second;       // the tree keeps its own block; the caller's duplicate stays private
    }
    child->last_access = now;
    node = child;
  }
  return created;
}

int atlas_radix_evict(atlas_radix* r, int want) {
  std::lock_guard<std::mutex> g(r->mu);
  int freed = 0;
  while (freed < want) {
    std::vector<Node*> leaves;
    for (auto& kv : r->roots) r->collect_leaves(kv.second, leaves);
    if (leaves.empty()) break;
    Node* victim = leaves[0];
    for (Node* l : leaves)
      if (l->last_access < victim->last_access) victim = l;
    victim->parent->children.erase(victim->key);
    freed += atlas_pool_free(r->pool, &victim->block, 1) > 0 ? 1 : 0;
    --r->num_nodes;
    delete victim;
  }
  return freed;
}

int atlas_radix_num_nodes(const atlas_radix* r) { return r->num_nodes; }

int atlas_radix_evictable(const atlas_radix* r) {
  auto* rr = const_cast<atlas_radix*>(r);
  std::lock_guard<std::mutex> g(rr->mu);
  // a node is evictable once its whole subtree is unpinned
  struct Rec {
    static int count(Node* n, bool& clean) {
      int c = 0;
      bool all = true;
      for (auto& kv : n->children) {
        bool sub = true;
        c += count(kv.second, sub);
        all = all && sub;
      }
      clean = all && n->pins == 0;
      if (n->parent && clean) ++c;
      return c;
    }
  };
  int total = 0;
  for (auto& kv : rr->roots) {
    bool clean = true;
    total += Rec::count(kv.second, clean);
  }
  return total;
}

}  // extern "C"
