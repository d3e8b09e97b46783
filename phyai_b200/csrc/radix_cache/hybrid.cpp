// Recurrent-state slots (Mamba / gated delta-net layers) hung on the nodes of the KV prefix tree.
// A hybrid model can resume from a cached prefix only where a state snapshot exists, so a match
// reports, besides the KV match, the deepest node on the matched path that carries a slot.
// Reference: phyai-ext/csrc/radix_cache/mamba/hybrid_prefix_cache.h, mamba_allocator.h, mamba_slot.h.
#include <algorithm>

#include "radix_cache.h"

namespace pbc {

HybridPrefixCache::HybridPrefixCache(std::shared_ptr<PrefixCache> kv, std::int32_t slots) : kv_(std::move(kv)), total_(slots) {
  if (!kv_) throw UsageError("hybrid cache needs a KV prefix cache");
  for (std::int32_t i = slots - 1; i >= 0; --i) free_.push_back(i);
  // a node that leaves the tree gives its slot back
  kv_->on_node_removed([this](Node& n) {
    if (n.mamba >= 0) { free_.push_back(n.mamba); n.mamba = -1; }
    holders_.erase(&n);
  });
}

HybridPrefixCache::Match HybridPrefixCache::match(std::string_view atoms) {
  std::lock_guard<std::recursive_mutex> g(kv_->mutex());
  Match m;
  m.kv = kv_->match(atoms);
  const std::uint64_t h = find_last_mamba_node(m.kv.last_node[int(Tier::Device)]);
  if (h) {
    const Node& n = kv_->node_info(h);
    m.mamba_node = h; m.mamba_atoms = n.depth_atoms; m.mamba_slot = n.mamba;
  }
  return m;
}

std::int32_t HybridPrefixCache::allocate_slot() {
  std::lock_guard<std::recursive_mutex> g(kv_->mutex());
  if (free_.empty()) return -1;
  const auto s = free_.back();
  free_.pop_back();
  return s;
}
void HybridPrefixCache::free_slot(std::int32_t slot) {
  std::lock_guard<std::recursive_mutex> g(kv_->mutex());
  if (slot < 0 || slot >= total_) throw UsageError("slot index outside the pool");
  if (std::find(free_.begin(), free_.end(), slot) != free_.end()) throw UsageError("slot is already free");
  free_.push_back(slot);
}
void HybridPrefixCache::attach(std::uint64_t node, std::int32_t slot) {
  std::lock_guard<std::recursive_mutex> g(kv_->mutex());
  Node* n = kv_->checked(node);
  if (!n->parent) throw UsageError("the root cannot carry a state slot");
  if (slot < 0 || slot >= total_) throw UsageError("slot index outside the pool");
  if (n->mamba >= 0) throw UsageError("node already carries a state slot");
  n->mamba = slot;
  holders_.insert(n);
}
std::int32_t HybridPrefixCache::detach(std::uint64_t node) {
  std::lock_guard<std::recursive_mutex> g(kv_->mutex());
  Node* n = kv_->checked(node);
  const auto s = n->mamba;
  n->mamba = -1;
  holders_.erase(n);
  return s;
}
std::uint64_t HybridPrefixCache::find_last_mamba_node(std::uint64_t from) const {
  std::lock_guard<std::recursive_mutex> g(kv_->mutex());
  for (const Node* n = kv_->checked(from); n && n->parent; n = n->parent)
    if (n->mamba >= 0) return std::uint64_t(reinterpret_cast<std::uintptr_t>(n));
  return 0;
}
bool HybridPrefixCache::ensure_slots_by_evict(std::int32_t need) {
  std::lock_guard<std::recursive_mutex> g(kv_->mutex());
  while (std::int32_t(free_.size()) < need) {
    Node* best = nullptr;
    for (Node* n : holders_) {
      bool pinned = false;
      for (int t = 0; t < kTiers; ++t) pinned = pinned || n->pins[t] > 0;
      if (!pinned && (!best || n->last_ns < best->last_ns)) best = n;
    }
    if (!best) return false;
    free_.push_back(best->mamba);   // the KV stays cached; only the state snapshot goes
    best->mamba = -1;
    holders_.erase(best);
  }
  return true;
}

}  // namespace pbc
