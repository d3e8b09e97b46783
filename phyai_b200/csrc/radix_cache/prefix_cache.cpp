// Radix tree, tier allocators, eviction and two-phase tier moves (see radix_cache.h).
#include <algorithm>
#include <cstring>

#include "radix_cache.h"

namespace pbc {

std::uint64_t hash_bytes(const void* data, std::size_t n, std::uint64_t seed) {
  const auto* p = static_cast<const unsigned char*>(data);
  std::uint64_t h = seed ^ (0x9e3779b97f4a7c15ull + n * 0xbf58476d1ce4e5b9ull);
  auto mix = [](std::uint64_t x) {
    x ^= x >> 32; x *= 0xd6e8feb86659fd93ull; x ^= x >> 32; x *= 0xd6e8feb86659fd93ull; x ^= x >> 32;
    return x;
  };
  while (n >= 8) {
    std::uint64_t w;
    std::memcpy(&w, p, 8);
    h = mix(h ^ w) + 0x94d049bb133111ebull;
    p += 8; n -= 8;
  }
  std::uint64_t tail = 0;
  std::memcpy(&tail, p, n);
  return mix(h ^ tail ^ (std::uint64_t(n) << 56));
}

// ------------------------------------------------------------------ allocator / owned units
UnitAllocator::UnitAllocator(std::int32_t total) : total_(total) {
  for (std::int32_t i = total - 1; i >= 1; --i) free_.push_back(i);   // id 1 is handed out first
}
bool UnitAllocator::take(std::int32_t n, std::vector<std::int32_t>& out) {
  if (n < 0 || std::size_t(n) > free_.size()) return false;
  for (std::int32_t i = 0; i < n; ++i) { out.push_back(free_.back()); free_.pop_back(); }
  return true;
}
void UnitAllocator::give(const std::vector<std::int32_t>& ids) { for (auto id : ids) give_one(id); }
void UnitAllocator::give_one(std::int32_t id) {
  if (id <= 0 || id >= total_) throw InvariantError("unit id " + std::to_string(id) + " outside the tier");
  free_.push_back(id);
}

OwnedUnits::OwnedUnits(std::weak_ptr<PrefixCache> owner, Tier t, std::vector<std::int32_t> ids)
    : owner_(std::move(owner)), tier_(t), ids_(std::move(ids)) {}
OwnedUnits::OwnedUnits(OwnedUnits&& o) noexcept : owner_(std::move(o.owner_)), tier_(o.tier_), ids_(std::move(o.ids_)) { o.ids_.clear(); }
OwnedUnits& OwnedUnits::operator=(OwnedUnits&& o) noexcept {
  if (this != &o) { drop(); owner_ = std::move(o.owner_); tier_ = o.tier_; ids_ = std::move(o.ids_); o.ids_.clear(); }
  return *this;
}
OwnedUnits::~OwnedUnits() { drop(); }
void OwnedUnits::drop() {
  if (ids_.empty()) return;
  if (auto c = owner_.lock()) c->give_back(tier_, ids_);
  ids_.clear();
}
OwnedUnits OwnedUnits::take_first(std::size_t n) {
  if (n > ids_.size()) throw UsageError("take_first: more units requested than owned");
  std::vector<std::int32_t> head(ids_.begin(), ids_.begin() + n);
  ids_.erase(ids_.begin(), ids_.begin() + n);
  return OwnedUnits(owner_, tier_, std::move(head));
}
OwnedUnits OwnedUnits::take_last(std::size_t n) {
  if (n > ids_.size()) throw UsageError("take_last: more units requested than owned");
  std::vector<std::int32_t> tail(ids_.end() - n, ids_.end());
  ids_.resize(ids_.size() - n);
  return OwnedUnits(owner_, tier_, std::move(tail));
}
void OwnedUnits::append(OwnedUnits&& o) {
  if (!o.ids_.empty() && !ids_.empty() && o.tier_ != tier_) throw UsageError("append: units of different tiers");
  if (ids_.empty()) { tier_ = o.tier_; owner_ = o.owner_; }
  ids_.insert(ids_.end(), o.ids_.begin(), o.ids_.end());
  o.ids_.clear();
}
std::vector<std::int32_t> OwnedUnits::release() { auto v = std::move(ids_); ids_.clear(); return v; }

void NodeRef::release() {
  if (node_ == 0) return;
  if (auto c = c_.lock()) c->unpin(node_, tiers_);
  node_ = 0;
}

// ------------------------------------------------------------------ tree helpers
std::size_t Node::child_count() const {
  std::size_t n = 0;
  for (auto& kv : children) n += kv.second.size();
  return n;
}

std::int64_t PrefixCache::now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

PrefixCache::PrefixCache(Config cfg) : cfg_(std::move(cfg)) {
  if (cfg_.atom_bytes == 0 || cfg_.atoms_per_unit == 0) throw UsageError("atom_bytes and atoms_per_unit must be positive");
  static const char* kPolicies[] = {"lru", "lfu", "slru", "priority"};
  if (std::find_if(std::begin(kPolicies), std::end(kPolicies), [&](const char* p) { return cfg_.policy == p; }) == std::end(kPolicies))
    throw UsageError("unknown eviction policy '" + cfg_.policy + "' (lru, lfu, slru, priority)");
  root_ = std::make_unique<Node>();
  for (int t = 0; t < kTiers; ++t) {
    alloc_[t] = UnitAllocator(cfg_.tiers[t].total_units);
    root_->state[t] = ResState::Ready;   // the empty prefix is present everywhere
  }
  live_.insert(root_.get());
}
PrefixCache::~PrefixCache() = default;

Node* PrefixCache::checked(std::uint64_t handle) const {
  auto* n = reinterpret_cast<Node*>(static_cast<std::uintptr_t>(handle));
  if (handle == 0 || !live_.count(n)) throw UsageError("stale or foreign node handle");
  return n;
}

Node* PrefixCache::find_child(Node* n, std::string_view first_page) const {
  auto it = n->children.find(hash_bytes(first_page.data(), first_page.size()));
  if (it == n->children.end()) return nullptr;
  for (auto& c : it->second)
    if (std::memcmp(c->key.data(), first_page.data(), first_page.size()) == 0) return c.get();
  return nullptr;
}

Node* PrefixCache::add_child(Node* parent, std::string key) {
  auto c = std::make_unique<Node>();
  c->parent = parent;
  c->depth_atoms = parent->depth_atoms + std::uint32_t(key.size() / cfg_.atom_bytes);
  c->last_step = step_;
  c->last_ns = now_ns();
  const std::uint64_t h = hash_bytes(key.data(), page_bytes());
  c->key = std::move(key);
  Node* raw = c.get();
  parent->children[h].push_back(std::move(c));
  live_.insert(raw);
  return raw;
}

// `n` keeps its first `pages` pages; the remainder (with its share of every tier's units, the
// children, the recurrent-state slot) moves into a new child. Pins stay on both halves, since a
// reference to the old node referred to the whole edge.
Node* PrefixCache::split(Node* n, std::size_t pages) {
  const std::size_t pb = page_bytes(), total = n->key.size() / pb;
  if (pages == 0 || pages >= total) throw InvariantError("split point outside the edge");
  auto tail = std::make_unique<Node>();
  tail->parent = n;
  tail->key = n->key.substr(pages * pb);
  tail->children = std::move(n->children);
  n->children.clear();
  for (auto& kv : tail->children) for (auto& c : kv.second) c->parent = tail.get();
  for (int t = 0; t < kTiers; ++t) {
    auto& u = n->units[t];
    if (!u.empty()) {
      tail->units[t].assign(u.begin() + pages, u.end());
      u.resize(pages);
    }
    tail->state[t] = n->state[t];
    tail->pins[t] = n->pins[t];
    tail->inflight[t] = n->inflight[t];
  }
  tail->hits = n->hits; tail->last_step = n->last_step; tail->last_ns = n->last_ns; tail->priority = n->priority;
  tail->mamba = n->mamba; n->mamba = -1;               // the state describes the end of the old edge
  tail->depth_atoms = n->depth_atoms;
  n->depth_atoms -= std::uint32_t(tail->key.size() / cfg_.atom_bytes);
  n->key.resize(pages * pb);
  Node* raw = tail.get();
  for (auto& kv : ops_) if (kv.second.node == n) { /* ops address whole edges: refuse to split under one */ throw UsageError("cannot split a node with an operation in flight"); }
  n->children[hash_bytes(raw->key.data(), pb)].push_back(std::move(tail));
  live_.insert(raw);
  return raw;
}

void PrefixCache::touch(Node* n) { n->hits += 1; n->last_step = step_; n->last_ns = now_ns(); }

// ------------------------------------------------------------------ match / insert
PrefixCache::Match PrefixCache::match(std::string_view atoms) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  const std::size_t pb = page_bytes();
  if (atoms.size() % cfg_.atom_bytes) throw UsageError("query length is not a whole number of atoms");
  Match m;
  std::array<bool, kTiers> alive;
  for (int t = 0; t < kTiers; ++t) { alive[t] = true; m.last_node[t] = reinterpret_cast<std::uintptr_t>(root_.get()); }
  Node* cur = root_.get();
  std::size_t pos = 0;
  while (atoms.size() - pos >= pb) {
    Node* c = find_child(cur, atoms.substr(pos, pb));
    if (!c) break;
    const std::size_t pages = c->key.size() / pb;
    std::size_t same = 1;
    while (same < pages && atoms.size() - pos >= (same + 1) * pb &&
           std::memcmp(c->key.data() + same * pb, atoms.data() + pos + same * pb, pb) == 0)
      ++same;
    if (same < pages) {
      bool busy = false;
      for (auto& kv : ops_) busy = busy || kv.second.node == c;
      if (busy) break;          // an edge under a tier move cannot be split: stop in front of it
      split(c, same);
    }
    touch(c);
    pos += same * pb;
    for (int t = 0; t < kTiers; ++t) {
      alive[t] = alive[t] && c->has(Tier(t));
      if (alive[t]) { m.last_node[t] = reinterpret_cast<std::uintptr_t>(c); m.matched_atoms[t] = std::uint32_t(pos / cfg_.atom_bytes); }
    }
    cur = c;
    if (same < pages) break;
  }
  return m;
}

std::vector<std::int32_t> PrefixCache::collect_units(std::uint64_t node, Tier t) const {
  std::lock_guard<std::recursive_mutex> g(mu_);
  std::vector<const Node*> path;
  for (const Node* n = checked(node); n && n->parent; n = n->parent) path.push_back(n);
  std::vector<std::int32_t> out;
  for (auto it = path.rbegin(); it != path.rend(); ++it) {
    if (!(*it)->has(t)) throw UsageError("collect_units: a node on the path has no ready units on this tier");
    out.insert(out.end(), (*it)->units[int(t)].begin(), (*it)->units[int(t)].end());
  }
  return out;
}

PrefixCache::Inserted PrefixCache::insert(Tier t, std::string_view atoms, OwnedUnits&& units) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  const std::size_t pb = page_bytes();
  if (atoms.size() % pb) throw UsageError("insert: atoms must be a whole number of pages (use page_align)");
  const std::size_t pages = atoms.size() / pb;
  if (units.size() != pages) throw UsageError("insert: need exactly one unit per page");
  if (units.size() && units.tier() != t) throw UsageError("insert: units belong to another tier");
  std::vector<std::int32_t> ids = units.release();
  Inserted r;
  Node* cur = root_.get();
  std::size_t page = 0;
  std::vector<std::int32_t> freed;
  while (page < pages) {
    Node* c = find_child(cur, atoms.substr(page * pb, pb));
    if (!c) break;
    const std::size_t cp = c->key.size() / pb;
    std::size_t same = 1;
    while (same < cp && page + same < pages && std::memcmp(c->key.data() + same * pb, atoms.data() + (page + same) * pb, pb) == 0) ++same;
    if (same < cp) split(c, same);
    touch(c);
    const int ti = int(t);
    if (c->state[ti] == ResState::Ready || c->state[ti] == ResState::Pending) {
      freed.insert(freed.end(), ids.begin() + page, ids.begin() + page + same);   // already cached: caller's copies are surplus
    } else {
      c->units[ti].assign(ids.begin() + page, ids.begin() + page + same);
      c->state[ti] = ResState::Ready;
      r.inserted_atoms += std::uint32_t(same * cfg_.atoms_per_unit);
    }
    page += same;
    cur = c;
  }
  if (page < pages) {
    Node* c = add_child(cur, std::string(atoms.substr(page * pb)));
    c->units[int(t)].assign(ids.begin() + page, ids.end());
    c->state[int(t)] = ResState::Ready;
    c->hits = 1;
    r.inserted_atoms += std::uint32_t((pages - page) * cfg_.atoms_per_unit);
    cur = c;
  }
  if (!freed.empty()) alloc_[int(t)].give(freed);
  r.freed_units = std::uint32_t(freed.size());
  r.last_node = reinterpret_cast<std::uintptr_t>(cur);
  Event e{EventKind::Insert};
  e.node = r.last_node; e.tier_to = int(t); e.step = step_;
  push_event(std::move(e));
  return r;
}

OwnedUnits PrefixCache::allocate(Tier t, std::int32_t n) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  std::vector<std::int32_t> ids;
  if (!alloc_[int(t)].take(n, ids))
    throw CapacityError("tier " + std::to_string(int(t)) + ": " + std::to_string(n) + " units requested, " +
                        std::to_string(alloc_[int(t)].available()) + " free");
  return OwnedUnits(weak_from_this(), t, std::move(ids));
}

void PrefixCache::give_back(Tier t, const std::vector<std::int32_t>& ids) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  alloc_[int(t)].give(ids);
}

std::shared_ptr<NodeRef> PrefixCache::lock(std::uint64_t node, const std::vector<Tier>& tiers) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  for (Node* n = checked(node); n; n = n->parent)
    for (Tier t : tiers) n->pins[int(t)] += 1;
  return std::make_shared<NodeRef>(weak_from_this(), node, tiers);
}
void PrefixCache::unpin(std::uint64_t node, const std::vector<Tier>& tiers) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  auto* start = reinterpret_cast<Node*>(static_cast<std::uintptr_t>(node));
  if (!live_.count(start)) return;   // the node went away with the cache contents
  for (Node* n = start; n; n = n->parent)
    for (Tier t : tiers) if (n->pins[int(t)] > 0) n->pins[int(t)] -= 1;
}

// ------------------------------------------------------------------ eviction
bool PrefixCache::evictable(const Node& n, Tier t) const {
  const int ti = int(t);
  if (!n.parent || n.state[ti] != ResState::Ready || n.pins[ti] > 0 || n.inflight[ti] > 0) return false;
  // a prefix must stay resident while a longer one is: only the deepest holders of a tier may go
  for (auto& kv : n.children)
    for (auto& c : kv.second)
      if (c->state[ti] == ResState::Ready || c->state[ti] == ResState::Pending) return false;
  return true;
}

bool PrefixCache::better_victim(const Node& a, const Node& b) const {
  const std::string& p = cfg_.policy;
  if (p == "lfu") { if (a.hits != b.hits) return a.hits < b.hits; }
  else if (p == "slru") {
    const bool ap = a.hits < cfg_.slru_threshold, bp = b.hits < cfg_.slru_threshold;   // probationary segment goes first
    if (ap != bp) return ap;
  } else if (p == "priority") { if (a.priority != b.priority) return a.priority < b.priority; }
  if (a.last_ns != b.last_ns) return a.last_ns < b.last_ns;
  return a.depth_atoms > b.depth_atoms;
}

void PrefixCache::prune(Node* n) {
  while (n && n->parent) {
    bool holds = n->mamba >= 0 || n->child_count() > 0;
    for (int t = 0; t < kTiers; ++t) holds = holds || n->state[t] != ResState::Absent || n->pins[t] > 0 || n->inflight[t] > 0;
    if (holds) return;
    Node* parent = n->parent;
    auto it = parent->children.find(hash_bytes(n->key.data(), page_bytes()));
    if (it == parent->children.end()) throw InvariantError("node missing from its parent's child map");
    auto& vec = it->second;
    auto pos = std::find_if(vec.begin(), vec.end(), [&](auto& u) { return u.get() == n; });
    if (pos == vec.end()) throw InvariantError("node missing from its parent's bucket");
    if (removed_hook_) removed_hook_(*n);
    live_.erase(n);
    vec.erase(pos);
    if (vec.empty()) parent->children.erase(it);
    n = parent;
  }
}

std::uint32_t PrefixCache::evict_node(Node* n, Tier t, std::optional<Tier> promote_to) {
  const int ti = int(t);
  const auto handle = std::uint64_t(reinterpret_cast<std::uintptr_t>(n));
  if (promote_to && *promote_to != t && n->state[int(*promote_to)] == ResState::Absent && tier_enabled(*promote_to)) {
    const auto need = std::int32_t(n->units[ti].size());
    if (alloc_[int(*promote_to)].available() < need) ensure_capacity(*promote_to, need);
    start_move(handle, t, *promote_to, true);       // units leave tier t when the caller completes the op
    return 0;
  }
  const auto freed = std::uint32_t(n->units[ti].size());
  Event e{EventKind::Evict};
  e.node = handle; e.tier_from = ti; e.units_from = n->units[ti]; e.step = step_;
  alloc_[ti].give(n->units[ti]);
  n->units[ti].clear();
  n->state[ti] = ResState::Absent;
  push_event(std::move(e));
  for (auto& kv : observers_) kv.second(handle, ti);
  prune(n);
  return freed;
}

void PrefixCache::ensure_capacity(Tier t, std::int32_t need, std::optional<Tier> promote_to) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  const int ti = int(t);
  if (need >= alloc_[ti].total()) throw CapacityError("request exceeds the tier's size");
  while (alloc_[ti].available() < need) {
    Node* best = nullptr;
    for (const Node* cn : live_) {
      auto* n = const_cast<Node*>(cn);
      if (evictable(*n, t) && (!best || better_victim(*n, *best))) best = n;
    }
    if (!best) {
      if (pending_[ti] > 0) throw CapacityError("tier is full of units with moves in flight; complete them first");
      throw CapacityError("nothing evictable: every cached prefix on this tier is pinned");
    }
    const std::int32_t before = alloc_[ti].available() + pending_[ti];
    evict_node(best, t, promote_to);
    if (promote_to && alloc_[ti].available() + pending_[ti] == before && alloc_[ti].available() < need) {
      // demotions free their units only on completion; respect the in-flight budget
      const std::int32_t cap = cfg_.tiers[ti].max_pending_units;
      if (cap > 0 && pending_[ti] >= cap) throw CapacityError("pending-move budget of the tier is exhausted");
    }
    if (promote_to) {
      std::int32_t leaving = 0;
      for (auto& kv : ops_) if (!kv.second.done && kv.second.demote && kv.second.src == t) leaving += std::int32_t(kv.second.node->units[ti].size());
      if (alloc_[ti].available() + leaving >= need) return;   // enough will be free once the caller finishes the copies
    }
  }
}

std::uint32_t PrefixCache::evict_if(Tier t, const std::function<bool(const Node&)>& pred) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  std::uint32_t freed = 0;
  bool again = true;
  while (again) {        // removing a leaf can expose its parent
    again = false;
    std::vector<Node*> victims;
    for (const Node* cn : live_) {
      auto* n = const_cast<Node*>(cn);
      if (evictable(*n, t) && pred(*n)) victims.push_back(n);
    }
    for (Node* n : victims)
      if (live_.count(n) && evictable(*n, t)) { freed += evict_node(n, t, std::nullopt); again = true; }
  }
  return freed;
}

std::uint32_t PrefixCache::evict_named(Tier t, const std::string& pred, std::int64_t arg) {
  const std::int64_t now = now_ns();
  if (pred == "step_le") return evict_if(t, [&](const Node& n) { return std::int64_t(n.last_step) <= arg; });
  if (pred == "step_lt") return evict_if(t, [&](const Node& n) { return std::int64_t(n.last_step) < arg; });
  if (pred == "hits_lt") return evict_if(t, [&](const Node& n) { return std::int64_t(n.hits) < arg; });
  if (pred == "priority_le") return evict_if(t, [&](const Node& n) { return n.priority <= arg; });
  if (pred == "age_ns_ge") return evict_if(t, [&](const Node& n) { return now - n.last_ns >= arg; });
  throw UsageError("unknown predicate '" + pred + "' (step_le, step_lt, hits_lt, priority_le, age_ns_ge)");
}

// ------------------------------------------------------------------ statistics
std::int32_t PrefixCache::available(Tier t) const { std::lock_guard<std::recursive_mutex> g(mu_); return alloc_[int(t)].available(); }
std::int32_t PrefixCache::total(Tier t) const { return alloc_[int(t)].total(); }
std::int32_t PrefixCache::active(Tier t) const {
  std::lock_guard<std::recursive_mutex> g(mu_);
  const auto tot = alloc_[int(t)].total();
  return tot > 0 ? tot - 1 - alloc_[int(t)].available() : 0;
}
std::int32_t PrefixCache::pending_units(Tier t) const { std::lock_guard<std::recursive_mutex> g(mu_); return pending_[int(t)]; }

// ------------------------------------------------------------------ two-phase tier moves
std::uint64_t PrefixCache::start_move(std::uint64_t node, Tier src, Tier dst, bool demote) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  Node* n = checked(node);
  const int si = int(src), di = int(dst);
  if (src == dst) throw UsageError("source and destination tiers are the same");
  if (!n->parent) throw UsageError("the root holds no units");
  if (n->state[si] != ResState::Ready) throw UsageError("node has no ready units on the source tier");
  if (n->state[di] != ResState::Absent) throw UsageError("node already has (or is receiving) units on the destination tier");
  const auto k = std::int32_t(n->units[si].size());
  const std::int32_t cap = cfg_.tiers[di].max_pending_units;
  if (cap > 0 && pending_[di] + k > cap) throw CapacityError("pending-move budget of the destination tier is exhausted");
  std::vector<std::int32_t> ids;
  if (!alloc_[di].take(k, ids)) throw CapacityError("destination tier has no room for the move");
  n->units[di] = std::move(ids);
  n->state[di] = ResState::Pending;
  n->inflight[si] += 1; n->inflight[di] += 1;
  pending_[di] += k;
  const std::uint64_t id = next_op_++;
  ops_.emplace(id, Op{id, n, src, dst, demote});
  Event e{demote ? EventKind::DemoteStart : EventKind::PromoteStart};
  e.node = node; e.tier_from = si; e.tier_to = di; e.units_from = n->units[si]; e.units_to = n->units[di]; e.op = id; e.step = step_;
  push_event(std::move(e));
  return id;
}

void PrefixCache::complete_op(std::uint64_t op, bool success) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  auto it = ops_.find(op);
  if (it == ops_.end()) throw UsageError("unknown operation handle");
  Op& o = it->second;
  if (o.done) throw UsageError("operation already completed");
  Node* n = o.node;
  const int si = int(o.src), di = int(o.dst);
  pending_[di] -= std::int32_t(n->units[di].size());
  n->inflight[si] -= 1; n->inflight[di] -= 1;
  if (success) {
    n->state[di] = ResState::Ready;
    if (o.demote) {               // the payload now lives below: release the upper copy
      alloc_[si].give(n->units[si]);
      n->units[si].clear();
      n->state[si] = ResState::Absent;
      for (auto& kv : observers_) kv.second(std::uint64_t(reinterpret_cast<std::uintptr_t>(n)), si);
    }
  } else {
    alloc_[di].give(n->units[di]);
    n->units[di].clear();
    n->state[di] = ResState::Absent;
  }
  o.done = true; o.ok = success;
  Event e{success ? EventKind::OpDone : EventKind::OpFailed};
  e.node = std::uint64_t(reinterpret_cast<std::uintptr_t>(n)); e.tier_from = si; e.tier_to = di; e.op = op; e.step = step_;
  push_event(std::move(e));
  prune(n);
  op_cv_.notify_all();
}

bool PrefixCache::wait_op(std::uint64_t op, std::int64_t timeout_ms) {
  std::unique_lock<std::recursive_mutex> g(mu_);
  auto finished = [&] { auto it = ops_.find(op); return it == ops_.end() || it->second.done; };
  if (ops_.find(op) == ops_.end()) throw UsageError("unknown operation handle");
  if (timeout_ms <= 0) op_cv_.wait(g, finished);
  else if (!op_cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), finished)) return false;
  auto it = ops_.find(op);
  const bool ok = it != ops_.end() && it->second.ok;
  if (it != ops_.end()) ops_.erase(it);
  return ok;
}

std::size_t PrefixCache::fail_all_inflight() {
  std::lock_guard<std::recursive_mutex> g(mu_);
  std::vector<std::uint64_t> open;
  for (auto& kv : ops_) if (!kv.second.done) open.push_back(kv.first);
  for (auto id : open) complete_op(id, false);
  return open.size();
}
std::vector<std::uint64_t> PrefixCache::inflight_ops() const {
  std::lock_guard<std::recursive_mutex> g(mu_);
  std::vector<std::uint64_t> v;
  for (auto& kv : ops_) if (!kv.second.done) v.push_back(kv.first);
  std::sort(v.begin(), v.end());
  return v;
}

// ------------------------------------------------------------------ observers, events, node metadata
std::uint64_t PrefixCache::add_evict_observer(std::function<void(std::uint64_t, int)> cb) {
  std::lock_guard<std::recursive_mutex> g(mu_);
  observers_[next_obs_] = std::move(cb);
  return next_obs_++;
}
bool PrefixCache::remove_evict_observer(std::uint64_t id) { std::lock_guard<std::recursive_mutex> g(mu_); return observers_.erase(id) > 0; }
void PrefixCache::push_event(Event e) {
  if (cfg_.max_events == 0) return;
  if (events_.size() >= cfg_.max_events) { events_.pop_front(); ++dropped_; }
  events_.push_back(std::move(e));
}
std::vector<Event> PrefixCache::take_events() {
  std::lock_guard<std::recursive_mutex> g(mu_);
  std::vector<Event> v(std::make_move_iterator(events_.begin()), std::make_move_iterator(events_.end()));
  events_.clear();
  return v;
}
void PrefixCache::touch_step(std::uint64_t node) { std::lock_guard<std::recursive_mutex> g(mu_); Node* n = checked(node); n->last_step = step_; n->last_ns = now_ns(); }
std::uint64_t PrefixCache::node_path_hash(std::uint64_t node) const {
  std::lock_guard<std::recursive_mutex> g(mu_);
  std::vector<const Node*> path;
  for (const Node* n = checked(node); n && n->parent; n = n->parent) path.push_back(n);
  std::uint64_t h = 0;
  for (auto it = path.rbegin(); it != path.rend(); ++it) h = hash_bytes((*it)->key.data(), (*it)->key.size(), h);
  return h;
}
const Node& PrefixCache::node_info(std::uint64_t node) const { std::lock_guard<std::recursive_mutex> g(mu_); return *checked(node); }
void PrefixCache::set_priority(std::uint64_t node, std::int64_t p) { std::lock_guard<std::recursive_mutex> g(mu_); checked(node)->priority = p; }

}  // namespace pbc
