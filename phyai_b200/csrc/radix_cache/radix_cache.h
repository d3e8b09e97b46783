// Multi-tier radix prefix cache (host-side C++20, no CUDA).
//
// The cache maps byte strings ("atoms": fixed-size records such as token ids or content
// hashes) to *unit ids* of caller-owned storage (KV pages, embedding rows). It never touches
// the payload itself. A unit covers `atoms_per_unit` atoms (one page); tree edges hold whole
// pages and are split at page boundaries only. Each node can hold units on several tiers
// (device, host, disk, remote) at once; moving a node's payload between tiers is a two-phase
// operation (start -> the caller copies -> complete) tracked by an op handle.
//
// Same role and Python surface as the reference's native cache
// (phyai-ext/csrc/radix_cache/prefix_cache.h:75-330, tree/radix_tree.h, tree/eviction.h,
// unit_allocator.h, owned_units.h, storage_backend.h, mamba/hybrid_prefix_cache.h).
#pragma once
#include <array>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace pbc {

constexpr int kTiers = 4;
enum class Tier : int { Device = 0, Host = 1, Disk = 2, Remote = 3 };

struct CapacityError : std::runtime_error { using std::runtime_error::runtime_error; };
struct UsageError : std::invalid_argument { using std::invalid_argument::invalid_argument; };
struct InvariantError : std::logic_error { using std::logic_error::logic_error; };

// 64-bit non-cryptographic hash of a byte span (multiply-xorshift over 8-byte lanes).
std::uint64_t hash_bytes(const void* data, std::size_t n, std::uint64_t seed = 0);

enum class ResState : std::uint8_t { Absent = 0, Ready = 1, Pending = 2, Failed = 3 };

// ------------------------------------------------------------------ unit allocator
// Hands out ids 1..N-1 (0 is the "no unit" sentinel), most recently freed first.
class UnitAllocator {
 public:
  explicit UnitAllocator(std::int32_t total = 0);
  std::int32_t total() const { return total_; }
  std::int32_t available() const { return std::int32_t(free_.size()); }
  bool take(std::int32_t n, std::vector<std::int32_t>& out);
  void give(const std::vector<std::int32_t>& ids);
  void give_one(std::int32_t id);
 private:
  std::int32_t total_ = 0;
  std::vector<std::int32_t> free_;
};

class PrefixCache;

// Units taken from a tier's allocator and not yet attached to the tree. Move-only; whatever is
// still owned when the object dies goes back to the allocator.
class OwnedUnits {
 public:
  OwnedUnits() = default;
  OwnedUnits(std::weak_ptr<PrefixCache> owner, Tier t, std::vector<std::int32_t> ids);
  OwnedUnits(OwnedUnits&&) noexcept;
  OwnedUnits& operator=(OwnedUnits&&) noexcept;
  OwnedUnits(const OwnedUnits&) = delete;
  OwnedUnits& operator=(const OwnedUnits&) = delete;
  ~OwnedUnits();
  Tier tier() const { return tier_; }
  std::size_t size() const { return ids_.size(); }
  const std::vector<std::int32_t>& ids() const { return ids_; }
  OwnedUnits take_first(std::size_t n);
  OwnedUnits take_last(std::size_t n);
  void append(OwnedUnits&& other);
  std::vector<std::int32_t> release();   // give up ownership (the ids now belong to the caller)
 private:
  void drop();
  std::weak_ptr<PrefixCache> owner_;
  Tier tier_ = Tier::Device;
  std::vector<std::int32_t> ids_;
};

// ------------------------------------------------------------------ tree
struct Node {
  Node* parent = nullptr;
  std::string key;                                   // whole pages of atoms on the edge into this node
  std::unordered_map<std::uint64_t, std::vector<std::unique_ptr<Node>>> children;  // by hash of first page
  std::array<std::vector<std::int32_t>, kTiers> units;   // one id per page of `key`, per tier
  std::array<ResState, kTiers> state{};
  std::array<std::int32_t, kTiers> pins{};           // live references through NodeRef, per tier
  std::array<std::int32_t, kTiers> inflight{};       // ops reading or writing this tier's units
  std::uint64_t hits = 0;
  std::uint64_t last_step = 0;
  std::int64_t last_ns = 0;
  std::int64_t priority = 0;
  std::int32_t mamba = -1;                           // attached recurrent-state slot, -1 = none
  std::uint32_t depth_atoms = 0;                     // atoms from the root to the end of this node
  std::size_t child_count() const;
  bool has(Tier t) const { return state[int(t)] == ResState::Ready; }
};

enum class EventKind : int { Insert = 0, Evict = 1, DemoteStart = 2, PromoteStart = 3, OpDone = 4, OpFailed = 5, MambaEvict = 6 };
struct Event {
  EventKind kind;
  std::uint64_t node = 0;
  int tier_from = -1, tier_to = -1;
  std::vector<std::int32_t> units_from, units_to;
  std::uint64_t op = 0;
  std::uint64_t step = 0;
};

struct TierConfig { std::int32_t total_units = 0; std::int32_t max_pending_units = 0; };
struct Config {
  std::uint32_t atom_bytes = 4, atoms_per_unit = 1;
  std::array<TierConfig, kTiers> tiers{};
  std::string policy = "lru";
  std::uint32_t slru_threshold = 2;
  std::size_t max_events = 16384;
};

class NodeRef;

class PrefixCache : public std::enable_shared_from_this<PrefixCache> {
 public:
  explicit PrefixCache(Config cfg);
  ~PrefixCache();
  static std::shared_ptr<PrefixCache> create(Config cfg) { return std::make_shared<PrefixCache>(std::move(cfg)); }

  struct Match { std::array<std::uint64_t, kTiers> last_node{}; std::array<std::uint32_t, kTiers> matched_atoms{}; };
  Match match(std::string_view atoms);
  std::vector<std::int32_t> collect_units(std::uint64_t node, Tier t) const;
  struct Inserted { std::uint64_t last_node = 0; std::uint32_t inserted_atoms = 0, freed_units = 0; };
  Inserted insert(Tier t, std::string_view atoms, OwnedUnits&& units);
  OwnedUnits allocate(Tier t, std::int32_t n);
  std::shared_ptr<NodeRef> lock(std::uint64_t node, const std::vector<Tier>& tiers);
  void ensure_capacity(Tier t, std::int32_t need, std::optional<Tier> promote_to = std::nullopt);
  std::uint32_t evict_if(Tier t, const std::function<bool(const Node&)>& pred);
  std::uint32_t evict_named(Tier t, const std::string& pred, std::int64_t arg);

  std::int32_t available(Tier t) const;
  std::int32_t total(Tier t) const;
  std::int32_t active(Tier t) const;
  std::int32_t pending_units(Tier t) const;
  std::int32_t max_pending_units(Tier t) const { return cfg_.tiers[int(t)].max_pending_units; }
  bool tier_enabled(Tier t) const { return cfg_.tiers[int(t)].total_units > 1; }

  std::uint64_t start_move(std::uint64_t node, Tier src, Tier dst, bool demote);
  void complete_op(std::uint64_t op, bool success);
  bool wait_op(std::uint64_t op, std::int64_t timeout_ms);
  std::size_t fail_all_inflight();
  std::vector<std::uint64_t> inflight_ops() const;

  std::uint64_t add_evict_observer(std::function<void(std::uint64_t, int)> cb);
  bool remove_evict_observer(std::uint64_t id);
  std::vector<Event> take_events();
  std::uint64_t dropped_events() const { return dropped_; }

  std::uint64_t current_step() const { return step_; }
  void advance_step(std::uint64_t n) { std::lock_guard<std::recursive_mutex> g(mu_); step_ += n; }
  void touch_step(std::uint64_t node);
  std::uint64_t node_path_hash(std::uint64_t node) const;
  const Node& node_info(std::uint64_t node) const;
  void set_priority(std::uint64_t node, std::int64_t p);
  std::size_t node_count() const { return live_.size(); }

  const Config& config() const { return cfg_; }
  std::uint32_t page_bytes() const { return cfg_.atom_bytes * cfg_.atoms_per_unit; }

  // internals shared with OwnedUnits / NodeRef / the hybrid cache
  void give_back(Tier t, const std::vector<std::int32_t>& ids);
  void unpin(std::uint64_t node, const std::vector<Tier>& tiers);
  Node* checked(std::uint64_t handle) const;
  std::recursive_mutex& mutex() const { return mu_; }
  void on_node_removed(std::function<void(Node&)> hook) { removed_hook_ = std::move(hook); }
  Node* root() const { return root_.get(); }

 private:
  struct Op { std::uint64_t id; Node* node; Tier src, dst; bool demote; bool done = false, ok = false; };
  Node* split(Node* n, std::size_t pages);           // n keeps the first `pages`, the rest moves to a new child
  Node* find_child(Node* n, std::string_view first_page) const;
  Node* add_child(Node* parent, std::string key);
  void touch(Node* n);
  bool evictable(const Node& n, Tier t) const;
  bool better_victim(const Node& a, const Node& b) const;   // true when a should go before b
  std::uint32_t evict_node(Node* n, Tier t, std::optional<Tier> promote_to);
  void prune(Node* n);
  void push_event(Event e);
  static std::int64_t now_ns();

  Config cfg_;
  mutable std::recursive_mutex mu_;
  std::unique_ptr<Node> root_;
  std::unordered_set<const Node*> live_;
  std::array<UnitAllocator, kTiers> alloc_;
  std::array<std::int32_t, kTiers> pending_{};
  std::uint64_t step_ = 0, next_op_ = 1, next_obs_ = 1, dropped_ = 0;
  std::unordered_map<std::uint64_t, Op> ops_;
  std::condition_variable_any op_cv_;
  std::unordered_map<std::uint64_t, std::function<void(std::uint64_t, int)>> observers_;
  std::deque<Event> events_;
  std::function<void(Node&)> removed_hook_;
};

// Pins the path root -> node on the given tiers until destroyed (or release() is called).
class NodeRef {
 public:
  NodeRef(std::weak_ptr<PrefixCache> c, std::uint64_t node, std::vector<Tier> tiers) : c_(std::move(c)), node_(node), tiers_(std::move(tiers)) {}
  ~NodeRef() { release(); }
  void release();
  bool valid() const { return node_ != 0; }
  std::uint64_t node() const { return node_; }
  const std::vector<Tier>& tiers() const { return tiers_; }
 private:
  std::weak_ptr<PrefixCache> c_;
  std::uint64_t node_;
  std::vector<Tier> tiers_;
};

// ------------------------------------------------------------------ payload stores for the lower tiers
class StorageBackend {
 public:
  virtual ~StorageBackend() = default;
  virtual std::string name() const = 0;
  virtual std::size_t unit_bytes() const = 0;
  virtual bool write(std::uint64_t key, std::string_view payload) = 0;     // payload: k * unit_bytes
  virtual std::optional<std::string> read(std::uint64_t key) = 0;
  virtual bool contains(std::uint64_t key) const = 0;
  virtual bool erase(std::uint64_t key) = 0;
  virtual std::size_t entries() const = 0;
  virtual void drain() = 0;                                                  // flush buffered writes
};
std::shared_ptr<StorageBackend> make_memory_backend(std::size_t unit_bytes);
std::shared_ptr<StorageBackend> make_file_backend(const std::string& path, std::size_t unit_bytes);

// ------------------------------------------------------------------ recurrent-state (Mamba / GDN) slots on the same tree
class HybridPrefixCache {
 public:
  HybridPrefixCache(std::shared_ptr<PrefixCache> kv, std::int32_t slots);
  struct Match { PrefixCache::Match kv; std::uint64_t mamba_node = 0; std::uint32_t mamba_atoms = 0; std::int32_t mamba_slot = -1; };
  Match match(std::string_view atoms);
  std::int32_t allocate_slot();                       // -1 when none is free
  void free_slot(std::int32_t slot);
  void attach(std::uint64_t node, std::int32_t slot);
  std::int32_t detach(std::uint64_t node);            // returns the slot (still allocated) or -1
  std::uint64_t find_last_mamba_node(std::uint64_t from) const;
  bool ensure_slots_by_evict(std::int32_t n);
  std::int32_t available_slots() const { return std::int32_t(free_.size()); }
  std::int32_t total_slots() const { return total_; }
  std::int32_t active_slots() const { return total_ - std::int32_t(free_.size()); }
  std::shared_ptr<PrefixCache> kv() const { return kv_; }
 private:
  std::shared_ptr<PrefixCache> kv_;
  std::int32_t total_;
  std::vector<std::int32_t> free_;
  std::unordered_set<Node*> holders_;
};

}  // namespace pbc
