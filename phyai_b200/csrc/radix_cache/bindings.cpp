// pybind11 surface of the prefix cache: module phyai_b200._radix (no CUDA, no torch).
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "radix_cache.h"

namespace py = pybind11;
using namespace pbc;

namespace {

std::string_view view_of(const py::bytes& b, std::string& keep) {
  keep = b;   // one copy; queries are short (a prompt's worth of atoms)
  return keep;
}

}  // namespace

PYBIND11_MODULE(_radix, m) {
  m.doc() = "Multi-tier radix prefix cache (C++)";
  py::register_exception<CapacityError>(m, "CacheCapacityError", PyExc_RuntimeError);
  py::register_exception<UsageError>(m, "CacheUsageError", PyExc_ValueError);
  py::register_exception<InvariantError>(m, "CacheInvariantError", PyExc_RuntimeError);

  py::class_<OwnedUnits, std::shared_ptr<OwnedUnits>>(m, "OwnedUnits")
      .def_property_readonly("tier", [](const OwnedUnits& u) { return int(u.tier()); })
      .def_property_readonly("size", &OwnedUnits::size)
      .def("__len__", &OwnedUnits::size)
      .def("ids", [](const OwnedUnits& u) { return u.ids(); })
      .def("take_first", [](OwnedUnits& u, std::size_t n) { return std::make_shared<OwnedUnits>(u.take_first(n)); })
      .def("take_last", [](OwnedUnits& u, std::size_t n) { return std::make_shared<OwnedUnits>(u.take_last(n)); })
      .def("append", [](OwnedUnits& u, OwnedUnits& o) { u.append(std::move(o)); });

  py::class_<NodeRef, std::shared_ptr<NodeRef>>(m, "NodeRef")
      .def_property_readonly("node_handle", &NodeRef::node)
      .def_property_readonly("valid", &NodeRef::valid)
      .def_property_readonly("tiers", [](const NodeRef& r) { std::vector<int> v; for (Tier t : r.tiers()) v.push_back(int(t)); return v; })
      .def("release", &NodeRef::release);

  py::class_<Event>(m, "CacheEvent")
      .def_property_readonly("kind", [](const Event& e) { return int(e.kind); })
      .def_readonly("node", &Event::node)
      .def_readonly("tier_from", &Event::tier_from)
      .def_readonly("tier_to", &Event::tier_to)
      .def_readonly("units_from", &Event::units_from)
      .def_readonly("units_to", &Event::units_to)
      .def_readonly("op", &Event::op)
      .def_readonly("step", &Event::step);

  py::class_<PrefixCache, std::shared_ptr<PrefixCache>>(m, "PrefixCache")
      .def(py::init([](std::uint32_t atom_bytes, std::uint32_t atoms_per_unit, std::vector<std::int32_t> tier_units,
                       std::vector<std::int32_t> max_pending, std::string policy, std::uint32_t slru, std::size_t max_events) {
             Config c;
             c.atom_bytes = atom_bytes; c.atoms_per_unit = atoms_per_unit; c.policy = std::move(policy);
             c.slru_threshold = slru; c.max_events = max_events;
             for (int t = 0; t < kTiers; ++t) {
               c.tiers[t].total_units = t < int(tier_units.size()) ? tier_units[t] : 0;
               c.tiers[t].max_pending_units = t < int(max_pending.size()) ? max_pending[t] : 0;
             }
             return PrefixCache::create(std::move(c));
           }),
           py::arg("atom_bytes"), py::arg("atoms_per_unit"), py::arg("tier_units"), py::arg("max_pending"),
           py::arg("policy") = "lru", py::arg("slru_threshold") = 2, py::arg("max_events") = 16384)
      .def("match", [](PrefixCache& c, const py::bytes& atoms) {
             std::string keep;
             auto r = c.match(view_of(atoms, keep));
             return py::make_tuple(std::vector<std::uint64_t>(r.last_node.begin(), r.last_node.end()),
                                   std::vector<std::uint32_t>(r.matched_atoms.begin(), r.matched_atoms.end()));
           })
      .def("collect_units", [](const PrefixCache& c, std::uint64_t node, int tier) { return c.collect_units(node, Tier(tier)); })
      .def("insert", [](PrefixCache& c, int tier, const py::bytes& atoms, OwnedUnits& units) {
             std::string keep;
             auto r = c.insert(Tier(tier), view_of(atoms, keep), std::move(units));
             return py::make_tuple(r.last_node, r.inserted_atoms, r.freed_units);
           })
      .def("allocate", [](PrefixCache& c, int tier, std::int32_t n) { return std::make_shared<OwnedUnits>(c.allocate(Tier(tier), n)); })
      .def("lock", [](PrefixCache& c, std::uint64_t node, std::vector<int> tiers) {
             std::vector<Tier> ts;
             for (int t : tiers) ts.push_back(Tier(t));
             return c.lock(node, ts);
           })
      .def("ensure_capacity", [](PrefixCache& c, int tier, std::int32_t n, int promote_to) {
             c.ensure_capacity(Tier(tier), n, promote_to < 0 ? std::nullopt : std::optional<Tier>(Tier(promote_to)));
           }, py::arg("tier"), py::arg("n"), py::arg("promote_to") = -1)
      .def("evict_by_predicate", [](PrefixCache& c, int tier, py::function cb) {
             return c.evict_if(Tier(tier), [&](const Node& n) {
               return cb(std::uint64_t(reinterpret_cast<std::uintptr_t>(&n)), n.depth_atoms, n.hits, n.last_step, n.priority).cast<bool>();
             });
           })
      .def("evict_by_named_predicate", [](PrefixCache& c, int tier, const std::string& p, std::int64_t a) { return c.evict_named(Tier(tier), p, a); })
      .def("available", [](const PrefixCache& c, int t) { return c.available(Tier(t)); })
      .def("total", [](const PrefixCache& c, int t) { return c.total(Tier(t)); })
      .def("active", [](const PrefixCache& c, int t) { return c.active(Tier(t)); })
      .def("pending_units", [](const PrefixCache& c, int t) { return c.pending_units(Tier(t)); })
      .def("max_pending_units", [](const PrefixCache& c, int t) { return c.max_pending_units(Tier(t)); })
      .def("tier_enabled", [](const PrefixCache& c, int t) { return c.tier_enabled(Tier(t)); })
      .def("start_demote", [](PrefixCache& c, std::uint64_t n, int s, int d) { return c.start_move(n, Tier(s), Tier(d), true); })
      .def("start_promote", [](PrefixCache& c, std::uint64_t n, int s, int d) { return c.start_move(n, Tier(s), Tier(d), false); })
      .def("complete_op", &PrefixCache::complete_op)
      .def("wait_op", &PrefixCache::wait_op, py::arg("op"), py::arg("timeout_ms") = 0, py::call_guard<py::gil_scoped_release>())
      .def("fail_all_inflight", &PrefixCache::fail_all_inflight)
      .def("inflight_ops", &PrefixCache::inflight_ops)
      .def("add_evict_observer", [](PrefixCache& c, py::function cb) {
             return c.add_evict_observer([cb](std::uint64_t node, int tier) { py::gil_scoped_acquire g; cb(node, tier); });
           })
      .def("remove_evict_observer", &PrefixCache::remove_evict_observer)
      .def("take_events", &PrefixCache::take_events)
      .def_property_readonly("dropped_events", &PrefixCache::dropped_events)
      .def_property_readonly("current_step", &PrefixCache::current_step)
      .def("advance_step", &PrefixCache::advance_step)
      .def("touch_step", &PrefixCache::touch_step)
      .def("node_path_hash", &PrefixCache::node_path_hash)
      .def("set_priority", &PrefixCache::set_priority)
      .def_property_readonly("node_count", &PrefixCache::node_count)
      .def_property_readonly("page_bytes", &PrefixCache::page_bytes)
      .def("node_info", [](const PrefixCache& c, std::uint64_t h) {
             const Node& n = c.node_info(h);
             py::dict d;
             d["depth_atoms"] = n.depth_atoms; d["atoms"] = n.key.size() / c.config().atom_bytes; d["hits"] = n.hits;
             d["last_step"] = n.last_step; d["priority"] = n.priority; d["mamba"] = n.mamba; d["children"] = n.child_count();
             std::vector<int> st;
             for (auto s : n.state) st.push_back(int(s));
             d["state"] = st;
             return d;
           });

  py::class_<HybridPrefixCache, std::shared_ptr<HybridPrefixCache>>(m, "HybridPrefixCache")
      .def(py::init<std::shared_ptr<PrefixCache>, std::int32_t>())
      .def("match", [](HybridPrefixCache& h, const py::bytes& atoms) {
             std::string keep;
             auto r = h.match(view_of(atoms, keep));
             return py::make_tuple(std::vector<std::uint64_t>(r.kv.last_node.begin(), r.kv.last_node.end()),
                                   std::vector<std::uint32_t>(r.kv.matched_atoms.begin(), r.kv.matched_atoms.end()),
                                   r.mamba_node, r.mamba_atoms, r.mamba_slot);
           })
      .def("allocate_slot", &HybridPrefixCache::allocate_slot)
      .def("free_slot", &HybridPrefixCache::free_slot)
      .def("attach", &HybridPrefixCache::attach)
      .def("detach", &HybridPrefixCache::detach)
      .def("find_last_mamba_node", &HybridPrefixCache::find_last_mamba_node)
      .def("ensure_slots_by_evict", &HybridPrefixCache::ensure_slots_by_evict)
      .def_property_readonly("available_slots", &HybridPrefixCache::available_slots)
      .def_property_readonly("total_slots", &HybridPrefixCache::total_slots)
      .def_property_readonly("active_slots", &HybridPrefixCache::active_slots)
      .def_property_readonly("kv", &HybridPrefixCache::kv);

  py::class_<StorageBackend, std::shared_ptr<StorageBackend>>(m, "StorageBackend")
      .def_property_readonly("name", &StorageBackend::name)
      .def_property_readonly("unit_bytes", &StorageBackend::unit_bytes)
      .def("write", [](StorageBackend& s, std::uint64_t key, const py::bytes& b) { std::string keep = b; return s.write(key, keep); })
      .def("read", [](StorageBackend& s, std::uint64_t key) -> py::object {
             auto r = s.read(key);
             if (!r) return py::none();
             return py::bytes(*r);
           })
      .def("contains", &StorageBackend::contains)
      .def("erase", &StorageBackend::erase)
      .def("entries", &StorageBackend::entries)
      .def("drain", &StorageBackend::drain);
  m.def("memory_backend", &make_memory_backend);
  m.def("file_backend", &make_file_backend);
  m.def("hash64", [](const py::bytes& b, std::uint64_t seed) { std::string s = b; return hash_bytes(s.data(), s.size(), seed); },
        py::arg("data"), py::arg("seed") = 0);
}
