// Python module prefixserve_b200.cache._core: the page pool, the prefix tree,
// the slot pool and the per-slot page tables.
//
// Calling conventions follow the reference's module (csrc/bindings.cpp:96-171
// of PrefixServe): integer arrays come in as anything convertible to a
// contiguous int32 array and are only borrowed for the call, results are fresh
// Python lists, a status other than ok becomes CoreError, malformed arguments
// become ValueError, and the tree keeps its pool alive.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "block_manager.hpp"
#include "radix_tree.hpp"
#include "seq_tables.hpp"

namespace py = pybind11;
using namespace psb200;

namespace {

struct CoreFailure : std::runtime_error {
  using std::runtime_error::runtime_error;
};

using IntArray = py::array_t<int32_t, py::array::c_style | py::array::forcecast>;

const int32_t* flat(const IntArray& a, const char* what, int64_t* n) {
  if (a.ndim() != 1) throw py::value_error(std::string(what) + " must be one-dimensional");
  *n = static_cast<int64_t>(a.shape(0));
  return a.data();
}

void require(Code c, const std::string& where = "") {
  if (c != Code::ok) throw CoreFailure(where.empty() ? describe(c) : where + ": " + describe(c));
}

py::list to_list(const std::vector<PageId>& v, size_t n) {
  py::list out(n);
  for (size_t i = 0; i < n; ++i) out[i] = py::int_(v[i]);
  return out;
}

// The tree plus a scratch vector sized once, so matching allocates nothing on
// the C++ side.
class TreeHandle {
 public:
  TreeHandle(BlockManager& pool, int32_t page_tokens, std::optional<uint64_t> seed)
      : tree_(pool, page_tokens, seed ? *seed : RadixTree::fresh_seed()) {
    scratch_.reserve(static_cast<size_t>(pool.num_blocks()));
  }
  RadixTree tree_;
  std::vector<PageId> scratch_;
};

}  // namespace

PYBIND11_MODULE(_core, m) {
  m.doc() = "page pool, prefix tree, request slots and page tables (host side)";
  m.attr("BLOCK_SIZE") = kDefaultPageTokens;
  py::register_exception<CoreFailure>(m, "CoreError", PyExc_RuntimeError);

  py::class_<BlockManager>(m, "BlockManager")
      .def(py::init([](int64_t n) {
             if (n < 1 || n > kPoolLimit) throw py::value_error("num_blocks must be in [1, 2**26]");
             return std::make_unique<BlockManager>(static_cast<int32_t>(n));
           }),
           py::arg("num_blocks"))
      .def("allocate",
           [](BlockManager& p) -> py::object {
             const PageId id = p.take();
             return id == kNoPage ? py::object(py::none()) : py::object(py::int_(id));
           })
      .def("allocate_many",
           [](BlockManager& p, int64_t n) -> py::object {
             if (n < 0) throw py::value_error("cannot allocate a negative number of blocks");
             if (n > p.num_free()) return py::none();
             std::vector<PageId> ids(static_cast<size_t>(n));
             p.take_many(static_cast<int32_t>(n), ids.data());
             return to_list(ids, ids.size());
           },
           py::arg("n"))
      .def("incref", [](BlockManager& p, int64_t id) { require(p.share(static_cast<PageId>(id))); }, py::arg("block_id"))
      .def("decref", [](BlockManager& p, int64_t id) { require(p.drop(static_cast<PageId>(id))); }, py::arg("block_id"))
      .def("decref_many",
           [](BlockManager& p, const IntArray& ids) {
             int64_t n = 0;
             const int32_t* d = flat(ids, "block_ids", &n);
             for (int64_t i = 0; i < n; ++i) require(p.drop(d[i]), "index " + std::to_string(i));
           },
           py::arg("block_ids"))
      .def("ref_count",
           [](const BlockManager& p, int64_t id) {
             if (!p.in_range(static_cast<PageId>(id))) throw CoreFailure(describe(Code::bad_id));
             return p.count(static_cast<PageId>(id));
           },
           py::arg("block_id"))
      .def_property_readonly("num_free", &BlockManager::num_free)
      .def_property_readonly("num_blocks", &BlockManager::num_blocks)
      .def("check_invariants", [](const BlockManager& p) {
        std::string why;
        if (!p.consistent(&why)) throw CoreFailure("block manager: " + why);
      });

  py::class_<TreeHandle>(m, "RadixTree")
      .def(py::init([](BlockManager& pool, int64_t block_size, std::optional<uint64_t> seed) {
             if (block_size < 1 || block_size > 4096) throw py::value_error("block_size must be in [1, 4096]");
             return std::make_unique<TreeHandle>(pool, static_cast<int32_t>(block_size), seed);
           }),
           py::arg("block_manager"), py::arg("block_size") = kDefaultPageTokens, py::arg("hash_seed") = py::none(),
           py::keep_alive<1, 2>())
      .def("match_prefix",
           [](TreeHandle& t, const IntArray& tokens) {
             int64_t n = 0;
             const int32_t* d = flat(tokens, "tokens", &n);
             const int64_t matched = t.tree_.match_prefix(d, n, t.scratch_);
             return py::make_tuple(matched, to_list(t.scratch_, t.scratch_.size()));
           },
           py::arg("tokens"))
      .def("insert",
           [](TreeHandle& t, const IntArray& tokens, const IntArray& blocks) {
             int64_t n = 0, nb = 0;
             const int32_t* d = flat(tokens, "tokens", &n);
             const int32_t* b = flat(blocks, "block_ids", &nb);
             if (nb < n / t.tree_.page_tokens()) throw py::value_error("fewer block ids than full blocks of tokens");
             int32_t added = 0;
             require(t.tree_.insert(d, n, b, nb, &added));
             return added;
           },
           py::arg("tokens"), py::arg("block_ids"))
      .def("evict",
           [](TreeHandle& t, int64_t want) {
             if (want < 0) throw py::value_error("cannot evict a negative number of blocks");
             return t.tree_.evict(static_cast<int32_t>(std::min<int64_t>(want, kPoolLimit)));
           },
           py::arg("num_blocks"))
      .def("is_cached", [](const TreeHandle& t, int64_t id) { return t.tree_.is_cached(static_cast<PageId>(id)); })
      .def_property_readonly("num_cached_blocks", [](const TreeHandle& t) { return t.tree_.num_cached_blocks(); })
      .def_property_readonly("block_size", [](const TreeHandle& t) { return t.tree_.page_tokens(); })
      .def("check_invariants", [](const TreeHandle& t) {
        std::string why;
        if (!t.tree_.consistent(&why)) throw CoreFailure("radix tree: " + why);
      });

  py::class_<SlotPool>(m, "SlotPool")
      .def(py::init([](int64_t n) {
             if (n < 1 || n > (1 << 24)) throw py::value_error("num_slots must be in [1, 2**24]");
             return std::make_unique<SlotPool>(static_cast<int32_t>(n));
           }),
           py::arg("num_slots"))
      .def("take",
           [](SlotPool& p) -> py::object {
             const int32_t s = p.take();
             return s < 0 ? py::object(py::none()) : py::object(py::int_(s));
           })
      .def("give_back",
           [](SlotPool& p, int64_t s) {
             if (!p.give_back(static_cast<int32_t>(s))) throw CoreFailure("slot " + std::to_string(s) + " is not taken (released twice?)");
           },
           py::arg("slot"))
      .def("taken", [](const SlotPool& p, int64_t s) { return p.taken(static_cast<int32_t>(s)); })
      .def_property_readonly("num_free", &SlotPool::num_free)
      .def_property_readonly("num_slots", &SlotPool::num_slots);

  py::class_<SlotRecords>(m, "SlotRecords")
      .def(py::init([](int64_t n) {
             if (n < 1 || n > (1 << 24)) throw py::value_error("num_slots must be in [1, 2**24]");
             return std::make_unique<SlotRecords>(static_cast<int32_t>(n));
           }),
           py::arg("num_slots"))
      .def_property_readonly("num_slots", &SlotRecords::num_slots)
      .def_property_readonly_static("WORDS", [](py::object) { return SlotRecords::kWords; })
      .def("view",
           [](py::object self) {
             auto& r = self.cast<SlotRecords&>();
             // int32 [num_slots, WORDS] over the records themselves; the array keeps the object alive
             return py::array_t<int32_t>({static_cast<py::ssize_t>(r.num_slots()), static_cast<py::ssize_t>(SlotRecords::kWords)},
                                         r.data(), self);
           })
      .def("set_sampling",
           [](SlotRecords& r, int64_t s, double temperature, uint64_t seed) {
             if (!r.slot_ok(static_cast<int32_t>(s))) throw py::value_error("slot out of range");
             r.set_sampling(static_cast<int32_t>(s), static_cast<float>(temperature), seed);
           },
           py::arg("slot"), py::arg("temperature"), py::arg("seed"))
      .def_property_readonly("pending", &SlotRecords::pending)
      .def("drain",
           [](SlotRecords& r, int64_t base, py::array_t<int32_t, py::array::c_style> out, int64_t at) {
             if (at < 0 || out.size() < at + 2 * static_cast<int64_t>(r.pending())) throw py::value_error("output array is too small");
             return r.drain(static_cast<int32_t>(base), out.mutable_data() + at);
           },
           py::arg("base"), py::arg("out"), py::arg("at"));

  py::class_<SeqTables>(m, "SeqTables")
      .def(py::init([](int64_t slots, int64_t pages) {
             if (slots < 1 || pages < 1 || slots * pages > (int64_t{1} << 31)) throw py::value_error("bad table shape");
             return std::make_unique<SeqTables>(static_cast<int32_t>(slots), static_cast<int32_t>(pages));
           }),
           py::arg("num_slots"), py::arg("max_pages"))
      .def_property_readonly("num_slots", &SeqTables::num_slots)
      .def_property_readonly("max_pages", &SeqTables::max_pages)
      .def("length",
           [](const SeqTables& t, int64_t s) {
             if (!t.slot_ok(static_cast<int32_t>(s))) throw py::value_error("slot out of range");
             return t.length(static_cast<int32_t>(s));
           })
      .def("first_live",
           [](const SeqTables& t, int64_t s) {
             if (!t.slot_ok(static_cast<int32_t>(s))) throw py::value_error("slot out of range");
             return t.first_live(static_cast<int32_t>(s));
           })
      .def("append",
           [](SeqTables& t, int64_t s, const IntArray& ids) {
             if (!t.slot_ok(static_cast<int32_t>(s))) throw py::value_error("slot out of range");
             int64_t n = 0;
             const int32_t* d = flat(ids, "block_ids", &n);
             if (!t.append(static_cast<int32_t>(s), d, static_cast<int32_t>(n))) {
               throw CoreFailure("page table row of slot " + std::to_string(s) + " is full");
             }
           },
           py::arg("slot"), py::arg("block_ids"))
      .def("release_front",
           [](SeqTables& t, int64_t s, int64_t upto) {
             if (!t.slot_ok(static_cast<int32_t>(s))) throw py::value_error("slot out of range");
             std::vector<PageId> out(static_cast<size_t>(t.max_pages()));
             const int32_t n = t.release_front(static_cast<int32_t>(s), static_cast<int32_t>(std::max<int64_t>(upto, 0)), out.data());
             return to_list(out, static_cast<size_t>(n));
           },
           py::arg("slot"), py::arg("upto_page"))
      .def("clear",
           [](SeqTables& t, int64_t s) {
             if (!t.slot_ok(static_cast<int32_t>(s))) throw py::value_error("slot out of range");
             std::vector<PageId> out(static_cast<size_t>(t.max_pages()));
             const int32_t n = t.clear(static_cast<int32_t>(s), out.data());
             return to_list(out, static_cast<size_t>(n));
           },
           py::arg("slot"))
      .def("row",
           [](const SeqTables& t, int64_t s) {
             if (!t.slot_ok(static_cast<int32_t>(s))) throw py::value_error("slot out of range");
             const int32_t n = t.length(static_cast<int32_t>(s));
             py::list out(static_cast<size_t>(n));
             for (int32_t i = 0; i < n; ++i) out[static_cast<size_t>(i)] = py::int_(t.row(static_cast<int32_t>(s))[i]);
             return out;
           },
           py::arg("slot"))
      .def_property_readonly("pending", &SeqTables::pending)
      .def("drain",
           [](SeqTables& t, int64_t base, py::array_t<int32_t, py::array::c_style> out, int64_t at) {
             if (at < 0 || out.size() < at + 2 * static_cast<int64_t>(t.pending())) throw py::value_error("output array is too small");
             return t.drain(static_cast<int32_t>(base), out.mutable_data() + at);
           },
           py::arg("base"), py::arg("out"), py::arg("at"))
      .def("covered",
           [](const SeqTables& t, const IntArray& slots, const IntArray& first, const IntArray& upto, int64_t num_pages) {
             // index of the first slot whose row lacks a valid page id somewhere in [first, upto); -1 when all are whole
             int64_t n = 0, nf = 0, nu = 0;
             const int32_t* s = flat(slots, "slots", &n);
             const int32_t* f = flat(first, "first", &nf);
             const int32_t* u = flat(upto, "upto", &nu);
             if (nf != n || nu != n) throw py::value_error("slots, first and upto must have one entry per item");
             for (int64_t i = 0; i < n; ++i) {
               if (!t.slot_ok(s[i])) throw py::value_error("slot out of range");
               if (!t.covered(s[i], f[i], u[i], static_cast<int32_t>(num_pages))) return i;
             }
             return int64_t{-1};
           },
           py::arg("slots"), py::arg("first"), py::arg("upto"), py::arg("num_pages"))
      .def("gather",
           [](const SeqTables& t, const IntArray& slots, int64_t width, py::array_t<int32_t, py::array::c_style> out) {
             int64_t n = 0;
             const int32_t* s = flat(slots, "slots", &n);
             for (int64_t i = 0; i < n; ++i) {
               if (!t.slot_ok(s[i])) throw py::value_error("slot out of range");
             }
             if (width < 0 || out.size() < n * width) throw py::value_error("output array is too small");
             t.gather(s, static_cast<int32_t>(n), static_cast<int32_t>(width), out.mutable_data());
           },
           py::arg("slots"), py::arg("width"), py::arg("out"));
}
