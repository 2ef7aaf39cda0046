// Fixed pool of cache page ids with reference counts.
//
// Observable behaviour follows the reference's pool (csrc/block_manager.hpp:49-119
// of PrefixServe): ids 0..n-1, the first allocation returns 0, freed ids come
// back last-in-first-out, a page returns to the pool only when its count drops
// to zero, and dropping a count that is already zero is always refused (a
// double free would hand one page to two requests).  Pool sizes outside
// [1, 2^26] are refused at construction.  After construction nothing allocates.
//
// Single-threaded by contract: one scheduler owns it.
#pragma once

#include <cstdint>
#include <limits>
#include <stdexcept>
#include <string>
#include <vector>

namespace psb200 {

using PageId = int32_t;

constexpr int32_t kDefaultPageTokens = 16;
constexpr PageId kNoPage = -1;
constexpr int32_t kPoolLimit = 1 << 26;

enum class Code : uint8_t {
  ok = 0,
  bad_id,         // id outside [0, n)
  not_held,       // count already zero: double free or use after free
  count_overflow,
  already_cached, // page is owned by a prefix-tree node already
  no_nodes,       // prefix tree ran out of nodes (an invariant broke)
  bad_argument,
};

inline const char* describe(Code c) noexcept {
  switch (c) {
    case Code::ok: return "ok";
    case Code::bad_id: return "block id out of range";
    case Code::not_held: return "block is not allocated (double free or use after free)";
    case Code::count_overflow: return "reference count overflow";
    case Code::already_cached: return "block is already owned by the prefix cache";
    case Code::no_nodes: return "prefix cache has no free node";
    case Code::bad_argument: return "invalid argument";
  }
  return "unknown";
}

class BlockManager {
 public:
  explicit BlockManager(int32_t n) : n_(n) {
    if (n < 1 || n > kPoolLimit) {
      throw std::invalid_argument("num_blocks must be in [1, " + std::to_string(kPoolLimit) + "], got " +
                                  std::to_string(n));
    }
    count_.assign(static_cast<size_t>(n), 0);
    free_.reserve(static_cast<size_t>(n));
    // Filled from the top so that popping the back yields 0, 1, 2, ...
    for (PageId id = n - 1; id >= 0; --id) free_.push_back(id);
  }
  BlockManager(const BlockManager&) = delete;
  BlockManager& operator=(const BlockManager&) = delete;

  // A page with count 1, or kNoPage when none is free (not an error: the
  // caller evicts or preempts).
  PageId take() noexcept {
    if (free_.empty()) return kNoPage;
    const PageId id = free_.back();
    free_.pop_back();
    count_[static_cast<size_t>(id)] = 1;
    return id;
  }

  // All-or-nothing: writes n ids to out, or takes none and returns false.
  bool take_many(int32_t n, PageId* out) noexcept {
    if (n < 0 || static_cast<size_t>(n) > free_.size()) return false;
    for (int32_t i = 0; i < n; ++i) out[i] = take();
    return true;
  }

  Code share(PageId id) noexcept {
    if (!in_range(id)) return Code::bad_id;
    int32_t& c = count_[static_cast<size_t>(id)];
    if (c == 0) return Code::not_held;
    if (c == std::numeric_limits<int32_t>::max()) return Code::count_overflow;
    ++c;
    return Code::ok;
  }

  Code drop(PageId id) noexcept {
    if (!in_range(id)) return Code::bad_id;
    int32_t& c = count_[static_cast<size_t>(id)];
    if (c == 0) return Code::not_held;
    if (--c == 0) free_.push_back(id);  // capacity reserved above
    return Code::ok;
  }

  // 0 = free, -1 = id out of range.
  int32_t count(PageId id) const noexcept { return in_range(id) ? count_[static_cast<size_t>(id)] : -1; }
  bool in_range(PageId id) const noexcept { return id >= 0 && id < n_; }
  int32_t num_free() const noexcept { return static_cast<int32_t>(free_.size()); }
  int32_t num_blocks() const noexcept { return n_; }

  // Full consistency check (tests): every id is either on the free list once
  // with count zero, or off it with a positive count.
  bool consistent(std::string* why) const {
    std::vector<uint8_t> seen(static_cast<size_t>(n_), 0);
    for (PageId id : free_) {
      if (!in_range(id)) return fail(why, "free list holds an id out of range");
      if (seen[static_cast<size_t>(id)]++) return fail(why, "block " + std::to_string(id) + " is on the free list twice");
      if (count_[static_cast<size_t>(id)] != 0) return fail(why, "free block " + std::to_string(id) + " has a count");
    }
    for (PageId id = 0; id < n_; ++id) {
      const int32_t c = count_[static_cast<size_t>(id)];
      if (c < 0) return fail(why, "negative count");
      if (c == 0 && !seen[static_cast<size_t>(id)]) return fail(why, "block " + std::to_string(id) + " is lost");
    }
    return true;
  }

 private:
  static bool fail(std::string* why, std::string msg) {
    if (why) *why = std::move(msg);
    return false;
  }
  int32_t n_;
  std::vector<int32_t> count_;
  std::vector<PageId> free_;
};

}  // namespace psb200
