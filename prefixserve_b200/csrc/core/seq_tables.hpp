// Per-request bookkeeping that sits beside the page pool: a pool of request
// slots (each slot is one row of every per-request array on the device) and,
// for each cache group, one page table row per slot.
//
// The reference keeps a request's pages in a Python list on the request and
// flattens all lists on every step (prefixserve/scheduler.py:80,
// prefixserve/llama_engine.py:183-201).  Here the rows live in one flat int32
// array indexed by absolute page number, so a step's tables are a row gather,
// and a group that only needs a window of keys can hand back the pages the
// window has passed while later entries keep their index.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "block_manager.hpp"

namespace psb200 {

class SlotPool {
 public:
  explicit SlotPool(int32_t n) : n_(n) {
    if (n < 1) throw std::invalid_argument("num_slots must be >= 1");
    busy_.assign(static_cast<size_t>(n), 0);
    free_.reserve(static_cast<size_t>(n));
    for (int32_t s = n - 1; s >= 0; --s) free_.push_back(s);
  }
  int32_t take() noexcept {
    if (free_.empty()) return -1;
    const int32_t s = free_.back();
    free_.pop_back();
    busy_[static_cast<size_t>(s)] = 1;
    return s;
  }
  // false: slot out of range or not taken (released twice)
  bool give_back(int32_t s) noexcept {
    if (s < 0 || s >= n_ || !busy_[static_cast<size_t>(s)]) return false;
    busy_[static_cast<size_t>(s)] = 0;
    free_.push_back(s);
    return true;
  }
  bool taken(int32_t s) const noexcept { return s >= 0 && s < n_ && busy_[static_cast<size_t>(s)]; }
  int32_t num_free() const noexcept { return static_cast<int32_t>(free_.size()); }
  int32_t num_slots() const noexcept { return n_; }

 private:
  int32_t n_;
  std::vector<uint8_t> busy_;
  std::vector<int32_t> free_;
};

// rows[slot][page_index] = page id, or kNoPage where nothing is held.
class SeqTables {
 public:
  SeqTables(int32_t num_slots, int32_t max_pages) : slots_(num_slots), width_(max_pages) {
    if (num_slots < 1 || max_pages < 1) throw std::invalid_argument("num_slots and max_pages must be >= 1");
    rows_.assign(static_cast<size_t>(num_slots) * static_cast<size_t>(max_pages), kNoPage);
    begin_.assign(static_cast<size_t>(num_slots), 0);
    end_.assign(static_cast<size_t>(num_slots), 0);
  }

  int32_t num_slots() const noexcept { return slots_; }
  int32_t max_pages() const noexcept { return width_; }
  bool slot_ok(int32_t s) const noexcept { return s >= 0 && s < slots_; }
  int32_t first_live(int32_t s) const noexcept { return begin_[static_cast<size_t>(s)]; }
  int32_t length(int32_t s) const noexcept { return end_[static_cast<size_t>(s)]; }
  const PageId* row(int32_t s) const noexcept { return &rows_[static_cast<size_t>(s) * static_cast<size_t>(width_)]; }
  PageId* row(int32_t s) noexcept { return &rows_[static_cast<size_t>(s) * static_cast<size_t>(width_)]; }
  PageId* data() noexcept { return rows_.data(); }

  // Appends n page ids at the end of the row; false when the row is full.
  bool append(int32_t s, const PageId* ids, int32_t n) noexcept {
    int32_t& e = end_[static_cast<size_t>(s)];
    if (n < 0 || e + n > width_) return false;
    PageId* r = row(s);
    for (int32_t i = 0; i < n; ++i) r[e + i] = ids[i];
    e += n;
    return true;
  }

  // Takes the live entries with index < upto out of the row (they become
  // kNoPage) and writes them to out; returns how many.
  int32_t release_front(int32_t s, int32_t upto, PageId* out) noexcept {
    int32_t& b = begin_[static_cast<size_t>(s)];
    const int32_t e = end_[static_cast<size_t>(s)];
    if (upto > e) upto = e;
    PageId* r = row(s);
    int32_t n = 0;
    for (; b < upto; ++b) {
      if (r[b] != kNoPage) out[n++] = r[b];
      r[b] = kNoPage;
    }
    return n;
  }

  // Empties the row; the live ids go to out.
  int32_t clear(int32_t s, PageId* out) noexcept {
    const int32_t n = release_front(s, end_[static_cast<size_t>(s)], out);
    begin_[static_cast<size_t>(s)] = 0;
    end_[static_cast<size_t>(s)] = 0;
    return n;
  }

  // out[i*width + j] = rows[slots[i]][j] for j < width (dense block for one step)
  void gather(const int32_t* slots, int32_t n, int32_t width, PageId* out) const noexcept {
    const int32_t w = width < width_ ? width : width_;
    for (int32_t i = 0; i < n; ++i) {
      const PageId* r = row(slots[i]);
      PageId* o = out + static_cast<size_t>(i) * static_cast<size_t>(width);
      int32_t j = 0;
      for (; j < w; ++j) o[j] = r[j];
      for (; j < width; ++j) o[j] = kNoPage;
    }
  }

 private:
  int32_t slots_;
  int32_t width_;
  std::vector<PageId> rows_;
  std::vector<int32_t> begin_;
  std::vector<int32_t> end_;
};

}  // namespace psb200
