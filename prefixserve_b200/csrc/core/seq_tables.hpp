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
//
// The rows and the slot records are mirrors of arrays that stay on the device
// for the life of the engine.  Each keeps a log of the words that changed
// since the device last saw them; a step sends only those (index, value)
// pairs, so a step that appends no page uploads no table at all.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "block_manager.hpp"

namespace psb200 {

// Which words of a mirrored int32 array the device has not seen yet.  An index is logged once however often it is
// written; drain() reads the values current at that moment.  Capacity equals the array, so the log cannot overflow
// and nothing allocates after construction.
class DeltaLog {
 public:
  explicit DeltaLog(int64_t words) {
    dirty_.assign(static_cast<size_t>(words), 0);
    order_.reserve(static_cast<size_t>(words));
  }
  void touch(int64_t index) noexcept {
    uint8_t& d = dirty_[static_cast<size_t>(index)];
    if (!d) {
      d = 1;
      order_.push_back(static_cast<int32_t>(index));
    }
  }
  int32_t pending() const noexcept { return static_cast<int32_t>(order_.size()); }
  // Writes (base + index, value) pairs to out (room for 2 * pending() words) and empties the log.
  int32_t drain(const int32_t* mirror, int32_t base, int32_t* out) noexcept {
    const int32_t n = pending();
    for (int32_t i = 0; i < n; ++i) {
      const int32_t at = order_[static_cast<size_t>(i)];
      out[2 * i] = base + at;
      out[2 * i + 1] = mirror[at];
      dirty_[static_cast<size_t>(at)] = 0;
    }
    order_.clear();
    return n;
  }

 private:
  std::vector<uint8_t> dirty_;
  std::vector<int32_t> order_;
};

// One fixed-size record per request slot, kept on the device and mirrored here: the position (tokens computed; the
// device writes its own copy each step, so the host's is not sent), the sampling temperature and the sampling seed.
class SlotRecords {
 public:
  static constexpr int32_t kWords = 4;  // position, temperature (float bits), seed low, seed high
  enum Word : int32_t { kPosition = 0, kTemperature = 1, kSeedLow = 2, kSeedHigh = 3 };

  explicit SlotRecords(int32_t num_slots) : slots_(num_slots), log_(static_cast<int64_t>(num_slots) * kWords) {
    if (num_slots < 1) throw std::invalid_argument("num_slots must be >= 1");
    words_.assign(static_cast<size_t>(num_slots) * kWords, 0);
  }
  int32_t num_slots() const noexcept { return slots_; }
  bool slot_ok(int32_t s) const noexcept { return s >= 0 && s < slots_; }
  int32_t* data() noexcept { return words_.data(); }
  int32_t position(int32_t s) const noexcept { return words_[static_cast<size_t>(s) * kWords + kPosition]; }
  void set_position(int32_t s, int32_t p) noexcept { words_[static_cast<size_t>(s) * kWords + kPosition] = p; }
  void set_sampling(int32_t s, float temperature, uint64_t seed) noexcept {
    int32_t t;
    static_assert(sizeof(t) == sizeof(temperature), "float must be 32 bits");
    __builtin_memcpy(&t, &temperature, sizeof(t));
    put(s, kTemperature, t);
    put(s, kSeedLow, static_cast<int32_t>(static_cast<uint32_t>(seed)));
    put(s, kSeedHigh, static_cast<int32_t>(static_cast<uint32_t>(seed >> 32)));
  }
  int32_t pending() const noexcept { return log_.pending(); }
  int32_t drain(int32_t base, int32_t* out) noexcept { return log_.drain(words_.data(), base, out); }

 private:
  void put(int32_t s, int32_t word, int32_t value) noexcept {
    const int64_t at = static_cast<int64_t>(s) * kWords + word;
    if (words_[static_cast<size_t>(at)] != value) {
      words_[static_cast<size_t>(at)] = value;
      log_.touch(at);
    }
  }
  int32_t slots_;
  std::vector<int32_t> words_;
  DeltaLog log_;
};

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
  SeqTables(int32_t num_slots, int32_t max_pages)
      : slots_(num_slots), width_(max_pages),
        log_(num_slots < 1 || max_pages < 1 ? 0 : static_cast<int64_t>(num_slots) * max_pages) {
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
    const int64_t base = static_cast<int64_t>(s) * width_;
    for (int32_t i = 0; i < n; ++i) {
      r[e + i] = ids[i];
      log_.touch(base + e + i);
    }
    e += n;
    return true;
  }

  // Entries the device has not seen.  Only appended ids are sent: an entry given back (kNoPage here) keeps its old
  // id on the device, where nothing reads it any more: kernels read the entries [first needed, pages held) of the
  // slots a step names, and covered() has vouched for those.
  int32_t pending() const noexcept { return log_.pending(); }
  int32_t drain(int32_t base, int32_t* out) noexcept { return log_.drain(rows_.data(), base, out); }

  // True when slot s holds a valid page id (below num_pages) at every index in [first, upto).
  bool covered(int32_t s, int32_t first, int32_t upto, int32_t num_pages) const noexcept {
    if (first < 0) first = 0;
    if (upto > end_[static_cast<size_t>(s)]) return false;
    const PageId* r = row(s);
    for (int32_t j = first; j < upto; ++j) {
      if (r[j] < 0 || r[j] >= num_pages) return false;
    }
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
  DeltaLog log_;
};

}  // namespace psb200
