// The page pool and the prefix tree allocate nothing after construction.  Global operator new is replaced by a
// counting one; the counter must stay at zero across allocate / share / drop and match / insert / evict.
// (PrefixServe checks the same property of its core in tests/cpp/test_no_alloc.cpp.)
#include <cstdio>
#include <cstdlib>
#include <new>
#include <vector>

#include "block_manager.hpp"
#include "radix_tree.hpp"
#include "seq_tables.hpp"

static long g_allocations = 0;
static bool g_counting = false;

void* operator new(std::size_t n) {
  if (g_counting) ++g_allocations;
  if (void* p = std::malloc(n ? n : 1)) return p;
  throw std::bad_alloc();
}
void* operator new(std::size_t n, std::align_val_t a) {
  if (g_counting) ++g_allocations;
  void* p = nullptr;
  if (posix_memalign(&p, static_cast<std::size_t>(a) < sizeof(void*) ? sizeof(void*) : static_cast<std::size_t>(a), n ? n : 1) != 0)
    throw std::bad_alloc();
  return p;
}
void operator delete(void* p) noexcept { std::free(p); }
void operator delete(void* p, std::size_t) noexcept { std::free(p); }
void operator delete(void* p, std::align_val_t) noexcept { std::free(p); }
void operator delete(void* p, std::size_t, std::align_val_t) noexcept { std::free(p); }

#define CHECK(cond)                                                   \
  do {                                                                \
    if (!(cond)) {                                                    \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);   \
      return 1;                                                       \
    }                                                                 \
  } while (0)

int main() {
  using namespace psb200;
  // the counter itself counts
  g_counting = true;
  { std::vector<int> v(10); (void)v; }
  g_counting = false;
  CHECK(g_allocations == 1);
  g_allocations = 0;

  constexpr int kPages = 64, kPage = 16;
  BlockManager pool(kPages);
  RadixTree tree(pool, kPage, 42);
  std::vector<PageId> out;
  out.reserve(kPages);
  std::vector<int32_t> tokens(kPage * 8);
  std::vector<PageId> pages(8);
  std::string why;

  g_counting = true;
  unsigned rng = 1;
  for (int round = 0; round < 2000; ++round) {
    rng = rng * 1664525u + 1013904223u;
    const int blocks = 1 + (rng >> 8) % 8;
    for (int i = 0; i < blocks * kPage; ++i) tokens[i] = (int32_t)(((rng >> 4) % 5) * 1000 + i / kPage * 17 + i % 3);
    const int64_t matched = tree.match_prefix(tokens.data(), blocks * kPage, out);
    const int have = (int)out.size();
    for (int i = 0; i < have; ++i) pages[i] = out[i];
    int need = blocks - have;
    if (pool.num_free() < need) tree.evict(need - pool.num_free());
    if (!pool.take_many(need, pages.data() + have)) {
      for (int i = 0; i < have; ++i) (void)pool.drop(pages[i]);
      continue;
    }
    int32_t added = 0;
    (void)matched;
    if (tree.insert(tokens.data(), blocks * kPage, pages.data(), blocks, &added) != Code::ok) return 2;
    (void)pool.share(pages[0]);
    (void)pool.drop(pages[0]);
    for (int i = 0; i < blocks; ++i) (void)pool.drop(pages[i]);
    if (round % 7 == 0) tree.evict(3);
  }
  g_counting = false;
  CHECK(g_allocations == 0);

  // the slot pool, the page table rows, the slot records and their logs of changed words
  SlotPool slots(8);
  SeqTables tables(8, 32);
  SlotRecords records(8);
  std::vector<int32_t> pairs(2 * (8 * 32 + 8 * SlotRecords::kWords));
  PageId given[32];
  g_counting = true;
  for (int round = 0; round < 2000; ++round) {
    rng = rng * 1664525u + 1013904223u;
    const int32_t s = slots.take();
    if (s < 0) return 3;
    records.set_sampling(s, (float)(rng % 7) * 0.25f, rng);
    const PageId ids[3] = {(PageId)(rng % 64), (PageId)((rng >> 8) % 64), (PageId)((rng >> 16) % 64)};
    for (int k = 0; k < 1 + (int)(rng % 9); ++k) (void)tables.append(s, ids, 3);
    (void)tables.release_front(s, (int32_t)(rng % 5), given);
    if (round % 3 == 0) { (void)tables.drain(0, pairs.data()); (void)records.drain(0, pairs.data()); }
    (void)tables.clear(s, given);
    (void)slots.give_back(s);
  }
  g_counting = false;
  CHECK(g_allocations == 0);
  CHECK(pool.consistent(&why));
  CHECK(tree.consistent(&why));
  tree.evict(kPages);
  CHECK(pool.num_free() == kPages);
  std::printf("ok: no allocation in %d rounds\n", 2000);
  return 0;
}
