// The cases the host core must get right, as a plain C++ program so that it can be built with
// -fsanitize=address,undefined: the page pool (ids in order, last-in-first-out reuse, counts, refused double free),
// the prefix tree (whole pages only, verified hits, all-or-nothing insert, the tree keeps its copy of duplicate
// content, least-recently-used eviction that spares pages in use, a parent following its last child, the destructor
// giving references back), the slot pool, the page table rows and the logs of changed words.
// (PrefixServe pins the same behaviour of its own core in tests/cpp/test_core.cpp with a test framework that cannot
// be fetched here; its CMakeLists.txt:50-54 offers the sanitizer build this file is meant for.)
#include <cstdio>
#include <cstring>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "block_manager.hpp"
#include "radix_tree.hpp"
#include "seq_tables.hpp"

using namespace psb200;

static int g_failures = 0;
#define CHECK(cond)                                                 \
  do {                                                              \
    if (!(cond)) {                                                  \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++g_failures;                                                 \
    }                                                               \
  } while (0)

static std::vector<int32_t> run(int n, int base) {
  std::vector<int32_t> v(static_cast<size_t>(n));
  for (int i = 0; i < n; ++i) v[static_cast<size_t>(i)] = base + i;
  return v;
}

static void pool_cases() {
  BlockManager pool(4);
  CHECK(pool.take() == 0 && pool.take() == 1 && pool.take() == 2);
  CHECK(pool.drop(1) == Code::ok && pool.take() == 1);            // last freed, first reused
  CHECK(pool.share(2) == Code::ok && pool.count(2) == 2);
  CHECK(pool.drop(2) == Code::ok && pool.drop(2) == Code::ok && pool.count(2) == 0);
  CHECK(pool.drop(2) == Code::not_held);                          // a double free is refused, never silent
  CHECK(pool.share(2) == Code::not_held && pool.share(9) == Code::bad_id && pool.drop(-1) == Code::bad_id);
  PageId ids[4];
  CHECK(!pool.take_many(3, ids) && pool.num_free() == 2);         // all or nothing
  CHECK(pool.take_many(2, ids) && pool.num_free() == 0 && pool.take() == kNoPage);
  std::string why;
  CHECK(pool.consistent(&why));
  bool threw = false;
  try { BlockManager bad(0); } catch (const std::invalid_argument&) { threw = true; }
  CHECK(threw);
}

static void tree_cases() {
  constexpr int kPage = 4;
  BlockManager pool(8);
  std::string why;
  {
    RadixTree tree(pool, kPage, 7);
    std::vector<PageId> out;
    auto a = run(10, 100);                                        // two full pages and a tail
    PageId pa[3];
    CHECK(pool.take_many(3, pa));
    int32_t added = -1;
    CHECK(tree.insert(a.data(), 10, pa, 3, &added) == Code::ok && added == 2);   // the partial page is ignored
    CHECK(tree.is_cached(pa[0]) && tree.is_cached(pa[1]) && !tree.is_cached(pa[2]) && pool.count(pa[0]) == 2);
    CHECK(tree.insert(a.data(), 10, pa, 1, &added) == Code::bad_argument);       // fewer ids than full pages
    CHECK(tree.match_prefix(a.data(), 10, out) == 8 && out.size() == 2 && out[0] == pa[0] && out[1] == pa[1]);
    CHECK(pool.count(pa[0]) == 3);                                // one reference per returned page for the caller
    CHECK(pool.drop(pa[0]) == Code::ok && pool.drop(pa[1]) == Code::ok);
    CHECK(tree.match_prefix(a.data(), 7, out) == 4 && out.size() == 1);          // whole pages only
    CHECK(pool.drop(out[0]) == Code::ok);
    auto b = a;
    b[5] = -3;                                                    // same first page, other second page
    CHECK(tree.match_prefix(b.data(), 8, out) == 4);
    CHECK(pool.drop(out[0]) == Code::ok);
    // the same content under other page ids: the tree keeps its copy, adopts nothing
    PageId dup[2];
    CHECK(pool.take_many(2, dup));
    CHECK(tree.insert(a.data(), 8, dup, 2, &added) == Code::ok && added == 0 && !tree.is_cached(dup[0]));
    // a page already in the tree cannot come in again under other tokens; nothing of the call stays
    auto c = run(8, 900);
    PageId mixed[2] = {dup[0], pa[1]};
    const int32_t cached_before = tree.num_cached_blocks();
    CHECK(tree.insert(c.data(), 8, mixed, 2, &added) == Code::already_cached);
    CHECK(tree.num_cached_blocks() == cached_before && !tree.is_cached(dup[0]) && pool.count(dup[0]) == 1);
    PageId twice[2] = {dup[0], dup[0]};
    CHECK(tree.insert(c.data(), 8, twice, 2, &added) != Code::ok && !tree.is_cached(dup[0]));
    CHECK(pool.drop(dup[0]) == Code::ok && pool.drop(dup[1]) == Code::ok);
    // least recently used first; pages somebody holds are spared; a parent follows its last child
    CHECK(pool.drop(pa[2]) == Code::ok);
    auto d = run(4, 500);
    PageId pd[1];
    CHECK(pool.take_many(1, pd));
    CHECK(tree.insert(d.data(), 4, pd, 1, &added) == Code::ok && added == 1);
    CHECK(tree.match_prefix(a.data(), 8, out) == 8);              // touches a's path: d is now the oldest leaf
    CHECK(pool.drop(out[0]) == Code::ok && pool.drop(out[1]) == Code::ok);
    CHECK(tree.evict(1) == 0);                                    // d is still held by its request, a's leaf too
    CHECK(pool.drop(pd[0]) == Code::ok);
    CHECK(tree.evict(1) == 1 && !tree.is_cached(pd[0]) && tree.is_cached(pa[1]));
    CHECK(pool.drop(pa[0]) == Code::ok && pool.drop(pa[1]) == Code::ok);
    CHECK(tree.evict(5) == 2 && tree.num_cached_blocks() == 0);   // the leaf, then its parent in the same call
    CHECK(pool.num_free() == 8 && tree.consistent(&why) && pool.consistent(&why));
    // what is left in the tree when it dies goes back to the pool
    CHECK(pool.take_many(2, pa));
    CHECK(tree.insert(a.data(), 8, pa, 2, &added) == Code::ok && added == 2);
    CHECK(pool.drop(pa[0]) == Code::ok && pool.drop(pa[1]) == Code::ok && pool.num_free() == 6);
  }
  CHECK(pool.num_free() == 8 && pool.consistent(&why));
}

// Random traffic against a model that counts holders: no page lost, none held by mistake.
static void tree_random(unsigned seed) {
  constexpr int kPage = 3, kPages = 24;
  BlockManager pool(kPages);
  RadixTree tree(pool, kPage, seed);
  std::mt19937 rng(seed);
  std::vector<PageId> out;
  std::vector<std::vector<PageId>> held;   // what "requests" hold
  std::string why;
  for (int round = 0; round < 3000; ++round) {
    const int kind = static_cast<int>(rng() % 10);
    if (kind < 5) {
      const int pages = 1 + static_cast<int>(rng() % 4);
      std::vector<int32_t> toks(static_cast<size_t>(pages * kPage + rng() % kPage));
      const int family = static_cast<int>(rng() % 3);
      for (size_t i = 0; i < toks.size(); ++i) toks[i] = family * 50 + static_cast<int32_t>(i / kPage) * (1 + static_cast<int>(rng() % 2));
      const int64_t matched = tree.match_prefix(toks.data(), static_cast<int64_t>(toks.size()), out);
      std::vector<PageId> mine(out.begin(), out.end());
      const int need = pages - static_cast<int>(mine.size());
      if (pool.num_free() < need) tree.evict(need - pool.num_free());
      std::vector<PageId> fresh(static_cast<size_t>(need));
      if (!pool.take_many(need, fresh.data())) {
        for (PageId p : mine) CHECK(pool.drop(p) == Code::ok);
        continue;
      }
      mine.insert(mine.end(), fresh.begin(), fresh.end());
      int32_t added = 0;
      CHECK(tree.insert(toks.data(), static_cast<int64_t>(toks.size()), mine.data(), pages, &added) == Code::ok);
      CHECK(added <= need && matched % kPage == 0);
      held.push_back(mine);
    } else if (kind < 9 && !held.empty()) {
      const size_t at = rng() % held.size();
      for (PageId p : held[at]) CHECK(pool.drop(p) == Code::ok);
      held.erase(held.begin() + static_cast<long>(at));
    } else {
      tree.evict(static_cast<int32_t>(rng() % 5));
    }
    if (round % 50 == 0) {
      std::vector<int> holders(kPages, 0);
      for (const auto& h : held) for (PageId p : h) ++holders[static_cast<size_t>(p)];
      for (PageId p = 0; p < kPages; ++p) CHECK(pool.count(p) == holders[static_cast<size_t>(p)] + (tree.is_cached(p) ? 1 : 0));
      CHECK(tree.consistent(&why) && pool.consistent(&why));
    }
  }
  for (const auto& h : held) for (PageId p : h) CHECK(pool.drop(p) == Code::ok);
  tree.evict(kPages);
  CHECK(pool.num_free() == kPages);
}

static void slot_and_table_cases() {
  SlotPool slots(3);
  CHECK(slots.take() == 0 && slots.take() == 1 && slots.take() == 2 && slots.take() == -1);
  CHECK(slots.give_back(1) && !slots.give_back(1) && !slots.give_back(7) && slots.taken(0) && !slots.taken(1));
  CHECK(slots.take() == 1);

  SeqTables tables(3, 6);
  const PageId ids[4] = {9, 4, 7, 2};
  CHECK(tables.append(1, ids, 4) && tables.length(1) == 4 && tables.pending() == 4);
  CHECK(tables.covered(1, 0, 4, 10) && !tables.covered(1, 0, 5, 10) && !tables.covered(1, 0, 4, 9));
  std::vector<int32_t> device(3 * 6, -1), pairs(2 * 18);
  auto send = [&] {
    const int32_t n = tables.drain(0, pairs.data());
    for (int32_t i = 0; i < n; ++i) device[static_cast<size_t>(pairs[2 * i])] = pairs[2 * i + 1];
    return n;
  };
  CHECK(send() == 4 && tables.pending() == 0 && device[6] == 9 && device[9] == 2);
  PageId out[6];
  CHECK(tables.release_front(1, 2, out) == 2 && out[0] == 9 && out[1] == 4 && tables.first_live(1) == 2);
  CHECK(!tables.covered(1, 0, 4, 10) && tables.covered(1, 2, 4, 10) && tables.pending() == 0);   // given back: not sent
  const PageId more[3] = {5, 5, 5};
  CHECK(!tables.append(1, more, 3) && tables.append(1, more, 2) && tables.pending() == 2);       // a full row refuses
  CHECK(tables.clear(1, out) == 4 && tables.length(1) == 0);
  const PageId again[1] = {3};
  CHECK(tables.append(1, again, 1));                               // the slot's next request
  CHECK(send() == 3 && device[6] == 3);                            // index 6 once, with the value it has now
  CHECK(tables.row(1)[0] == 3 && tables.row(1)[1] == kNoPage);

  SlotRecords records(2);
  records.set_sampling(1, 0.5f, 0x0123456789abcdefULL);
  CHECK(records.pending() == 3);
  records.set_sampling(1, 0.5f, 0x0123456789abcdefULL);            // nothing changed: nothing more to send
  CHECK(records.pending() == 3);
  records.set_position(1, 44);                                     // the device writes its own: not sent
  CHECK(records.pending() == 3 && records.position(1) == 44);
  std::vector<int32_t> rec(16);
  CHECK(records.drain(100, rec.data()) == 3 && rec[0] == 100 + 4 + 1 && records.pending() == 0);
  float t;
  std::memcpy(&t, &rec[1], sizeof(t));
  CHECK(t == 0.5f && static_cast<uint32_t>(rec[3]) == 0x89abcdefu && static_cast<uint32_t>(rec[5]) == 0x01234567u);
}

int main() {
  pool_cases();
  tree_cases();
  for (unsigned seed = 1; seed <= 4; ++seed) tree_random(seed);
  slot_and_table_cases();
  if (g_failures) {
    std::printf("%d checks failed\n", g_failures);
    return 1;
  }
  std::printf("ok: host core cases\n");
  return 0;
}
