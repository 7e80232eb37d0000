// Host-only run of the KV swap tier and the LRU slot map (the "device" pointers are host pointers, copies are memcpy):
// built with AddressSanitizer + UndefinedBehaviorSanitizer by tests/test_host_sanitizers.py. No CUDA call is made at run
// time; the CUDA runtime is linked only because the same sources also hold the device paths.
#include <cstdio>
#include <cstring>
#include <numeric>
#include <stdexcept>
#include <vector>

#include "../engine/kv_swap.hpp"
#include "../engine/staging.hpp"

// The device scatter kernel lives in the kernel library; the host-only mode never reaches it.
extern "C" int pk_scatter_rows(const void*, const int*, int, int, void*, cudaStream_t) { return -1; }

#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::fprintf(stderr, "%s:%d: CHECK(%s) failed\n", __FILE__, __LINE__, #cond); \
      return 1;                                                            \
    }                                                                      \
  } while (0)

static int test_lru() {
  pk::LruSlotMap lru(3);
  std::vector<std::pair<long long, int>> loads;
  std::vector<int> s = lru.assign({10, 11, 10, 12}, &loads);
  CHECK(s.size() == 4 && s[0] == s[2] && loads.size() == 3 && lru.resident() == 3 && lru.misses == 3);
  loads.clear();                                    // assign() appends
  s = lru.assign({11, 13}, &loads);                 // 13 evicts the least recently used key that this step does not need
  CHECK(loads.size() == 1 && loads[0].first == 13 && lru.contains(11) && lru.contains(13) && lru.evictions == 1 && lru.hits == 1);
  CHECK(!lru.contains(10));
  bool threw = false;
  try {
    lru.assign({1, 2, 3, 4}, &loads);
  } catch (const std::runtime_error&) {
    threw = true;
  }
  CHECK(threw);
  return 0;
}

static int test_tier() {
  const int capacity = 64, slots = 8, window = 5;
  const size_t row = 48;
  pk::KvSwapTier tier(capacity, slots, row, window, true);
  std::vector<uint8_t> rows((size_t)capacity * row);
  for (size_t i = 0; i < rows.size(); ++i) rows[i] = (uint8_t)((i / row) * 3 + (i % row));
  tier.store(0, 40, rows.data(), nullptr);
  tier.store(40, 24, rows.data() + 40 * row, nullptr);
  CHECK(tier.stored_rows() == 64 && tier.host_bytes() == (size_t)capacity * row);
  std::vector<uint8_t> pool((size_t)slots * row, 0xee);
  for (int step = 0; step < 20; ++step) {
    std::vector<int> sel = {(step * 7) % 64, (step * 7 + 1) % 64, -1, (step * 3) % 64, 63 - step, (step * 7) % 64};
    std::vector<int> phys(sel.size(), -7);
    tier.swap_in(sel.data(), (int)sel.size(), pool.data(), phys.data(), nullptr);
    for (size_t i = 0; i < sel.size(); ++i) {
      if (sel[i] < 0) {
        CHECK(phys[i] == -1);
        continue;
      }
      CHECK(phys[i] >= window && phys[i] < window + slots);
      CHECK(std::memcmp(pool.data() + (size_t)(phys[i] - window) * row, rows.data() + (size_t)sel[i] * row, row) == 0);
    }
  }
  CHECK(tier.stats().steps == 20 && tier.stats().hits > 0 && tier.stats().misses > 0 && tier.stats().evictions > 0);
  std::vector<int> many(slots + 1), phys(slots + 1);
  std::iota(many.begin(), many.end(), 0);
  bool threw = false;
  try {
    tier.swap_in(many.data(), (int)many.size(), pool.data(), phys.data(), nullptr);    // more distinct rows than slots
  } catch (const std::runtime_error&) {
    threw = true;
  }
  CHECK(threw);
  tier.reset();
  CHECK(tier.stored_rows() == 0);
  int one = 3, p = 0;
  threw = false;
  try {
    tier.swap_in(&one, 1, pool.data(), &p, nullptr);                                    // a row that was never stored
  } catch (const std::runtime_error&) {
    threw = true;
  }
  CHECK(threw);
  return 0;
}

int main() {
  try {
    if (test_lru()) return 1;
    if (test_tier()) return 1;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "host_swap_selftest: unexpected exception: %s\n", e.what());
    return 1;
  }
  std::printf("host_swap_selftest=ok\n");
  return 0;
}
