// Host-only check of tfb::QueueWords (csrc/registry.h): which work-item counter
// word a launch of the two-tile attention kernel gets.  Built and run by
// tests/test_cabi_cpu.py with the host compiler; no CUDA involved.
#include <cstdio>
#include <set>
#include <thread>
#include <vector>

#include "registry.h"

#define CHECK(cond)                                                  \
  do {                                                               \
    if (!(cond)) {                                                   \
      std::printf("FAILED line %d: %s\n", __LINE__, #cond);          \
      return 1;                                                      \
    }                                                                \
  } while (0)

int main() {
  using tfb::QueueWords;
  {
    QueueWords q;
    // a stream keeps its word, however many launches other streams make in between
    const int a = q.eager(0x1000), b = q.eager(0x2000);
    CHECK(a >= 0 && b >= 0 && a != b);
    for (int i = 0; i < 1000; ++i) CHECK(q.eager(0x2000) == b);
    CHECK(q.eager(0x1000) == a);
    CHECK(q.eager(0) >= 0 && q.eager(0) == q.eager(0));          // the legacy stream is a key like any other
    // captured launches never share a word, neither with each other nor with a stream
    std::set<int> seen = {a, b, q.eager(0)};
    for (int i = 0; i < QueueWords::kCapturedWords; ++i) {
      const int w = q.captured();
      CHECK(w >= QueueWords::kEagerWords && w < QueueWords::kWords);
      CHECK(seen.insert(w).second);
    }
    CHECK(q.captured() == -1);                                   // exhausted: reported, not recycled
    CHECK(q.eager(0x1000) == a);                                 // eager words are unaffected
  }
  {
    QueueWords q;
    std::set<int> seen;
    for (int i = 0; i < QueueWords::kEagerWords; ++i) {
      const int w = q.eager(0x100 + 8 * i);
      CHECK(w >= 0 && w < QueueWords::kEagerWords && seen.insert(w).second);
    }
    CHECK(q.eager(0xdead0) == -1);                               // table full: reported
    CHECK(q.eager(0x100) >= 0);                                  // known streams still resolve
  }
  {
    // concurrent callers (host threads launching on their own streams)
    QueueWords q;
    std::vector<int> got(64, -1);
    std::vector<std::thread> threads;
    for (int t = 0; t < 64; ++t)
      threads.emplace_back([&, t] {
        for (int i = 0; i < 200; ++i) got[t] = q.eager(0x4000 + 16 * t);
      });
    for (auto& th : threads) th.join();
    std::set<int> seen(got.begin(), got.end());
    CHECK(seen.size() == 64 && *seen.begin() >= 0);
  }
  std::printf("ok\n");
  return 0;
}
