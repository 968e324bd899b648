// Small host utilities of the runtime.
#pragma once
#include <algorithm>
#include <cstdint>
#include <thread>
#include <vector>

namespace ainfer {

// Splits [0, n) into contiguous blocks over the host threads. Every index is
// computed independently, so results do not depend on the split.
template <typename F>
inline void parallel_for(uint64_t n, F &&f) {
  unsigned hw = std::thread::hardware_concurrency();
  uint64_t nt = std::min<uint64_t>(hw ? hw : 1, 32);
  if (n < 4096 || nt <= 1) {
    for (uint64_t i = 0; i < n; ++i) f(i);
    return;
  }
  std::vector<std::thread> th;
  uint64_t per = (n + nt - 1) / nt;
  for (uint64_t t = 0; t < nt; ++t) {
    uint64_t a = t * per, b = std::min(n, a + per);
    if (a >= b) break;
    th.emplace_back([a, b, &f] {
      for (uint64_t i = a; i < b; ++i) f(i);
    });
  }
  for (auto &t : th) t.join();
}

}  // namespace ainfer
