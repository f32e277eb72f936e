// Process-wide count of this library's kernel launches (reported by the benchmark).
#pragma once
#include <atomic>
#include <cstdint>

namespace rt {
std::atomic<int64_t>& launch_counter();
inline void count_launch(int n = 1) { launch_counter().fetch_add(n, std::memory_order_relaxed); }
}  // namespace rt
