// Process-wide count of kernel launches issued through the Python bindings (one per bound call that launches).
#pragma once
#include <atomic>

namespace tb {
inline std::atomic<long long> g_kernel_launches{0};
inline void note_launch(int n = 1) { g_kernel_launches.fetch_add(n, std::memory_order_relaxed); }
}  // namespace tb
