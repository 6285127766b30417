// Minimal fork-join helper for the host-side encoders and generators.
#pragma once

#include <algorithm>
#include <cstdlib>
#include <thread>
#include <vector>

namespace spmm_b200 {

// Number of host threads to use: SPMM_B200_THREADS if set, else all hardware threads.
inline int host_thread_count()
{
    if (const char* env = std::getenv("SPMM_B200_THREADS")) {
        const int n = std::atoi(env);
        if (n > 0)
            return n;
    }
    const unsigned hw = std::thread::hardware_concurrency();
    return hw ? static_cast<int>(hw) : 1;
}

// Calls body(begin, end) over a partition of [0, n) into contiguous blocks, one block per thread.
template<typename Body>
void parallel_for(long n, Body body)
{
    const int threads = static_cast<int>(std::min<long>(host_thread_count(), n));
    if (threads <= 1) {
        if (n > 0)
            body(0L, n);
        return;
    }
    std::vector<std::thread> pool;
    pool.reserve(threads);
    for (int t = 0; t < threads; t++) {
        const long begin = n * t / threads, end = n * (t + 1) / threads;
        pool.emplace_back([=] { body(begin, end); });
    }
    for (auto& th : pool)
        th.join();
}

}  // namespace spmm_b200
