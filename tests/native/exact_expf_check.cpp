// Host build of lumen_b200/csrc/exact_expf.h for the CPU test-suite: compares the
// library's restated expf with the C library's expf over whole ranges of float
// bit patterns (multi-threaded) and returns the number of mismatches.
#include "../../lumen_b200/csrc/exact_expf.h"
#include <atomic>
#include <thread>
#include <vector>

extern "C" float lumen_expf_libm_host(float x) { return lumen_exact::expf_libm(x); }

extern "C" uint64_t lumen_expf_count_mismatches(uint32_t lo_bits, uint32_t hi_bits, int threads,
                                                uint32_t* first_bad_bits) {
    std::atomic<uint64_t> total{0};
    std::atomic<uint32_t> bad{0};
    std::vector<std::thread> th;
    const uint64_t n = (uint64_t)hi_bits - lo_bits;
    for (int i = 0; i < threads; ++i)
        th.emplace_back([&, i] {
            const uint64_t a = lo_bits + n * i / threads, b = lo_bits + n * (i + 1) / threads;
            uint64_t m = 0;
            for (uint64_t u = a; u < b; ++u) {
                const uint32_t bits = (uint32_t)u;
                float x;
                memcpy(&x, &bits, 4);
                const float ref = expf(x), got = lumen_exact::expf_libm(x);
                if (memcmp(&ref, &got, 4) != 0 && !(ref != ref && got != got)) {
                    if (m == 0) bad = bits;
                    ++m;
                }
            }
            total += m;
        });
    for (auto& t : th) t.join();
    if (first_bad_bits) *first_bad_bits = bad.load();
    return total.load();
}
