// Host-side helpers behind include/spmm_b200.h: the 2:4 + residual split of
// kernel_benchmark/spmm_decompose.h:12-142 and the seeded input generator.
#include <cmath>
#include <cstdint>
#include <cstring>

#include <cuda_fp16.h>

#include "../../include/spmm_b200.h"
#include "host_threads.h"

namespace {

// __half2float(v) != 0.0f, the test decompose uses (spmm_decompose.h:26): true for NaN, false for +-0.
inline bool splits_as_nonzero(uint16_t bits)
{
    return (bits & 0x7fffu) != 0;
}

void split_groups(const uint16_t* A, uint16_t* A1, uint16_t* A2, int length, bool sparse_groups_to_a2)
{
    const long groups = length / 4;
    spmm_b200::parallel_for(groups, [=](long g0, long g1) {
        for (long g = g0; g < g1; g++) {
            const uint16_t* a  = A + 4 * g;
            uint16_t*       a1 = A1 + 4 * g;
            uint16_t*       a2 = A2 + 4 * g;
            int             nnz = 0;
            for (int x = 0; x < 4; x++)
                nnz += splits_as_nonzero(a[x]);
            const int keep  = (sparse_groups_to_a2 && nnz <= 1) ? 0 : 2;
            int       taken = 0;
            for (int x = 0; x < 4; x++) {
                a1[x] = 0;
                a2[x] = 0;
                if (splits_as_nonzero(a[x])) {
                    if (taken < keep) {
                        a1[x] = a[x];
                        taken++;
                    }
                    else {
                        a2[x] = a[x];
                    }
                }
            }
        }
    });
    for (long i = groups * 4; i < length; i++)
        A1[i] = A2[i] = 0;
}

inline uint64_t splitmix64_at(uint64_t seed, uint64_t index)
{
    uint64_t z = seed + (index + 1) * 0x9e3779b97f4a7c15ull;
    z          = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z          = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

inline double unit_open(uint64_t x)
{
    return (static_cast<double>(x >> 11) + 0.5) * (1.0 / 9007199254740992.0);
}

}  // namespace

extern "C" {

void spmm_b200_decompose(const uint16_t* A, uint16_t* A1, uint16_t* A2, int length)
{
    split_groups(A, A1, A2, length, false);
}

void spmm_b200_decompose_v1(const uint16_t* A, uint16_t* A1, uint16_t* A2, int length)
{
    split_groups(A, A1, A2, length, true);
}

void spmm_b200_synth_fp16(uint16_t* out, long count, uint64_t seed, double sigma, double p_zero)
{
    spmm_b200::parallel_for(count, [=](long i0, long i1) {
        for (long i = i0; i < i1; i++) {
            const uint64_t base = static_cast<uint64_t>(i) * 3u;
            const double   u3   = unit_open(splitmix64_at(seed, base + 2));
            if (u3 < p_zero) {
                out[i] = 0;
                continue;
            }
            const double u1 = unit_open(splitmix64_at(seed, base));
            const double u2 = unit_open(splitmix64_at(seed, base + 1));
            const double g  = std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586476925 * u2);
            const __half h  = __float2half_rn(static_cast<float>(sigma * g));
            uint16_t     bits;
            std::memcpy(&bits, &h, 2);
            out[i] = bits;
        }
    });
}

}  // extern "C"
