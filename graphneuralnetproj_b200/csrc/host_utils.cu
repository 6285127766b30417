// Host-side helpers behind include/spmm_b200.h: the 2:4 + residual split of
// kernel_benchmark/spmm_decompose.h:12-142 and the seeded input generator.
#include <cassert>
#include <cmath>
#include <cstdio>
#include <cstdint>
#include <cstring>

#include <cuda_fp16.h>

#include "../../include/spmm_b200.h"
#include "../../include/spmm_decompose.h"
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

// Element `index` of the stream spmm_b200_synth_fp16 draws: three counter-based uniforms per element.
inline uint16_t synth_element(uint64_t index, uint64_t seed, double sigma, double p_zero)
{
    const uint64_t base = index * 3u;
    const double   u3   = unit_open(splitmix64_at(seed, base + 2));
    if (u3 < p_zero)
        return 0;
    const double u1 = unit_open(splitmix64_at(seed, base));
    const double u2 = unit_open(splitmix64_at(seed, base + 1));
    const double g  = std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586476925 * u2);
    const __half h  = __float2half_rn(static_cast<float>(sigma * g));
    uint16_t     bits;
    std::memcpy(&bits, &h, 2);
    return bits;
}

}  // namespace

// C++ entry points with the names and signatures of kernel_benchmark/spmm_decompose.h:12 and :53,
// declared in include/spmm_decompose.h.  Like the reference they report how the nonzeros were split.
namespace {
void report_split(const half* A1, const half* A2, int length)
{
    long nnz1 = 0, nnz2 = 0;
    const uint16_t* a1 = reinterpret_cast<const uint16_t*>(A1);
    const uint16_t* a2 = reinterpret_cast<const uint16_t*>(A2);
    for (long i = 0; i < length; i++) {
        nnz1 += splits_as_nonzero(a1[i]);
        nnz2 += splits_as_nonzero(a2[i]);
    }
    const double total = static_cast<double>(nnz1 + nnz2);
    printf("NNZ1= %ld ratio = %f pad_nnz=%d \nNNZ2= %ld ratio = %f\n", nnz1, total > 0 ? nnz1 / total : 0.0, length * 2 / 4,
           nnz2, total > 0 ? nnz2 / total : 0.0);
    printf("A1 padding ratio = %f\n", 1 - nnz1 * 1.0 / (length * 2 / 4));
}
}  // namespace

void decompose(half* A, half* A1, half* A2, int length)
{
    assert(length % 4 == 0);
    split_groups(reinterpret_cast<const uint16_t*>(A), reinterpret_cast<uint16_t*>(A1), reinterpret_cast<uint16_t*>(A2),
                 length, false);
    report_split(A1, A2, length);
}

void decompose_v1(half* A, half* A1, half* A2, int length)
{
    assert(length % 4 == 0);
    split_groups(reinterpret_cast<const uint16_t*>(A), reinterpret_cast<uint16_t*>(A1), reinterpret_cast<uint16_t*>(A2),
                 length, true);
    report_split(A1, A2, length);
}

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
        for (long i = i0; i < i1; i++)
            out[i] = synth_element(static_cast<uint64_t>(i), seed, sigma, p_zero);
    });
}

void spmm_b200_synth_fp16_block(
    uint16_t* out, long rows, long cols, long ld, long row0, long col0, uint64_t seed, double sigma, double p_zero)
{
    spmm_b200::parallel_for(rows, [=](long r0, long r1) {
        for (long r = r0; r < r1; r++)
            for (long c = 0; c < cols; c++)
                out[r * cols + c] = synth_element(static_cast<uint64_t>((row0 + r) * ld + col0 + c), seed, sigma, p_zero);
    });
}

}  // extern "C"
