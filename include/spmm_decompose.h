// The 2:4 + residual split of a weight matrix: the entry points of the reference's
// kernel_benchmark/spmm_decompose.h that its harness calls (decompose, spmm_test.cu:292) or keeps
// beside it (decompose_v1), with the same names, signatures and C++ linkage.  The reference
// defines them in the header; here they are defined in libSpMM_API.so.
#pragma once

#include <cuda_fp16.h>

// Replaces decompose, kernel_benchmark/spmm_decompose.h:12-51.  A, A1, A2: `length` halves each,
// host memory, length % 4 == 0 (asserted, as in the reference).  Every aligned group of four
// consecutive elements is split: its first two nonzeros (value != 0.0f, so -0 counts as zero and NaN
// as nonzero) keep their places in A1, later ones go to A2; everything else in A1 and A2 is +0.
// A1 + A2 == A element-wise, and A1 has at most two nonzeros per group of four.  Prints the two
// nonzero counts and A1's padding ratio, as the reference does.
void decompose(half* A, half* A1, half* A2, int length);

// Replaces decompose_v1, kernel_benchmark/spmm_decompose.h:53-142: as above, except that a group
// with at most one nonzero goes to A2 whole, so that A1 only holds groups that fill both slots.
void decompose_v1(half* A, half* A1, half* A2, int length);
