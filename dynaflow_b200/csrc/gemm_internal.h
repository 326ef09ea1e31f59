// Declarations shared by the GEMM translation units of the library (not part of the C ABI).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/dynaflow_b200.h"

namespace df {

// Tensor map of a row-major bf16 matrix [rows, cols] with leading dimension ld (elements), for
// boxes of box_rows x 64 elements written to shared memory with the 128-byte swizzle.
bool make_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);

// Returned by launch_small_rows when no form of the split-K kernel fits the shape.
constexpr int DF_SMALL_NOT_APPLICABLE = -1000;

// C = A B^T (or the gate/up form) for at most 128 rows of A as tiles x k-ranges CTAs (the k ranges
// of a tile are one thread-block cluster), sized for `units` SMs. With allow_split == false every
// tile is one CTA. force_bh / force_splits > 0 pin the launch form (development builds only pass them).
int launch_small_rows(bool gateup, const void* a, const void* b0, const void* b1, void* c, int M, int N, int K, int lda,
                      int ldb, int ldc, int units, bool allow_split, int force_bh, int force_splits,
                      df_status_t* dev_status, cudaStream_t stream);

}  // namespace df
