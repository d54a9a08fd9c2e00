// C launch interface of the covariance (SYRK) kernel; see covariance.cu.
#pragma once

#include <cuda_runtime.h>

extern "C" {
// dst[r] + (row - row_start[r]) * D + col  receives  sum_t x[t, row] * x[t, col]  for every
// row owned by rank r (row_start has world + 1 entries), col >= 256 * (row / 256) (block
// upper triangle).  `local` ([D, D] fp32, may be null) is folded into the same adds.
// dst pointers may be peer-mapped memory of other GPUs.  With `full` every 128 x 256 tile is
// visited, so the destinations receive complete rows (cross-rank reduce-scatter of the
// product and/or of `local`); T == 0 with `local` set is a pure push of `local`.
// `local_upper`: `local` was itself accumulated by non-full launches (only its upper tiles are
// valid); the fold reads the remaining elements from their mirror positions.
int bgn_cov_syrk(const void* x, long T, int D, int fmt, float* const* dst, const int* row_start,
                 int world, const float* local, int full, int local_upper, int sm_count, int* status,
                 cudaStream_t stream);
}
