// Packing of the halo messages of a slab-decomposed system (halo.cu).
#ifndef VESIN_B200_HALO_CUH
#define VESIN_B200_HALO_CUH

#include <cstddef>

#include <cuda_runtime.h>

#include "kernels.cuh"

namespace vb200 {

/// One launch on `stream`: selects the points within `reach` (in fractional
/// units along the cut direction) of the two faces of the slab [lower, upper)
/// and writes the two messages (layout: see PointSource). `counts`: three
/// words of device scratch that are zero at entry; the kernel leaves them zero.
/// The messages must be aligned to 16 bytes.
void launch_pack_halo(
    RealView points, const long long* global_index, size_t n_points, const double inverse_column[3], double lower, double upper,
    double reach, double* to_lower, double* to_upper, size_t capacity, unsigned long long* counts, cudaStream_t stream
);

} // namespace vb200

#endif
