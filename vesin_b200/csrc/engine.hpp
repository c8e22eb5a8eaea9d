// Host orchestration of one neighbor-list build on a CUDA device.
#ifndef VESIN_B200_ENGINE_HPP
#define VESIN_B200_ENGINE_HPP

#include <cstddef>
#include <cstdint>

#include "vesin.h"

namespace vb200 {

/// Compute the list for device-resident inputs. Replaces
/// vesin::cuda::neighbors (vesin/src/vesin_cuda.cpp:819-923). Throws
/// std::runtime_error / std::bad_alloc; the C entry point turns those into
/// error strings.
/// With `float_io`, `points` and `box` are float arrays and the distances /
/// vectors of the list are float arrays too (the decisions stay fp64).
void neighbors(
    const void* points,
    size_t n_points,
    const void* box,
    const bool periodic[3],
    VesinOptions options,
    VesinNeighborList& list,
    bool float_io
);

/// Lists of a batch of independent small systems in one call (no counterpart
/// in the reference, whose callers loop over systems). Throws like neighbors().
void neighbors_batch(
    const double (*points)[3],
    const size_t* system_offsets,
    size_t n_systems,
    const double (*boxes)[3][3],
    const bool (*periodic)[3],
    VesinOptions options,
    bool global_indices,
    VesinNeighborList& list,
    const size_t** pair_offsets
);

/// One rank's share of a slab-decomposed periodic system (no counterpart in
/// the reference). Throws like neighbors().
void neighbors_slab(
    const double (*points)[3],
    size_t n_points,
    size_t n_owned,
    const int64_t* global_index,
    const double box[3][3],
    const bool periodic[3],
    int axis,
    double lower,
    double upper,
    VesinOptions options,
    VesinNeighborList& list
);

/// Release everything a list holds on its device. Replaces
/// vesin::cuda::free_neighbors (vesin/src/vesin_cuda.cpp:129-138).
void free_neighbors(VesinNeighborList& list);

void set_profiling(bool enabled);
bool stage_times(const VesinNeighborList& list, double* stage_ms);

} // namespace vb200

#endif
