// Host orchestration of one neighbor-list build on a CUDA device.
#ifndef VESIN_B200_ENGINE_HPP
#define VESIN_B200_ENGINE_HPP

#include <cstddef>
#include <functional>
#include <cstdint>

#include <cuda_runtime.h>

#include "vesin.h"

namespace vb200 {

/// Compute the list for device-resident inputs. Replaces
/// vesin::cuda::neighbors (vesin/src/vesin_cuda.cpp:819-923). Throws
/// std::runtime_error / std::bad_alloc; the C entry point turns those into
/// error strings.
/// With `float_io`, `points` and `box` are float arrays and the distances /
/// vectors of the list are float arrays too (the decisions stay fp64).
/// With `canonical`, the list comes out sorted by (i, j, Sx, Sy, Sz).
void neighbors(
    const void* points,
    size_t n_points,
    const void* box,
    const bool periodic[3],
    VesinOptions options,
    VesinNeighborList& list,
    bool float_io,
    bool canonical = false
);

/// Lists of a batch of independent small systems in one call (no counterpart
/// in the reference, whose callers loop over systems). Throws like neighbors().
void neighbors_batch(
    const void* points,
    bool float_io,
    const size_t* system_offsets,
    size_t n_systems,
    const void* boxes,
    const bool (*periodic)[3],
    VesinOptions options,
    bool global_indices,
    VesinNeighborList& list,
    const size_t** pair_offsets
);

/// Halo of a slab that arrives as two messages (see PointSource in
/// kernels.cuh for their layout) instead of sitting behind the owned points.
struct HaloMessages {
    const double* from_upper;
    const double* from_lower;
    size_t capacity;         // records a message can hold
    cudaEvent_t received;    // recorded after the receives on their stream, or null
    size_t expected_records; // guess of the records both messages bring (sizes the work units of a first build)
    /// If set: the messages are not on their way yet. The build calls this once, as soon as it
    /// has queued the work that does not need them (or at once if there is none); the call
    /// queues the exchange and records `received`. It must not throw.
    std::function<void()> start_exchange;
};

/// One rank's share of a slab-decomposed periodic system (no counterpart in
/// the reference). `points` holds n_array points, the first n_owned of them
/// owned, the rest halo; more halo may come in `halo`. `box` and `periodic`
/// are HOST values. Throws like neighbors().
void neighbors_slab_core(
    const void* points,
    bool float_io,
    size_t n_array,
    size_t n_owned,
    const int64_t* global_index,
    const HaloMessages* halo,
    const double box[9],
    const bool periodic[3],
    int axis,
    double lower,
    double upper,
    VesinOptions options,
    VesinNeighborList& list
);

/// The same with box and periodicity in device memory and the whole halo in
/// `points` (float or double data, like neighbors()).
void neighbors_slab(
    const void* points,
    bool float_io,
    size_t n_points,
    size_t n_owned,
    const int64_t* global_index,
    const void* box,
    const bool periodic[3],
    int axis,
    double lower,
    double upper,
    VesinOptions options,
    VesinNeighborList& list
);

/// The stream the builds of this list run on (creates the list's workspace).
cudaStream_t list_stream(VesinNeighborList& list);

/// Bytes per element of `distances` / `vectors` of the list's last build (4 or
/// 8), 0 for a list that holds nothing.
int list_value_bytes(const VesinNeighborList& list);

/// Order-independent checksum of the list, see vesin_b200_list_checksum.
void list_checksum(const VesinNeighborList& list, unsigned long long result[4]);

/// Release everything a list holds on its device. Replaces
/// vesin::cuda::free_neighbors (vesin/src/vesin_cuda.cpp:129-138).
void free_neighbors(VesinNeighborList& list);

void set_profiling(bool enabled);
bool profiling_enabled();
bool stage_times(const VesinNeighborList& list, double* stage_ms);

} // namespace vb200

#endif
