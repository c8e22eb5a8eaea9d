// C entry points of the library: argument validation, error strings and the
// ownership rules of the reference C API (vesin/src/vesin.cpp:41-179), in
// front of the CUDA engine.
#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif

#include <cmath>
#include <cstddef>
#include <cstdlib>
#include <cstring>

#include <algorithm>
#include <iostream>
#include <mutex>
#include <new>
#include <stdexcept>
#include <string>
#include <vector>

#include <dlfcn.h>
#include <link.h>

#include "vesin.h"
#include "vesin_b200.h"

#include "engine.hpp"

// x86-64 layouts of the reference header (vesin/include/vesin.h:49-163)
static_assert(sizeof(VesinOptions) == 32, "VesinOptions layout");
static_assert(offsetof(VesinOptions, cutoff) == 0, "VesinOptions layout");
static_assert(offsetof(VesinOptions, full) == 8, "VesinOptions layout");
static_assert(offsetof(VesinOptions, sorted) == 9, "VesinOptions layout");
static_assert(offsetof(VesinOptions, algorithm) == 12, "VesinOptions layout");
static_assert(offsetof(VesinOptions, n_threads) == 16, "VesinOptions layout");
static_assert(offsetof(VesinOptions, return_shifts) == 20, "VesinOptions layout");
static_assert(offsetof(VesinOptions, return_distances) == 21, "VesinOptions layout");
static_assert(offsetof(VesinOptions, return_vectors) == 22, "VesinOptions layout");
static_assert(offsetof(VesinOptions, skin) == 24, "VesinOptions layout");
static_assert(sizeof(VesinDevice) == 8, "VesinDevice layout");
static_assert(sizeof(VesinNeighborList) == 56, "VesinNeighborList layout");
static_assert(offsetof(VesinNeighborList, length) == 0, "VesinNeighborList layout");
static_assert(offsetof(VesinNeighborList, device) == 8, "VesinNeighborList layout");
static_assert(offsetof(VesinNeighborList, pairs) == 16, "VesinNeighborList layout");
static_assert(offsetof(VesinNeighborList, shifts) == 24, "VesinNeighborList layout");
static_assert(offsetof(VesinNeighborList, distances) == 32, "VesinNeighborList layout");
static_assert(offsetof(VesinNeighborList, vectors) == 40, "VesinNeighborList layout");
static_assert(offsetof(VesinNeighborList, opaque) == 48, "VesinNeighborList layout");

// dynamically built messages live here until the next failure on this thread
static thread_local std::string LAST_ERROR;

static int neighbors_entry(
    const void* points,
    size_t n_points,
    const void* box,
    const bool periodic[3],
    VesinDevice device,
    VesinOptions options,
    VesinNeighborList* neighbors,
    const char** error_message,
    bool float_io,
    bool canonical = false
) {
    // Order and wording of the checks: vesin/src/vesin.cpp:51-105
    if (error_message == nullptr) {
        return EXIT_FAILURE;
    }
    if (points == nullptr) {
        *error_message = "`points` can not be a NULL pointer";
        return EXIT_FAILURE;
    }
    if (box == nullptr) {
        *error_message = "`cell` can not be a NULL pointer";
        return EXIT_FAILURE;
    }
    if (neighbors == nullptr) {
        *error_message = "`neighbors` can not be a NULL pointer";
        return EXIT_FAILURE;
    }
    if (!std::isfinite(options.cutoff) || options.cutoff <= 0) {
        *error_message = "cutoff must be a finite, positive number";
        return EXIT_FAILURE;
    }
    if (options.cutoff <= 1e-6) {
        *error_message = "cutoff is too small";
        return EXIT_FAILURE;
    }
    if (!std::isfinite(options.skin) || options.skin < 0.0) {
        // the reference sets this message and carries on (vesin.cpp:80-82)
        *error_message = "skin must be a finite, non-negative number";
    }
    if (options.n_threads < 0) {
        *error_message = "n_threads must be zero or a positive integer";
        return EXIT_FAILURE;
    }
    if (neighbors->device.type != VesinUnknownDevice && neighbors->device.type != device.type) {
        *error_message = "`neighbors` device and data `device` do not match, free the neighbors first";
        return EXIT_FAILURE;
    }
    if (device.type == VesinUnknownDevice) {
        *error_message = "got an unknown device type";
        return EXIT_FAILURE;
    }
    if (neighbors->device.type == VesinUnknownDevice) {
        neighbors->device = device;
    }

    try {
        if (device.type == VesinCUDA) {
            vb200::neighbors(points, n_points, box, periodic, options, *neighbors, float_io, canonical);
        } else if (device.type == VesinCPU) {
            throw std::runtime_error(
                "this build of vesin is the CUDA (sm_100a) engine only: data on VesinCPU is not supported, "
                "move it to a CUDA device"
            );
        } else {
            throw std::runtime_error("unknown device " + std::to_string(device.type));
        }
    } catch (const std::bad_alloc&) {
        LAST_ERROR = "failed to allocate memory";
        *error_message = LAST_ERROR.c_str();
        return EXIT_FAILURE;
    } catch (const std::exception& e) {
        LAST_ERROR = e.what();
        *error_message = LAST_ERROR.c_str();
        return EXIT_FAILURE;
    } catch (...) {
        *error_message = "fatal error: unknown type thrown as exception";
        return EXIT_FAILURE;
    }
    return EXIT_SUCCESS;
}

extern "C" int vesin_neighbors(
    const double (*points)[3],
    size_t n_points,
    const double box[3][3],
    const bool periodic[3],
    VesinDevice device,
    VesinOptions options,
    VesinNeighborList* neighbors,
    const char** error_message
) {
    return neighbors_entry(points, n_points, box, periodic, device, options, neighbors, error_message, /*float_io=*/false);
}

extern "C" int vesin_b200_neighbors_f32(
    const float (*points)[3],
    size_t n_points,
    const float box[3][3],
    const bool periodic[3],
    VesinDevice device,
    VesinOptions options,
    VesinNeighborList* neighbors,
    const char** error_message
) {
    return neighbors_entry(points, n_points, box, periodic, device, options, neighbors, error_message, /*float_io=*/true);
}

extern "C" int vesin_b200_neighbors_canonical(
    const double (*points)[3],
    size_t n_points,
    const double box[3][3],
    const bool periodic[3],
    VesinDevice device,
    VesinOptions options,
    VesinNeighborList* neighbors,
    const char** error_message
) {
    return neighbors_entry(points, n_points, box, periodic, device, options, neighbors, error_message, /*float_io=*/false, /*canonical=*/true);
}

extern "C" void vesin_free(VesinNeighborList* neighbors) {
    if (neighbors == nullptr) {
        return;
    }
    try {
        if (neighbors->device.type == VesinCUDA) {
            vb200::free_neighbors(*neighbors);
        } else if (neighbors->device.type != VesinUnknownDevice && neighbors->device.type != VesinCPU) {
            throw std::runtime_error("unknown device " + std::to_string(neighbors->device.type) + " when freeing memory");
        }
    } catch (const std::exception& e) {
        std::cerr << "error in vesin_free: " << e.what() << std::endl;
        return;
    } catch (...) {
        std::cerr << "fatal error in vesin_free, unknown type thrown as exception" << std::endl;
        return;
    }
    std::memset(neighbors, 0, sizeof(VesinNeighborList));
}

// ---- loaded shared objects (vesin/src/shared_libraries.cpp:89-107) ----

static std::mutex LIBRARIES_MUTEX;
static std::vector<std::string> LIBRARIES;

static int collect_library(struct dl_phdr_info* info, size_t, void* data) {
    static_cast<std::vector<std::string>*>(data)->emplace_back(info->dlpi_name);
    return 0;
}

extern "C" void vesin_list_libraries(const char* libs[], size_t* count) {
    std::lock_guard<std::mutex> guard(LIBRARIES_MUTEX);
    if (libs == nullptr || count == nullptr) {
        return;
    }
    LIBRARIES.clear();
    dl_iterate_phdr(collect_library, &LIBRARIES);
    size_t n = std::min(*count, LIBRARIES.size());
    for (size_t i = 0; i < n; i++) {
        libs[i] = LIBRARIES[i].c_str();
    }
    *count = LIBRARIES.size();
}

// ---- additive entry points ----

extern "C" void vesin_b200_set_profiling(int enabled) {
    vb200::set_profiling(enabled != 0);
}

extern "C" int vesin_b200_stage_times(const VesinNeighborList* neighbors, double* stage_ms) {
    if (neighbors == nullptr || stage_ms == nullptr) {
        return 1;
    }
    return vb200::stage_times(*neighbors, stage_ms) ? 0 : 1;
}

static int batch_entry(
    const void* points,
    bool float_io,
    const size_t* system_offsets,
    size_t n_systems,
    const void* boxes,
    const bool (*periodic)[3],
    VesinDevice device,
    VesinOptions options,
    bool global_indices,
    VesinNeighborList* neighbors,
    const size_t** pair_offsets,
    const char** error_message
) {
    if (error_message == nullptr) {
        return EXIT_FAILURE;
    }
    if (system_offsets == nullptr) {
        *error_message = "`system_offsets` can not be a NULL pointer";
        return EXIT_FAILURE;
    }
    if (points == nullptr && n_systems > 0 && system_offsets[n_systems] != system_offsets[0]) {
        *error_message = "`points` can not be a NULL pointer";
        return EXIT_FAILURE;
    }
    if (neighbors == nullptr) {
        *error_message = "`neighbors` can not be a NULL pointer";
        return EXIT_FAILURE;
    }
    if (!std::isfinite(options.cutoff) || options.cutoff <= 0) {
        *error_message = "cutoff must be a finite, positive number";
        return EXIT_FAILURE;
    }
    if (options.cutoff <= 1e-6) {
        *error_message = "cutoff is too small";
        return EXIT_FAILURE;
    }
    if (device.type != VesinCUDA) {
        *error_message = "vesin_b200_neighbors_batch only works on CUDA devices";
        return EXIT_FAILURE;
    }
    if (neighbors->device.type != VesinUnknownDevice &&
        (neighbors->device.type != device.type || neighbors->device.device_id != device.device_id)) {
        *error_message = "`neighbors` device and data `device` do not match, free the neighbors first";
        return EXIT_FAILURE;
    }
    neighbors->device = device;
    try {
        vb200::neighbors_batch(points, float_io, system_offsets, n_systems, boxes, periodic, options, global_indices, *neighbors, pair_offsets);
    } catch (const std::bad_alloc&) {
        LAST_ERROR = "failed to allocate memory";
        *error_message = LAST_ERROR.c_str();
        return EXIT_FAILURE;
    } catch (const std::exception& e) {
        LAST_ERROR = e.what();
        *error_message = LAST_ERROR.c_str();
        return EXIT_FAILURE;
    }
    return EXIT_SUCCESS;
}

extern "C" int vesin_b200_neighbors_batch(
    const double (*points)[3],
    const size_t* system_offsets,
    size_t n_systems,
    const double (*boxes)[3][3],
    const bool (*periodic)[3],
    VesinDevice device,
    VesinOptions options,
    bool global_indices,
    VesinNeighborList* neighbors,
    const size_t** pair_offsets,
    const char** error_message
) {
    return batch_entry(points, false, system_offsets, n_systems, boxes, periodic, device, options, global_indices, neighbors, pair_offsets, error_message);
}

extern "C" int vesin_b200_neighbors_batch_f32(
    const float (*points)[3],
    const size_t* system_offsets,
    size_t n_systems,
    const float (*boxes)[3][3],
    const bool (*periodic)[3],
    VesinDevice device,
    VesinOptions options,
    bool global_indices,
    VesinNeighborList* neighbors,
    const size_t** pair_offsets,
    const char** error_message
) {
    return batch_entry(points, true, system_offsets, n_systems, boxes, periodic, device, options, global_indices, neighbors, pair_offsets, error_message);
}

static int slab_entry(
    const void* points,
    bool float_io,
    size_t n_points,
    size_t n_owned,
    const int64_t* global_index,
    const void* box,
    const bool periodic[3],
    VesinB200Slab slab,
    VesinDevice device,
    VesinOptions options,
    VesinNeighborList* neighbors,
    const char** error_message
) {
    if (error_message == nullptr) {
        return EXIT_FAILURE;
    }
    if (points == nullptr || box == nullptr || periodic == nullptr || global_index == nullptr) {
        *error_message = "`points`, `global_index`, `box` and `periodic` can not be NULL pointers";
        return EXIT_FAILURE;
    }
    if (neighbors == nullptr) {
        *error_message = "`neighbors` can not be a NULL pointer";
        return EXIT_FAILURE;
    }
    if (!std::isfinite(options.cutoff) || options.cutoff <= 0) {
        *error_message = "cutoff must be a finite, positive number";
        return EXIT_FAILURE;
    }
    if (options.cutoff <= 1e-6) {
        *error_message = "cutoff is too small";
        return EXIT_FAILURE;
    }
    if (device.type != VesinCUDA) {
        *error_message = "vesin_b200_neighbors_slab only works on CUDA devices";
        return EXIT_FAILURE;
    }
    if (neighbors->device.type != VesinUnknownDevice &&
        (neighbors->device.type != device.type || neighbors->device.device_id != device.device_id)) {
        *error_message = "`neighbors` device and data `device` do not match, free the neighbors first";
        return EXIT_FAILURE;
    }
    neighbors->device = device;
    try {
        vb200::neighbors_slab(
            points, float_io, n_points, n_owned, global_index, box, periodic, slab.axis, slab.lower, slab.upper, options, *neighbors
        );
    } catch (const std::bad_alloc&) {
        LAST_ERROR = "failed to allocate memory";
        *error_message = LAST_ERROR.c_str();
        return EXIT_FAILURE;
    } catch (const std::exception& e) {
        LAST_ERROR = e.what();
        *error_message = LAST_ERROR.c_str();
        return EXIT_FAILURE;
    }
    return EXIT_SUCCESS;
}

extern "C" int vesin_b200_neighbors_slab(
    const double (*points)[3],
    size_t n_points,
    size_t n_owned,
    const int64_t* global_index,
    const double box[3][3],
    const bool periodic[3],
    VesinB200Slab slab,
    VesinDevice device,
    VesinOptions options,
    VesinNeighborList* neighbors,
    const char** error_message
) {
    return slab_entry(points, false, n_points, n_owned, global_index, box, periodic, slab, device, options, neighbors, error_message);
}

extern "C" int vesin_b200_neighbors_slab_f32(
    const float (*points)[3],
    size_t n_points,
    size_t n_owned,
    const int64_t* global_index,
    const float box[3][3],
    const bool periodic[3],
    VesinB200Slab slab,
    VesinDevice device,
    VesinOptions options,
    VesinNeighborList* neighbors,
    const char** error_message
) {
    return slab_entry(points, true, n_points, n_owned, global_index, box, periodic, slab, device, options, neighbors, error_message);
}

extern "C" int vesin_b200_list_value_bytes(const VesinNeighborList* neighbors) {
    if (neighbors == nullptr) {
        return 0;
    }
    return vb200::list_value_bytes(*neighbors);
}

extern "C" int vesin_b200_list_checksum(const VesinNeighborList* neighbors, uint64_t checksum[4], const char** error_message) {
    if (error_message == nullptr) {
        return EXIT_FAILURE;
    }
    if (neighbors == nullptr || checksum == nullptr) {
        *error_message = "`neighbors` and `checksum` can not be NULL pointers";
        return EXIT_FAILURE;
    }
    try {
        unsigned long long result[4];
        vb200::list_checksum(*neighbors, result);
        for (int k = 0; k < 4; k++) {
            checksum[k] = result[k];
        }
    } catch (const std::exception& e) {
        LAST_ERROR = e.what();
        *error_message = LAST_ERROR.c_str();
        return EXIT_FAILURE;
    }
    return EXIT_SUCCESS;
}

extern "C" const char* vesin_b200_version(void) {
    return "vesin-b200 0.1.0 (C ABI of vesin 0.5.8)";
}
