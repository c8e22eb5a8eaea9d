/*
 * C ABI of the neighbor-list engine. This header is written fresh but is
 * layout- and signature-compatible with the reference's public header
 * (vesin/include/vesin.h:36-200): a program or binding compiled against either
 * header can be linked against this library. The x86-64 layouts are pinned by
 * static_asserts in vesin_b200/csrc/api.cu.
 *
 * Only the CUDA device kind is served (VesinDevice.type == VesinCUDA): the
 * engine is sm_100a CUDA with no CPU path. A call with VesinCPU fails with an
 * error message, like the reference's own no-CUDA stub does for VesinCUDA
 * (vesin/src/vesin_cuda_stub.cpp:5-18).
 */
#ifndef VESIN_H
#define VESIN_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__) || defined(__clang__)
#define VESIN_API __attribute__((visibility("default")))
#else
#define VESIN_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces: enum VesinAlgorithm, vesin/include/vesin.h:36-46 */
enum VesinAlgorithm {
    VesinAutoAlgorithm = 0, /* engine picks */
    VesinBruteForce = 1,    /* all-pairs; needs 2 * cutoff <= smallest face distance */
    VesinCellList = 2,      /* cell list */
};

/* Replaces: struct VesinOptions, vesin/include/vesin.h:49-78 (32 bytes) */
struct VesinOptions {
    double cutoff;         /* spherical cutoff; pairs with d < cutoff are kept */
    bool full;             /* both i->j and j->i (true) or each pair once (false) */
    bool sorted;           /* sort by first index i */
    enum VesinAlgorithm algorithm;
    int32_t n_threads;     /* CPU threads; validated (>= 0), unused on CUDA */
    bool return_shifts;    /* fill VesinNeighborList.shifts */
    bool return_distances; /* fill VesinNeighborList.distances */
    bool return_vectors;   /* fill VesinNeighborList.vectors */
    double skin;           /* Verlet skin; this engine rebuilds on every call */
};

/* Replaces: enum VesinDeviceKind, vesin/include/vesin.h:81-89 */
enum VesinDeviceKind {
    VesinUnknownDevice = 0,
    VesinCPU = 1,
    VesinCUDA = 2,
};

/* Replaces: struct VesinDevice, vesin/include/vesin.h:103-108 (8 bytes) */
struct VesinDevice {
    enum VesinDeviceKind type;
    int device_id;
};

/*
 * Replaces: struct VesinNeighborList, vesin/include/vesin.h:129-163 (56 bytes).
 * All arrays are device memory owned by the library. For a pair (i, j, S) the
 * vector is r_j - r_i + S . box (box rows are the cell vectors).
 * Zero-initialise before the first call; re-use across calls; release with
 * vesin_free.
 */
struct VesinNeighborList {
    size_t length;         /* number of pairs */
    struct VesinDevice device;
    size_t (*pairs)[2];    /* [length][2] point indices */
    int32_t (*shifts)[3];  /* [length][3] or NULL */
    double* distances;     /* [length]    or NULL */
    double (*vectors)[3];  /* [length][3] or NULL */
    void* opaque;          /* library-private workspace */
};

/* Replaces: vesin_free, vesin/include/vesin.h:167 (vesin/src/vesin.cpp:155-179).
 * Frees everything held by `neighbors` and zeroes the struct. */
VESIN_API void vesin_free(struct VesinNeighborList* neighbors);

/*
 * Replaces: vesin_neighbors, vesin/include/vesin.h:191-200
 * (vesin/src/vesin.cpp:41-153 -> vesin/src/vesin_cuda.cpp:819-923).
 *
 * points   [n_points][3] doubles, DEVICE memory on device.device_id
 * box      [3][3] doubles, one cell vector per row, DEVICE memory
 * periodic [3] bools, DEVICE memory
 * Returns EXIT_SUCCESS (0) or EXIT_FAILURE (1) with *error_message pointing at
 * a string owned by the library (valid until the next failing call made by
 * the same thread). All device work is complete when the function returns.
 */
VESIN_API int vesin_neighbors(
    const double (*points)[3],
    size_t n_points,
    const double box[3][3],
    const bool periodic[3],
    struct VesinDevice device,
    struct VesinOptions options,
    struct VesinNeighborList* neighbors,
    const char** error_message
);

/* Replaces: vesin_list_libraries, vesin/src/shared_libraries.cpp:89-107.
 * Writes up to *count paths of the shared objects loaded in this process into
 * `libs` and always stores the total number in *count. */
VESIN_API void vesin_list_libraries(const char* libs[], size_t* count);

#ifdef __cplusplus
}
#endif

#endif
