/*
 * Additive entry points of the B200 engine. Nothing here exists in the
 * reference's C API (vesin/include/vesin.h); callers that only know the
 * reference header never need this one.
 */
#ifndef VESIN_B200_H
#define VESIN_B200_H

#include "vesin.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Stages of one build, in launch order (index into the timing array). */
enum VesinB200Stage {
    VesinB200StageBounds = 0,  /* header + min/max + finite check, incl. its read-back */
    VesinB200StageBin = 1,     /* wrap + bin + histogram */
    VesinB200StageScanCells = 2,
    VesinB200StageScatter = 3,
    VesinB200StageCount = 4,   /* pass 1: hit masks + pairs per point */
    VesinB200StageScanRows = 5,
    VesinB200StageEmit = 6,    /* pass 2: writes i, j, S, d, D */
    VesinB200StageCount_ = 7,
};

/* No counterpart in the reference. Switches per-stage device timing (CUDA
 * events on the engine's own stream) on or off for all later calls of
 * vesin_neighbors in this process. Off by default: recording costs a few
 * microseconds per call. */
VESIN_API void vesin_b200_set_profiling(int enabled);

/* No counterpart in the reference. Copies the device time, in milliseconds,
 * of every stage of the LAST build made with `neighbors` into `stage_ms`
 * (VesinB200StageCount_ doubles). Returns 0, or 1 when no timed build was
 * made with this list. */
VESIN_API int vesin_b200_stage_times(const struct VesinNeighborList* neighbors, double* stage_ms);

/*
 * No counterpart in the reference's C API, which is fp64 only: its bindings
 * upcast float32 inputs and downcast the results in separate passes
 * (python/vesin/vesin/_neighbors.py:251-252,330,339). This entry point reads
 * float32 points and box and writes float32 distances and vectors in the same
 * pass: `neighbors->distances` and `neighbors->vectors` then point at FLOAT
 * arrays (float[length], float[length][3]) although the struct declares
 * doubles. Every decision is taken in fp64 on the exactly converted inputs, so
 * pairs and shifts are those of vesin_neighbors on the upcast data; d and D are
 * the fp64 results rounded once. Everything else as vesin_neighbors. A list
 * used with this function must not be handed to vesin_neighbors without the
 * caller remembering which element type the value arrays hold.
 */
VESIN_API int vesin_b200_neighbors_f32(
    const float (*points)[3],
    size_t n_points,
    const float box[3][3],
    const bool periodic[3],
    struct VesinDevice device,
    struct VesinOptions options,
    struct VesinNeighborList* neighbors,
    const char** error_message
);

/*
 * No counterpart in the reference (its callers loop over systems, e.g.
 * python/vesin/vesin/metatomic/_neighbors.py:197-199): the lists of a batch of
 * independent small systems in ONE call.
 *
 * points          device, all systems back to back
 * system_offsets  HOST array of n_systems + 1 offsets into `points`
 * boxes, periodic device arrays with one box / one flag triple per system, or
 *                 both NULL when no system is periodic
 * global_indices  false: pair indices count from the start of each system (as
 *                 n_systems separate calls of vesin_neighbors would give);
 *                 true: from the start of the batch
 * pair_offsets    out: device array of n_systems + 1 entries owned by the list;
 *                 system k owns pairs [pair_offsets[k], pair_offsets[k + 1])
 * The pair set of every system is what vesin_neighbors gives for it. Pairs
 * are grouped by system; `options.sorted`, `algorithm` and `skin` are ignored.
 * At most 2048 points per system. Same error and ownership rules as
 * vesin_neighbors; `neighbors` is released with vesin_free.
 */
VESIN_API int vesin_b200_neighbors_batch(
    const double (*points)[3],
    const size_t* system_offsets,
    size_t n_systems,
    const double (*boxes)[3][3],
    const bool (*periodic)[3],
    struct VesinDevice device,
    struct VesinOptions options,
    bool global_indices,
    struct VesinNeighborList* neighbors,
    const size_t** pair_offsets,
    const char** error_message
);

/* The slab of one rank: the box is cut along direction `axis` (which must be
 * periodic); the rank owns the points whose fractional coordinate along that
 * direction, wrapped into [0, 1), lies in [lower, upper). */
struct VesinB200Slab {
    int axis;
    double lower;
    double upper;
};

/*
 * No counterpart in the reference (which has no multi-GPU notion): one rank's
 * share of the list of a periodic system that is slab-decomposed over several
 * GPUs.
 *
 * points        device: the rank's OWNED points first (n_owned of them), then its
 *               halo: copies of the other ranks' points that lie within the
 *               cutoff of the slab (any periodic image; the engine brings them
 *               next to the slab itself)
 * global_index  device: index of every local point in the whole system; these
 *               indices are written to `pairs`
 * box, periodic device: the box of the WHOLE system
 * Full lists: the rank gets every pair (i, j, S) whose i it owns. Half lists:
 * every pair of the system's half list comes out on exactly one rank. The
 * union over ranks is the list vesin_neighbors gives for the whole system;
 * shifts refer to the whole box and the original coordinates.
 * Needs: slab thickness >= cutoff, and box length along `axis` >= slab + 2 halo
 * layers. Unsorted lists only. Same error and ownership rules as
 * vesin_neighbors. The halo exchange itself (NCCL send/recv between
 * neighbouring ranks) is done by the caller; vesin_b200.ShardedNeighborList
 * does it with torch.distributed.
 */
VESIN_API int vesin_b200_neighbors_slab(
    const double (*points)[3],
    size_t n_points,
    size_t n_owned,
    const int64_t* global_index,
    const double box[3][3],
    const bool periodic[3],
    struct VesinB200Slab slab,
    struct VesinDevice device,
    struct VesinOptions options,
    struct VesinNeighborList* neighbors,
    const char** error_message
);

/*
 * No counterpart in the reference: builds the two halo messages of a rank of a
 * slab-decomposed system (see vesin_b200_neighbors_slab). Asynchronous, on the
 * legacy default stream of the current device.
 *
 * points, global_index  device: the points the rank owns
 * inverse_column        HOST: column `axis` of the inverse box, so that
 *                       f = x*c[0] + y*c[1] + z*c[2] is the fractional
 *                       coordinate along the cut direction
 * lower, upper          the rank's slab in wrapped fractional coordinates
 * reach                 cutoff / face distance along the cut direction
 * to_lower, to_upper    device: messages for the two neighbours, (capacity + 1)
 *                       rows of 4 doubles each: row 0 = number of records (it can
 *                       exceed `capacity`: then the message is incomplete), every
 *                       other row = x, y, z, global index (raw 64 bits)
 * counts                device: 2 counters, scratch of the call
 */
VESIN_API int vesin_b200_pack_halo(
    const double (*points)[3],
    const int64_t* global_index,
    size_t n_points,
    const double inverse_column[3],
    double lower,
    double upper,
    double reach,
    double* to_lower,
    double* to_upper,
    size_t capacity,
    uint64_t* counts,
    const char** error_message
);

/* Largest system vesin_b200_neighbors_no_alloc accepts. */
#define VESIN_B200_NO_ALLOC_MAX_POINTS 32768

/*
 * No counterpart in the reference: a list build that allocates nothing.
 *
 * For callers that must not call cudaMalloc when they need a list: a step
 * function that runs while a CUDA graph is captured or replayed in the same
 * process, an application that handed all device memory to its own pool, a
 * loop with a hard latency bound. vesin_neighbors allocates whenever a system
 * outgrows its workspace; this function never does. The caller passes the
 * inputs AND the output arrays (device memory on `device_id`, `capacity` pairs
 * each; shifts / distances / vectors may be NULL to skip them); the scratch of
 * the kernels is a fixed array of about 2.3 MB that every GPU holds from
 * library load to process exit. Hence:
 *   - `pairs` must be aligned to 16 bytes (the other arrays to their element:
 *     4 and 8 bytes); full lists are written fastest when `pairs` is aligned to
 *     32 bytes and `distances` / `vectors` to 16;
 *   - at most VESIN_B200_NO_ALLOC_MAX_POINTS points, larger systems get an error;
 *   - the list is unsorted, same pair set as vesin_neighbors;
 *   - when the list has more than `capacity` pairs the call fails, `*length`
 *     holds the number needed and the arrays hold nothing usable;
 *   - all calls share the scratch array (what must be zero is cleared at the
 *     start of each call); calls are serialised per device by a host lock and
 *     run on the legacy default stream; the function returns when the list is
 *     complete. Work that overlapped on the GPU with another user of the same
 *     array would race: there is none inside one process;
 *   - the FIRST call on a device looks up the array's device address and sets
 *     kernel attributes: make it before any stream capture starts.
 * Returns 0, or 1 with *error_message set (valid until this thread's next
 * failing call).
 */
VESIN_API int vesin_b200_neighbors_no_alloc(
    const double (*points)[3],
    size_t n_points,
    const double box[3][3],
    const bool periodic[3],
    int device_id,
    double cutoff,
    bool full,
    size_t capacity,
    size_t (*pairs)[2],
    int32_t (*shifts)[3],
    double* distances,
    double (*vectors)[3],
    size_t* length,
    const char** error_message
);

/* No counterpart in the reference. Version string of this library. */
VESIN_API const char* vesin_b200_version(void);

#ifdef __cplusplus
}
#endif

#endif
