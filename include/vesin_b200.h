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
    VesinB200StageHalo = 7,    /* sharded lists: wait for the halo messages, then bin / scan / scatter of the halo */
    VesinB200StageCount_ = 8,
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
 * doubles (vesin_b200_list_value_bytes tells which). Every decision is taken in fp64 on the exactly converted inputs, so
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
 * No counterpart in the reference, whose `sorted` option orders a list by the
 * first index only and leaves the order of second indices and shifts open
 * (vesin/include/vesin.h:55-58; device sort keyed on pairs[.][0],
 * vesin/src/cuda/sort_pairs.cu:3-12): this entry point returns THE canonical
 * list, sorted by (i, j, Sx, Sy, Sz), so that two lists of the same system can
 * be compared element by element without sorting them on the host.
 * `options.sorted` is taken as set. Rows are sorted on the device after the
 * build, into a second set of output arrays (the list then owns twice the
 * memory of an unsorted one). Everything else as vesin_neighbors.
 */
VESIN_API int vesin_b200_neighbors_canonical(
    const double (*points)[3],
    size_t n_points,
    const double box[3][3],
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

/* The same for float32 points and boxes: float distances and vectors come out,
 * every decision is taken in fp64 on the exactly converted values (see
 * vesin_b200_neighbors_f32). */
VESIN_API int vesin_b200_neighbors_batch_f32(
    const float (*points)[3],
    const size_t* system_offsets,
    size_t n_systems,
    const float (*boxes)[3][3],
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
 * layers. Unsorted lists only. Global indices must lie in [0, 2^31): larger
 * ones are refused with an error. Same error and ownership rules as
 * vesin_neighbors. Here the caller brings the halo; vesin_b200_sharded_neighbors
 * (below) also does the exchange.
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

/* The same for float32 points and box: float distances and vectors come out,
 * every decision is taken in fp64 (see vesin_b200_neighbors_f32). */
VESIN_API int vesin_b200_neighbors_slab_f32(
    const float (*points)[3],
    size_t n_points,
    size_t n_owned,
    const int64_t* global_index,
    const float box[3][3],
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
 * legacy default stream of the device the arrays live on (all of them must be
 * device memory of one device; anything else is refused before a launch).
 *
 * points, global_index  device: the points the rank owns
 * inverse_column        HOST: column `axis` of the inverse box, so that
 *                       f = x*c[0] + y*c[1] + z*c[2] is the fractional
 *                       coordinate along the cut direction
 * lower, upper          the rank's slab in wrapped fractional coordinates
 * reach                 cutoff / face distance along the cut direction
 * to_lower, to_upper    device, aligned to 16 bytes: messages for the two
 *                       neighbours, (capacity + 1) rows of 4 doubles each: row 0 =
 *                       number of records (it can exceed `capacity`: then the
 *                       message is incomplete), every other row = x, y, z,
 *                       global index (raw 64 bits)
 * counts                device: 3 words, scratch of the call
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

/*
 * No counterpart in the reference: the numbers a slab decomposition of a box
 * rests on, as the library computes them. `axis`: the direction that is cut
 * (the periodic direction with the largest distance between faces).
 * `inverse_column`: f = x c[0] + y c[1] + z c[2] is the fractional coordinate
 * of a point along that direction; rank r of R owns the points whose f, wrapped
 * into [0, 1), lies in [r / R, (r + 1) / R). `reach`: cutoff over face distance,
 * the fractional thickness of the layer a rank sends to a neighbour. `box` and
 * `periodic` are HOST arrays.
 */
VESIN_API int vesin_b200_slab_geometry(
    const double box[3][3],
    const bool periodic[3],
    double cutoff,
    int* axis,
    double inverse_column[3],
    double* reach,
    const char** error_message
);

/*
 * Sharded lists: one periodic system spread over the GPUs of a node, one slab
 * and one process (or thread) per GPU. No counterpart in the reference, which
 * builds one system on one device per call (vesin/include/vesin.h:103-108).
 *
 * Set-up: one rank calls vesin_b200_sharded_unique_id and hands the 128 bytes to
 * all others (by whatever means the application has: MPI, a file, torch's
 * store); every rank then calls vesin_b200_sharded_create, which is collective
 * (it creates an NCCL communicator; NCCL is loaded at run time). `device_id` is
 * the rank's GPU.
 *
 * A build, vesin_b200_sharded_neighbors, collective as well:
 *   points, global_index  device: the points this rank OWNS (see
 *                         vesin_b200_slab_geometry) and their indices in the
 *                         whole system, in [0, 2^31)
 *   box, periodic         HOST: the whole system's box, the same on every rank
 * The rank packs the points within the cutoff of the two faces of its slab,
 * exchanges them with its two neighbours (ncclSend / ncclRecv over NVLink, into
 * this GPU's own memory) and builds its share of the list in `neighbors` (see
 * vesin_b200_neighbors_slab for what a rank gets; unsorted lists only). The
 * union over ranks is the list of vesin_neighbors for the whole system. Needs
 * slab thickness >= cutoff and at least two slabs plus two cutoffs along the cut
 * direction. Messages have a fixed capacity that the ranks agree on at the
 * first build (1.5 times the share of an evenly filled slab); a rank whose
 * halo outgrows it gets an error: then call vesin_b200_sharded_set_halo_capacity
 * with the same value on every rank. Errors raised before the exchange are the
 * same on all ranks (they depend on box, options and set-up only); a rank that
 * fails after it has still taken part in the exchange, so the others do not
 * wait for it.
 * `neighbors` is released with vesin_free, the handle with
 * vesin_b200_sharded_free (after the last build; collective).
 */
#define VESIN_B200_UNIQUE_ID_BYTES 128
struct VesinB200Sharded;

VESIN_API int vesin_b200_sharded_unique_id(unsigned char id[VESIN_B200_UNIQUE_ID_BYTES], const char** error_message);

/* `id` == NULL: a handle without communicator, for callers that move the
 * messages themselves (vesin_b200_sharded_pack / vesin_b200_sharded_build). */
VESIN_API int vesin_b200_sharded_create(
    const unsigned char* id,
    int rank,
    int world_size,
    int device_id,
    struct VesinB200Sharded** sharded,
    const char** error_message
);

VESIN_API void vesin_b200_sharded_free(struct VesinB200Sharded* sharded);

VESIN_API int vesin_b200_sharded_set_halo_capacity(struct VesinB200Sharded* sharded, size_t records, const char** error_message);

VESIN_API int vesin_b200_sharded_neighbors(
    struct VesinB200Sharded* sharded,
    const double (*points)[3],
    const int64_t* global_index,
    size_t n_owned,
    const double box[3][3],
    const bool periodic[3],
    struct VesinOptions options,
    struct VesinNeighborList* neighbors,
    const char** error_message
);

/* float32 points and box in, float distances and vectors out, decisions in
 * fp64 (see vesin_b200_neighbors_f32). */
VESIN_API int vesin_b200_sharded_neighbors_f32(
    struct VesinB200Sharded* sharded,
    const float (*points)[3],
    const int64_t* global_index,
    size_t n_owned,
    const float box[3][3],
    const bool periodic[3],
    struct VesinOptions options,
    struct VesinNeighborList* neighbors,
    const char** error_message
);

/*
 * The two halves of vesin_b200_sharded_neighbors for callers with a transport
 * of their own. vesin_b200_sharded_pack fills the rank's two outgoing messages
 * and returns, complete, the device addresses of its four messages: to the
 * lower neighbour, to the upper neighbour, from the upper neighbour, from the
 * lower neighbour, `rows` rows of 4 doubles each (row 0 = number of records,
 * then x, y, z, global index as raw bits). The caller copies every rank's
 * "to lower" into the lower neighbour's "from upper" and every "to upper" into
 * the upper neighbour's "from lower" (whole messages, or row 0 and the records
 * it counts), then calls vesin_b200_sharded_build with the same inputs.
 */
VESIN_API int vesin_b200_sharded_pack(
    struct VesinB200Sharded* sharded,
    const double (*points)[3],
    const int64_t* global_index,
    size_t n_owned,
    const double box[3][3],
    const bool periodic[3],
    double cutoff,
    double* messages[4],
    size_t* rows,
    const char** error_message
);

VESIN_API int vesin_b200_sharded_build(
    struct VesinB200Sharded* sharded,
    const double (*points)[3],
    const int64_t* global_index,
    size_t n_owned,
    const double box[3][3],
    const bool periodic[3],
    struct VesinOptions options,
    struct VesinNeighborList* neighbors,
    const char** error_message
);

/* Device time (ms) of the packing kernel and of the NCCL exchange of the last
 * vesin_b200_sharded_neighbors on this handle; needs vesin_b200_set_profiling.
 * The stages of the local build come from vesin_b200_stage_times. Returns 1
 * when the last build was not timed. */
VESIN_API int vesin_b200_sharded_stage_times(const struct VesinB200Sharded* sharded, double* pack_ms, double* exchange_ms);

/*
 * No counterpart in the reference. Bytes per element of `distances` and
 * `vectors` as the LAST build left them in `neighbors`: 8 (double, every entry
 * point of the reference's API) or 4 (the *_f32 entry points, whose value arrays
 * hold floats behind the struct's double pointers); 0 for a list that holds
 * nothing. Code that wraps a list generically asks here before it reads.
 */
VESIN_API int vesin_b200_list_value_bytes(const struct VesinNeighborList* neighbors);

/*
 * No counterpart in the reference. Order-independent checksum of the list on
 * its device: checksum[0] and checksum[1] are sums (mod 2^64) of two 64-bit
 * hashes of every row (i, j, S), checksum[2] the same with the bits of the
 * distance mixed in, checksum[3] the number of rows. Arrays that were not
 * requested count as zeros. Lists of one system built in different orders or
 * split over ranks (add the ranks' sums) have equal checksums exactly when
 * they hold the same rows, up to hash collisions; the row hash is
 *   key = i*0x9e3779b97f4a7c15 + j*0xc2b2ae3d27d4eb4f + u32(Sx)*0x165667b19e3779f9
 *         + u32(Sy)*0x27d4eb2f165667c5 + u32(Sz)*0x85ebca77c2b2ae63   (mod 2^64)
 *   mix(x): x ^= x >> 33; x *= 0xff51afd7ed558ccd; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53; x ^= x >> 33
 *   rows add mix(key), mix(key ^ 0x5555555555555555), mix(key + bits(d)*0xd6e8feb86659fd93).
 */
VESIN_API int vesin_b200_list_checksum(const struct VesinNeighborList* neighbors, uint64_t checksum[4], const char** error_message);

/* Largest system vesin_b200_neighbors_no_alloc accepts. */
#define VESIN_B200_NO_ALLOC_MAX_POINTS 32768

/*
 * No counterpart in the reference: a list build that allocates nothing.
 *
 * For callers that may not call cudaMalloc when they need a list: an
 * application that handed all device memory to its own pool, a loop with a hard
 * bound on the latency of a step, a plugin inside a framework that forbids
 * allocations outside its allocator. vesin_neighbors allocates whenever a
 * system outgrows its workspace; this function never does. The caller passes
 * the inputs AND the output arrays (device memory on `device_id`, `capacity`
 * pairs each; shifts / distances / vectors may be NULL to skip them); the
 * scratch of the kernels is a fixed array of about 2.3 MB that every GPU holds from
 * library load to process exit. Hence:
 *   - `pairs` must be aligned to 16 bytes (the other arrays to their element:
 *     4 and 8 bytes); full lists are written fastest when `pairs` is aligned to
 *     32 bytes and `distances` / `vectors` to 16;
 *   - at most VESIN_B200_NO_ALLOC_MAX_POINTS points, larger systems get an error;
 *   - the list is unsorted, same pair set as vesin_neighbors;
 *   - when the list has more than `capacity` pairs the call fails, `*length`
 *     holds the number needed and the arrays hold nothing usable;
 *   - all calls share the scratch array (what must be zero is cleared at the
 *     start of each call); calls are serialised per device by a host lock, run
 *     on the legacy default stream and read a small header back twice with a
 *     blocking copy; the function returns when the list is complete. Work that
 *     overlapped on the GPU with another user of the same array would race:
 *     there is none inside one process;
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
