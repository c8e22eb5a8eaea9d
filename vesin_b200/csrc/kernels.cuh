// Device-side data structures and the launch wrappers of every kernel of the
// neighbor-list build. All kernels are written for sm_100a; none uses tensor
// cores: the build is a gather / compare / emit workload bounded by HBM
// bandwidth.
#ifndef VESIN_B200_KERNELS_CUH
#define VESIN_B200_KERNELS_CUH

#include <cstddef>
#include <cstdint>

#include <cuda_runtime.h>

#include "plan.hpp"

namespace vb200 {

/// Small block of device memory read back by the host (through a pinned
/// mirror) at the synchronisation points of a build.
struct DeviceHeader {
    unsigned long long min_key[3];   // order-preserving keys of the smallest coordinates
    unsigned long long max_key[3];   // ... and of the largest
    unsigned long long first_bad;    // smallest index of a point with a non-finite coordinate
    unsigned long long total_pairs;  // written by the scan over per-point pair counts
    unsigned long long mask_cursor;  // words of hit-mask storage claimed by the count pass
    unsigned long long pair_cursor;  // output elements claimed by the fused pass (= its pair total)
    unsigned long long run_cursor;   // runs of work units handed out by the fused pass (dynamic scheduling)
    unsigned int status;             // sticky error bits, see STATUS_*
    unsigned int pad;
    double box[9];                   // copy of the caller's box
    unsigned char periodic[8];       // copy of the caller's periodic flags
    unsigned long long halo_count[2]; // slab decomposition: records in the two halo messages of this build
};

constexpr unsigned int STATUS_MASK_OVERFLOW = 1u;
constexpr unsigned int STATUS_BAD_POINT = 2u;  // a point has a non-finite coordinate
constexpr unsigned int STATUS_PLAN_STALE = 4u; // box / periodicity / extent differ from what the plan was made for
constexpr unsigned int STATUS_ABORT_MASK = STATUS_BAD_POINT | STATUS_PLAN_STALE;
constexpr unsigned int STATUS_SINGULAR_BOX = 8u; // batches: the box of a system is not invertible
constexpr unsigned int STATUS_STENCIL_TOO_LARGE = 64u; // batches: the cutoff is hundreds of times the box of a system
constexpr unsigned int STATUS_HALO_OVERFLOW = 16u; // slab decomposition: a halo message holds fewer records than were selected
constexpr unsigned int STATUS_INDEX_RANGE = 32u;   // slab decomposition: a global index does not fit 31 bits
constexpr unsigned long long NO_BAD_POINT = ~0ull;

/// Cell-sorted copy of the points ("records"): original position, original
/// index and the wrap shift that brings the point into the box.
struct SortedPoints {
    double* pos;    // [n][3]
    int32_t* index; // [n]
    int32_t* shift; // [n][3]
};

/// Output arrays of the C ABI; null pointers are not written.
struct PairOutput {
    unsigned long long* pairs; // [total][2]
    int32_t* shifts;           // [total][3]
    double* distances;         // [total]
    double* vectors;           // [total][3]
    int values_float;          // distances / vectors are float arrays (fp32 entry point); decisions stay fp64
    int interleave_ok;         // set by launch_pairs: the arrays are aligned for the paired stores of full lists
};

/// Input coordinates: double (the reference's C API) or float (fp32 entry
/// point; converted exactly to double when read).
struct RealView {
    const void* data;
    int is_float;
};

/// Where the points of a build come from. Segment 0 is an array of the
/// caller (n0 points; `global_index`, when given, maps them to indices in a
/// larger system). Segments 1 and 2 exist for slab-decomposed systems only:
/// the halo messages received from the upper and the lower neighbour, rows of
/// 4 doubles each, row 0 = number of records, every other row = x, y, z and the
/// global index as raw 64 bits; a message holds at most `capacity` records.
/// Local indices: [0, n0) segment 0, [n0, n0 + capacity) segment 1,
/// [n0 + capacity, n0 + 2 capacity) segment 2; slots past a message's record
/// count are empty.
struct PointSource {
    RealView points;
    const long long* global_index;
    unsigned long long n0;
    const double* message[2];
    unsigned long long capacity;

    /// Size of the local index space.
    size_t n_index() const {
        return static_cast<size_t>(n0 + (message[0] != nullptr ? 2 * capacity : 0));
    }
};

inline PointSource flat_source(RealView points, size_t n) {
    return PointSource{points, nullptr, n, {nullptr, nullptr}, 0};
}

// ---- launch wrappers (all asynchronous on `stream`) ----

void launch_header_init(DeviceHeader* header, RealView box, const bool* periodic, cudaStream_t stream);

/// The same for a build that starts from the plan of the previous one: also
/// zeroes the `n_zero` counters of the cell histogram and compares box and
/// periodicity in device memory with what that plan was made for (a
/// difference sets STATUS_PLAN_STALE and every later kernel returns at once).
void launch_header_init_speculative(
    DeviceHeader* header, RealView box, const bool* periodic, int32_t* zero, size_t n_zero, const double expected_box[9],
    const bool expected_periodic[3], cudaStream_t stream
);

/// Header reset for a build whose box is known on the host (nothing is read
/// from device memory); also zeroes the `n_zero` counters of the cell histogram.
void launch_header_reset(DeviceHeader* header, int32_t* zero, size_t n_zero, cudaStream_t stream);

/// Min / max of every coordinate and the first non-finite point.
void launch_bounds(const PointSource& source, DeviceHeader* header, cudaStream_t stream);

/// Wrap into the cell, pick the cell, histogram with warp-aggregated atomics.
/// `check_points`: the plan is speculative; a non-finite point sets
/// STATUS_BAD_POINT (and first_bad), a point outside the cells of a
/// non-periodic direction STATUS_PLAN_STALE.
/// Bins the local indices [first, last). `chained`: the launch follows the
/// previous kernel of the stream as a programmatic dependent launch.
void launch_bin(
    const PointSource& source, size_t first, size_t last, const GridPlan& plan, int32_t* cell_of, int32_t* rank, int32_t* shift,
    int32_t* cell_count, DeviceHeader* header, bool check_points, bool chained, cudaStream_t stream
);

/// Exclusive scan of int32 counts into int32 starts (n + 1 entries).
/// `first_value` (device, may be null): what the first start is; lets a scan continue an earlier one.
void launch_scan_cells(
    const int32_t* counts, int32_t* starts, size_t n, void* tmp, cudaStream_t stream, const int32_t* first_value = nullptr
);
/// Exclusive scan of uint32 counts into uint64 starts (n + 1 entries); the
/// grand total also goes to *total.
void launch_scan_rows(
    const uint32_t* counts, unsigned long long* starts, size_t n, void* tmp, unsigned long long* total, cudaStream_t stream
);
/// Bytes of temporary storage the scans need for n elements.
size_t scan_tmp_bytes(size_t n);

/// Counting-sort scatter into the cell-sorted records. `n_cells`: cells of the
/// plan (cell_start[n_cells] is the number of records). `sorted_global`, when
/// not null, receives the global index of every record (31 bits; a larger one
/// sets STATUS_INDEX_RANGE). With [first, last): only these local indices are
/// scattered and only these records gathered (a slab build sorts its owned
/// points, whose records come first, before the halo has arrived).
void launch_scatter(
    const PointSource& source, const int32_t* cell_of, const int32_t* rank, const int32_t* shift, const int32_t* cell_start,
    size_t n_cells, SortedPoints sorted, int32_t* sorted_global, DeviceHeader* header, cudaStream_t stream, size_t first = 0,
    size_t last = static_cast<size_t>(-1)
);

/// Small systems: header reset and plan check (when `speculative`), binning,
/// scan and scatter in one launch of one CTA. Same results as
/// launch_header_init_speculative + launch_bin + launch_scan_cells +
/// launch_scatter (the order of the points inside a cell may differ, as it may
/// between two runs of those). Use when small_front_fits().
bool small_front_fits(size_t n_points, const GridPlan& plan);
void launch_small_front(
    RealView points, size_t n, const GridPlan& plan, int32_t* cell_of, int32_t* rank, int32_t* shift, int32_t* cell_start,
    SortedPoints sorted, DeviceHeader* header, RealView box, const bool* periodic, bool speculative, const double expected_box[9],
    const bool expected_periodic[3], cudaStream_t stream
);

/// Exclusive scan of uint64 counts into uint64 starts (n + 1 entries); the
/// grand total also goes to *total.
void launch_scan_units(
    const unsigned long long* counts, unsigned long long* starts, size_t n, void* tmp, unsigned long long* total, cudaStream_t stream
);

/// Sorted lists, pass 1: fp32 screen + fp64 decision for every (point,
/// candidate) of the full stencil; writes one hit bit per candidate and adds
/// the pairs of every point to row_count (which must start at zero).
void launch_count(
    const GridPlan& plan, const int32_t* cell_start, SortedPoints sorted, uint32_t* masks, unsigned long long mask_capacity,
    unsigned long long* unit_mask_base, uint32_t* unit_words, uint32_t* row_count, DeviceHeader* header, cudaStream_t stream
);

/// Sorted lists, pass 2: walks the hit bits and writes i, j, S, d, D, one row
/// per point in index order (row_start from the scan of row_count; row_fill
/// must start at zero).
void launch_emit(
    const GridPlan& plan, const int32_t* cell_start, SortedPoints sorted, const uint32_t* masks, const unsigned long long* unit_mask_base,
    const uint32_t* unit_words, const unsigned long long* row_start, uint32_t* row_fill, PairOutput out, cudaStream_t stream
);

/// Sorts the pairs inside every row by (second index, shift): `in` holds rows
/// [row_start[r], row_start[r + 1]), `out` receives the sorted rows.
/// (`duplicates_possible`: can a second index come twice in a row, i.e. is there a lattice
/// vector shorter than twice the cutoff? If not, the sort never looks at the shifts.)
void launch_sort_rows(
    const unsigned long long* row_start, size_t n_rows, PairOutput in, PairOutput out, bool duplicates_possible, cudaStream_t stream
);

/// Fused pass for unsorted lists: decides every candidate of the half-shell
/// stencil once and writes the pairs into ranges claimed from
/// header->pair_cursor. Blocks whose range would pass `capacity` (in pairs)
/// only count.
/// The indices written into the pairs are sorted.index: for a slab of a
/// decomposed system (plan.window_axis >= 0) the caller passes the records'
/// global indices there.
/// Slab builds cut along the last direction can launch the pair kernel in two parts: the
/// units whose candidates are all owned points (they need nothing from the halo), and the
/// units next to the halo. PAIR_PART_ALL launches both, back to back.
enum PairPart { PAIR_PART_ALL = 0, PAIR_PART_INTERIOR = 1, PAIR_PART_BOUNDARY = 2 };
/// Does the plan have units for PAIR_PART_INTERIOR?
bool pairs_have_interior(const GridPlan& plan);
void launch_pairs(
    const GridPlan& plan, const int32_t* cell_start, SortedPoints sorted, PairOutput out, unsigned long long capacity,
    DeviceHeader* header, cudaStream_t stream, size_t n_records = 0, int part = PAIR_PART_ALL
);
// (n_records: how many sorted records there are, if the caller knows; with it a launch of few
//  units can tell how many batches of candidates a unit holds and share them among CTAs)

// ---- batches of small systems (small_systems.cu) ----

/// A batch of independent systems stored back to back.
struct BatchInput {
    const void* points;                // [offsets[n_systems]][3], double or float (is_float)
    const unsigned long long* offsets; // [n_systems + 1], device memory
    const void* boxes;                 // [n_systems][9], double or float, or null (then nothing is periodic)
    const bool* periodic;              // [n_systems][3] or null (then nothing is periodic)
    unsigned n_systems;
    double cutoff;
    double cutoff2;
    int full;
    int global_indices; // pair indices count from the start of the batch, not of the system
    int is_float;       // points and boxes are float arrays (fp32 entry point); decisions stay fp64
};

/// Largest system the batch kernels accept (its points live in shared memory).
size_t small_systems_max_points();
void configure_small_systems();
/// Pass 1: pairs of every system -> system_count; the first non-finite point
/// and the first singular box are reported through the header.
/// (`any_for_cta_kernel`: some system is periodic or has more points than
/// molecules_max_points(), so the CTA-per-system kernel runs as well.)
void launch_small_count(
    const BatchInput& in, size_t max_points, bool any_for_cta_kernel, unsigned long long* system_count, DeviceHeader* header, cudaStream_t stream
);
/// Largest system the warp-per-system kernel takes.
size_t molecules_max_points();
/// Pass 2: every system writes its pairs at system_start[system]; a system whose block ends
/// beyond `capacity` elements writes nothing (the pass may run before the host knows the total).
void launch_small_emit(
    const BatchInput& in, size_t max_points, bool any_for_cta_kernel, const unsigned long long* system_start, PairOutput out,
    DeviceHeader* header, cudaStream_t stream, unsigned long long capacity = ~0ull
);

/// Order-independent checksum of a list: result[0], result[1] = two sums
/// (mod 2^64) of 64-bit hashes of every (i, j, S) row, result[2] = the same
/// with the bits of the distance mixed in (result[3] is cleared). Null
/// `shifts` count as zero shifts, null `distances` as zero distances.
void launch_checksum(
    const unsigned long long* pairs, const int32_t* shifts, const double* distances, int values_float, size_t n, unsigned long long* result,
    cudaStream_t stream
);

// ---- Verlet-skin cache (verlet.cu) ----

/// Device words of the cache of one list: what the check and the filter report.
struct VerletState {
    unsigned long long pair_cursor; // output elements claimed by the filter (= its pair total)
    int stale;                      // the candidates do not fit the inputs of this call
    int unpackable;                 // a candidate's shift does not fit its 10 bits
};

/// Candidates (pairs + shifts of a half list) to 12-byte records: the two
/// points as positions in the cell-sorted order `sorted_index` (position ->
/// index) of the build that found them, and the three shift components in 10
/// bits each; a shift outside [-512, 511] sets state->unpackable. `rank_of`:
/// n_points words of scratch (index -> position).
void launch_verlet_pack(
    const unsigned long long* pairs, const int32_t* shifts, size_t n, const int32_t* sorted_index, size_t n_points, uint32_t* rank_of,
    uint32_t* records, VerletState* state, cudaStream_t stream
);

/// Row p of `positions` (4 doubles, 32 bytes) = x, y, z of points[sorted_index[p]]
/// and sorted_index[p] as raw bits (nothing when state->stale is set).
void launch_verlet_positions(
    RealView points, const int32_t* sorted_index, size_t n_points, double* positions, const VerletState* state, cudaStream_t stream
);

/// Sets state->stale when some point moved further than (skin - corner
/// displacement of the box) / 2 from `reference_points`, when the box corners
/// moved by `skin` or more, or when the periodicity changed. `reference_box`
/// (9 doubles) and `reference_periodic` (3 bytes) live in device memory.
void launch_verlet_check(
    RealView points, RealView reference_points, size_t n, RealView box, const bool* periodic, const double* reference_box,
    const unsigned char* reference_periodic, double skin, VerletState* state, cudaStream_t stream
);

/// Writes the records within the cutoff (exact fp64 predicate on `positions`,
/// the current points in cell-sorted order, and the box) into ranges claimed from state->pair_cursor; a full list
/// gets both orientations of every kept record. Does nothing when
/// state->stale is set. Ranges past `capacity` are counted, not written.
void launch_verlet_filter(
    const uint32_t* records, size_t n, const double* positions, const int32_t* sorted_index, RealView box, double cutoff2, bool full,
    PairOutput out, unsigned long long capacity, VerletState* state, cudaStream_t stream
);

/// One-time per-device kernel attribute setup (shared-memory opt-in).
void configure_kernels();

} // namespace vb200

#endif
