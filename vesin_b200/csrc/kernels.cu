// Kernels of the neighbor-list build (sm_100a).
//
// Pipeline of one build (reference stages replaced are cited per kernel):
//   header_init -> bounds -> [host: grid plan] -> bin -> scan cells -> scatter
//   -> unsorted lists: pairs (decide + emit in one traversal; output ranges
//      are claimed with an atomic cursor)
//   -> sorted lists: count (hit masks + pairs per point) -> scan rows
//      -> [host: totals] -> emit (one row per point, in index order).
//
// Every candidate is decided ONCE, with the reference's exact fp64 arithmetic
// wherever an fp32 screen cannot decide; in the two-pass path the emit pass
// only walks the stored hit bits, so the passes can not disagree.
#include "kernels.cuh"

#include "emit.cuh"

#include <algorithm>
#include <cfloat>

namespace vb200 {

namespace {

constexpr int CTA_THREADS = 256;
constexpr int CTA_WARPS = CTA_THREADS / 32;
constexpr unsigned FULL_MASK = 0xffffffffu;

// ---------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------

__device__ __forceinline__ unsigned long long double_to_key(double x) {
    // order-preserving map double -> uint64
    unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(x));
    return (bits >> 63) ? ~bits : (bits | 0x8000000000000000ull);
}

__device__ __forceinline__ int floor_div(int a, int b) {
    int q = a / b;
    int r = a - q * b;
    return (r < 0) ? q - 1 : q;
}

__device__ __forceinline__ double load_real(const RealView& view, size_t k) {
    // float -> double is exact: fp32 inputs are decided with the same fp64 arithmetic
    return view.is_float ? static_cast<double>(static_cast<const float*>(view.data)[k]) : static_cast<const double*>(view.data)[k];
}

/// Records a halo message holds: its row 0, bounded by the capacity.
__device__ __forceinline__ unsigned long long message_records(const PointSource& source, int k) {
    const double claimed = (k ? source.message[1] : source.message[0])[0];
    const unsigned long long count = (claimed > 0.0) ? static_cast<unsigned long long>(claimed) : 0ull;
    return (count < source.capacity) ? count : source.capacity;
}

/// Point with local index i; false for an empty slot of a halo message.
/// Without HALO the source is a plain array.
template <bool HALO>
__device__ __forceinline__ bool load_point(const PointSource& source, size_t i, double& x, double& y, double& z) {
    if (!HALO || i < source.n0) {
        x = load_real(source.points, 3 * i + 0);
        y = load_real(source.points, 3 * i + 1);
        z = load_real(source.points, 3 * i + 2);
        return true;
    }
    size_t r = i - source.n0;
    const int k = (r >= source.capacity) ? 1 : 0;
    r -= k * source.capacity;
    if (r >= message_records(source, k)) {
        return false;
    }
    const double* row = (k ? source.message[1] : source.message[0]) + 4 * (r + 1);
    x = row[0];
    y = row[1];
    z = row[2];
    return true;
}

/// One coordinate of the point with local index i (which is not an empty slot).
template <bool HALO>
__device__ __forceinline__ double load_coordinate(const PointSource& source, size_t i, size_t c) {
    if (!HALO || i < source.n0) {
        return load_real(source.points, 3 * i + c);
    }
    size_t r = i - source.n0;
    const int k = (r >= source.capacity) ? 1 : 0;
    r -= k * source.capacity;
    return (k ? source.message[1] : source.message[0])[4 * (r + 1) + c];
}

/// Index of the point in the whole system.
template <bool HALO>
__device__ __forceinline__ long long global_index_of(const PointSource& source, size_t i) {
    if (!HALO || i < source.n0) {
        return (source.global_index != nullptr) ? source.global_index[i] : static_cast<long long>(i);
    }
    size_t r = i - source.n0;
    const int k = (r >= source.capacity) ? 1 : 0;
    r -= k * source.capacity;
    return __double_as_longlong((k ? source.message[1] : source.message[0])[4 * (r + 1) + 3]);
}

// Programmatic dependent launch: the kernels of a build form a chain on one
// stream, each reading what the one before wrote. A kernel lets the next one
// be scheduled as soon as all of its own blocks are running, and waits for the
// one before it (complete, memory visible) before it touches anything. Launch
// latency and block scheduling of the short kernels then overlap with the tail
// of their predecessor. Both instructions do nothing in a plain launch.
__device__ __forceinline__ void let_next_kernel_start() {
    asm volatile("griddepcontrol.launch_dependents;");
}
__device__ __forceinline__ void wait_for_previous_kernel() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned mask;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(mask));
    return mask;
}

/// Exclusive scan of one value per thread over the whole CTA (256 threads).
/// `warp_sums` is CTA_WARPS + 1 ints of shared memory; returns the exclusive
/// prefix and stores the CTA total in warp_sums[CTA_WARPS] (every thread
/// stores the same value, so the total is visible to the caller at once).
/// One barrier inside; two calls must be separated by another barrier.
/// Only the first ACTIVE_WARPS warps may hold non-zero values (the others
/// skip the shuffles).
template <int ACTIVE_WARPS = CTA_WARPS>
__device__ __forceinline__ int block_exclusive_scan(int value, int* warp_sums) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    int inclusive = value;
    if (ACTIVE_WARPS == CTA_WARPS || warp < ACTIVE_WARPS) {
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
            int up = __shfl_up_sync(FULL_MASK, inclusive, offset);
            if (lane >= offset) {
                inclusive += up;
            }
        }
        if (lane == 31) {
            warp_sums[warp] = inclusive;
        }
    }
    __syncthreads();
    int before = 0;
    int total = 0;
#pragma unroll
    for (int w = 0; w < ACTIVE_WARPS; w++) {
        const int sum = warp_sums[w];
        total += sum;
        if (w < warp) {
            before += sum;
        }
    }
    if (lane == 0) {
        warp_sums[CTA_WARPS] = total;
    }
    __syncwarp();
    return before + inclusive - value;
}

// Packed fp32 arithmetic of sm_100: two independent IEEE operations per instruction.
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
    unsigned long long packed;
    asm("mov.b64 %0, {%1, %2};" : "=l"(packed) : "f"(lo), "f"(hi));
    return packed;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long packed, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(packed));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

/// Position of the n-th (counting from 0) set bit of w. For a word with n or
/// fewer set bits the result is some position below 32.
__device__ __forceinline__ int select_bit(unsigned w, int n) {
    int pos = 0;
    int c = __popc(w & 0xffffu);
    if (n >= c) {
        n -= c;
        pos = 16;
        w >>= 16;
    }
    c = __popc(w & 0xffu);
    if (n >= c) {
        n -= c;
        pos += 8;
        w >>= 8;
    }
    c = __popc(w & 0xfu);
    if (n >= c) {
        n -= c;
        pos += 4;
        w >>= 4;
    }
    c = __popc(w & 0x3u);
    if (n >= c) {
        n -= c;
        pos += 2;
        w >>= 2;
    }
    c = static_cast<int>(w & 1u);
    if (n >= c) {
        pos += 1;
    }
    return pos;
}

// ---------------------------------------------------------------------------
// header + bounds
// Replaces compute_bounding_box (vesin/src/cuda/cell_list.cu:69-133, one block
// for all points) and the finite check of the CPU path
// (vesin/src/types.hpp:159-178).
// ---------------------------------------------------------------------------

// ---------------------------------------------------------------------------
// validation of a speculative plan
// The host builds the grid plan from the box, periodicity and bounds it saw at
// the end of the PREVIOUS build on the same list, and launches the whole build
// without waiting for a read-back. The kernels compare that assumption with
// what is in device memory now: the first kernel checks box and periodicity
// bit for bit, the binning kernel checks every point (finite, inside the cell
// window of non-periodic directions). When it does not hold they set
// STATUS_PLAN_STALE or STATUS_BAD_POINT, every later kernel of the build
// returns at once, and the host plans again from bounds it then has computed.
// Replaces the two blocking read-backs of check_box
// (vesin/src/vesin_cuda.cpp:393-399).
// ---------------------------------------------------------------------------

struct ExpectedInputs {
    double box[9];
    int periodic[3];
};

/// Reset of the header by the first threads of one block: box and periodicity
/// are copied, cursors and status cleared.
__device__ __forceinline__ void reset_header(DeviceHeader* header, const RealView& box, const bool* periodic, int t) {
    if (t < 3) {
        header->min_key[t] = ~0ull;
        header->max_key[t] = 0ull;
        if (periodic != nullptr) {
            header->periodic[t] = periodic[t] ? 1 : 0;
        }
    }
    if (t < 9 && box.data != nullptr) {
        header->box[t] = load_real(box, t);
    }
    if (t < 2) {
        header->halo_count[t] = 0;
    }
    if (t == 0) {
        header->first_bad = NO_BAD_POINT;
        header->total_pairs = 0;
        header->mask_cursor = 0;
        header->pair_cursor = 0;
        header->run_cursor = 0;
        header->status = 0;
    }
}

/// Box and periodicity in device memory against what the plan was made for;
/// call after a barrier that follows reset_header.
__device__ __forceinline__ void check_box(DeviceHeader* header, const RealView& box, const bool* periodic, const ExpectedInputs& expected, int t) {
    bool same = true;
    if (t < 9) {
        same = __double_as_longlong(load_real(box, t)) == __double_as_longlong(expected.box[t]);
    }
    if (t < 3) {
        same = same && ((periodic[t] ? 1 : 0) == (expected.periodic[t] != 0 ? 1 : 0));
    }
    if (!same) {
        atomicOr(&header->status, STATUS_PLAN_STALE);
    }
}

/// Resets the header (block 0) and zeroes `n_zero` counters (all blocks). With
/// `validate`, box and periodicity are compared with what the plan was made for.
__global__ void __launch_bounds__(CTA_THREADS) header_init_kernel(
    DeviceHeader* header, const RealView box, const bool* periodic, int32_t* __restrict__ zero, size_t n_zero, const int validate,
    const ExpectedInputs expected
) {
    let_next_kernel_start();
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t k = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; k < n_zero; k += stride) {
        zero[k] = 0;
    }
    if (blockIdx.x != 0) {
        return;
    }
    reset_header(header, box, periodic, threadIdx.x);
    if (validate) {
        __syncthreads(); // the status word has been reset
        check_box(header, box, periodic, expected, threadIdx.x);
    }
}

template <bool HALO>
__global__ void __launch_bounds__(CTA_THREADS) bounds_kernel(const PointSource source, size_t n, DeviceHeader* header) {
    double lo[3] = {DBL_MAX, DBL_MAX, DBL_MAX};
    double hi[3] = {-DBL_MAX, -DBL_MAX, -DBL_MAX};
    unsigned long long bad = NO_BAD_POINT;

    size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        double r[3];
        if (!load_point<HALO>(source, i, r[0], r[1], r[2])) {
            continue;
        }
#pragma unroll
        for (int c = 0; c < 3; c++) {
            double x = r[c];
            if (isfinite(x)) {
                lo[c] = fmin(lo[c], x);
                hi[c] = fmax(hi[c], x);
            } else if (i < bad) {
                bad = i;
            }
        }
    }

#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
#pragma unroll
        for (int c = 0; c < 3; c++) {
            lo[c] = fmin(lo[c], __shfl_xor_sync(FULL_MASK, lo[c], offset));
            hi[c] = fmax(hi[c], __shfl_xor_sync(FULL_MASK, hi[c], offset));
        }
        unsigned long long other = __shfl_xor_sync(FULL_MASK, bad, offset);
        bad = (other < bad) ? other : bad;
    }

    __shared__ double s_lo[CTA_WARPS][3];
    __shared__ double s_hi[CTA_WARPS][3];
    __shared__ unsigned long long s_bad[CTA_WARPS];
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    if (lane == 0) {
        for (int c = 0; c < 3; c++) {
            s_lo[warp][c] = lo[c];
            s_hi[warp][c] = hi[c];
        }
        s_bad[warp] = bad;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < CTA_WARPS; w++) {
            for (int c = 0; c < 3; c++) {
                lo[c] = fmin(lo[c], s_lo[w][c]);
                hi[c] = fmax(hi[c], s_hi[w][c]);
            }
            bad = (s_bad[w] < bad) ? s_bad[w] : bad;
        }
        for (int c = 0; c < 3; c++) {
            if (lo[c] <= hi[c]) {
                atomicMin(&header->min_key[c], double_to_key(lo[c]));
                atomicMax(&header->max_key[c], double_to_key(hi[c]));
            }
        }
        if (bad != NO_BAD_POINT) {
            atomicMin(&header->first_bad, bad);
        }
    }
}


// ---------------------------------------------------------------------------
// bin: wrap + cell + histogram
// Replaces assign_cell_indices + count_particles_per_cell
// (vesin/src/cuda/cell_list.cu:279-345) and CellList::add_point
// (vesin/src/cpu_cell_list.cpp:353-374).
// ---------------------------------------------------------------------------

// Slab decomposition. Along the cut direction a rank's cells are layers 0 ...
// n - 1 in space: 0 and n - 1 hold halo points, the layers between hold owned
// points. They are STORED in the order owned layers, upper halo layer, lower
// halo layer, so that the cell-sorted records of the owned points come first
// and do not depend on the halo: the owned points can be sorted while the
// halo is still on its way.
__device__ __forceinline__ int window_storage_layer(int layer, int n) {
    return (layer == 0) ? n - 1 : layer - 1;
}
__device__ __forceinline__ int window_space_layer(int stored, int n) {
    return (stored == n - 1) ? 0 : stored + 1;
}

/// Cell (linear index) and wrap shift of point i. `check`: the plan is
/// speculative; a point with a non-finite coordinate or outside the cells of a
/// non-periodic direction refuses it.
__device__ __forceinline__ int locate_point(
    double rx, double ry, double rz, size_t i, const GridPlan& plan, DeviceHeader* header, const int check, int wrap[3]
) {
    if (check && !(isfinite(rx) && isfinite(ry) && isfinite(rz))) {
        atomicMin(&header->first_bad, static_cast<unsigned long long>(i));
        atomicOr(&header->status, STATUS_BAD_POINT);
    }

    int cell[3];
#pragma unroll
    for (int k = 0; k < 3; k++) {
        double t = rx * plan.Hinv[0][k] + ry * plan.Hinv[1][k] + rz * plan.Hinv[2][k];
        double g = floor((t - plan.t0[k]) * plan.scale[k]);
        g = fmin(fmax(g, -1.0e9), 1.0e9);
        int gi = static_cast<int>(g);
        if (k == plan.window_axis) {
            // slab decomposition: the image shift is whatever brings the point
            // into this rank's window; owned points live in the inner layers,
            // halo points in the first or the last layer
            double image = floor(t - plan.t0[k]);
            image = fmin(fmax(image, -1.0e9), 1.0e9);
            wrap[k] = static_cast<int>(image);
            int layer = static_cast<int>(fmin(fmax(floor((t - image - plan.t0[k]) * plan.scale[k]), -1.0), 1.0e9));
            const int last = plan.n_cells[k] - 1;
            if (i < static_cast<size_t>(plan.n_owned)) {
                layer = min(max(layer, 1), last - 1);
            } else {
                layer = (2 * layer < last) ? 0 : last;
            }
            cell[k] = window_storage_layer(layer, last + 1);
        } else if (plan.periodic[k]) {
            int q = floor_div(gi, plan.n_cells[k]);
            wrap[k] = q;
            cell[k] = gi - q * plan.n_cells[k];
        } else {
            wrap[k] = 0;
            cell[k] = min(max(gi, 0), plan.n_cells[k] - 1);
            if (check && cell[k] != gi && (*reinterpret_cast<volatile unsigned*>(&header->status) & STATUS_PLAN_STALE) == 0) {
                atomicOr(&header->status, STATUS_PLAN_STALE); // the point left the window the plan covers
            }
        }
    }
    return (cell[2] * plan.n_cells[1] + cell[1]) * plan.n_cells[0] + cell[0];
}

template <bool HALO>
__global__ void __launch_bounds__(CTA_THREADS) bin_kernel(
    const PointSource source, size_t first, size_t last, const GridPlan plan, int32_t* __restrict__ cell_of, int32_t* __restrict__ rank,
    int32_t* __restrict__ shift, int32_t* __restrict__ cell_count, DeviceHeader* header, const int check
) {
    let_next_kernel_start();
    wait_for_previous_kernel();
    if (header->status & STATUS_ABORT_MASK) {
        return;
    }
    size_t i = first + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    double rx = 0.0, ry = 0.0, rz = 0.0;
    bool active = i < last && load_point<HALO>(source, i, rx, ry, rz);
    if (HALO && i < last && i >= source.n0 && (i - source.n0) % source.capacity == 0) {
        // first slot of a message: report how many records it brought
        const int k = (i - source.n0 >= source.capacity) ? 1 : 0;
        const double claimed = (k ? source.message[1] : source.message[0])[0];
        const unsigned long long count = (claimed > 0.0) ? static_cast<unsigned long long>(claimed) : 0ull;
        header->halo_count[k] = count;
        if (count > source.capacity) {
            atomicOr(&header->status, STATUS_HALO_OVERFLOW);
        }
    }
    unsigned active_mask = __ballot_sync(FULL_MASK, active);
    if (!active) {
        return;
    }
    int wrap[3];
    const int linear = locate_point(rx, ry, rz, i, plan, header, check, wrap);

    // warp-aggregated histogram: one atomic per distinct cell in the warp
    unsigned peers = __match_any_sync(active_mask, linear);
    int leader = __ffs(peers) - 1;
    int lane = threadIdx.x & 31;
    int base = 0;
    if (lane == leader) {
        base = atomicAdd(&cell_count[linear], __popc(peers));
    }
    base = __shfl_sync(peers, base, leader);

    cell_of[i] = linear;
    rank[i] = base + __popc(peers & lanemask_lt());
    shift[3 * i + 0] = wrap[0];
    shift[3 * i + 1] = wrap[1];
    shift[3 * i + 2] = wrap[2];
}

// ---------------------------------------------------------------------------
// scans
// Replaces prefix_sum_cells (vesin/src/cuda/cell_list.cu:347-390, a single
// block whose 8192-cell limit caps the reference's grid) and the pre-sized
// output + global append counter (vesin/src/vesin_cuda.cpp:866-886,
// cell_list.cu:643-668): per-point counts are scanned into private rows.
// Two launches (tile sums; apply, every block adding up the sums of the tiles
// before its own) up to 2048 tiles, three beyond (tile sums, spine, apply); no
// inter-CTA waiting.
// ---------------------------------------------------------------------------

constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_TILE = CTA_THREADS * SCAN_ITEMS;

template <typename TIn>
__global__ void __launch_bounds__(CTA_THREADS) scan_tile_sums_kernel(const TIn* __restrict__ in, size_t n, unsigned long long* __restrict__ tile_sums) {
    let_next_kernel_start();
    wait_for_previous_kernel();
    size_t base = static_cast<size_t>(blockIdx.x) * SCAN_TILE;
    unsigned long long sum = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        size_t idx = base + static_cast<size_t>(k) * CTA_THREADS + threadIdx.x;
        if (idx < n) {
            sum += static_cast<unsigned long long>(in[idx]);
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        sum += __shfl_xor_sync(FULL_MASK, sum, offset);
    }
    __shared__ unsigned long long s_sum[CTA_WARPS];
    if ((threadIdx.x & 31) == 0) {
        s_sum[threadIdx.x >> 5] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long total = 0;
        for (int w = 0; w < CTA_WARPS; w++) {
            total += s_sum[w];
        }
        tile_sums[blockIdx.x] = total;
    }
}

/// One CTA turns the tile sums into exclusive tile offsets, in place.
__global__ void __launch_bounds__(CTA_THREADS) scan_spine_kernel(unsigned long long* tile_sums, size_t n_tiles, unsigned long long* total_out) {
    __shared__ unsigned long long s_warp[CTA_WARPS];
    __shared__ unsigned long long s_carry;
    if (threadIdx.x == 0) {
        s_carry = 0;
    }
    __syncthreads();
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    for (size_t start = 0; start < n_tiles; start += CTA_THREADS) {
        size_t idx = start + threadIdx.x;
        unsigned long long value = (idx < n_tiles) ? tile_sums[idx] : 0;
        unsigned long long inclusive = value;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
            unsigned long long up = __shfl_up_sync(FULL_MASK, inclusive, offset);
            if (lane >= offset) {
                inclusive += up;
            }
        }
        if (lane == 31) {
            s_warp[warp] = inclusive;
        }
        __syncthreads();
        unsigned long long warp_prefix = 0;
        for (int w = 0; w < warp; w++) {
            warp_prefix += s_warp[w];
        }
        unsigned long long carry = s_carry;
        if (idx < n_tiles) {
            tile_sums[idx] = carry + warp_prefix + inclusive - value;
        }
        __syncthreads();
        if (threadIdx.x == CTA_THREADS - 1) {
            s_carry = carry + warp_prefix + inclusive;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0 && total_out != nullptr) {
        *total_out = s_carry;
    }
}

/// SPINE: `tile_offsets` still holds the sums of the tiles (the spine kernel
/// did not run): every block adds up the sums of the tiles before its own.
template <typename TIn, typename TOut, bool SPINE>
__global__ void __launch_bounds__(CTA_THREADS) scan_apply_kernel(
    const TIn* __restrict__ in, TOut* __restrict__ out, size_t n, const unsigned long long* __restrict__ tile_offsets,
    unsigned long long* __restrict__ total_out, const TOut* __restrict__ first_value
) {
    let_next_kernel_start();
    wait_for_previous_kernel();
    // each thread owns SCAN_ITEMS consecutive elements
    size_t base = static_cast<size_t>(blockIdx.x) * SCAN_TILE + static_cast<size_t>(threadIdx.x) * SCAN_ITEMS;
    unsigned long long values[SCAN_ITEMS];
    unsigned long long local = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        size_t idx = base + k;
        values[k] = (idx < n) ? static_cast<unsigned long long>(in[idx]) : 0;
        local += values[k];
    }
    // exclusive scan of `local` over the CTA (64-bit)
    int lane = threadIdx.x & 31;
    int warp = threadIdx.x >> 5;
    unsigned long long inclusive = local;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        unsigned long long up = __shfl_up_sync(FULL_MASK, inclusive, offset);
        if (lane >= offset) {
            inclusive += up;
        }
    }
    __shared__ unsigned long long s_warp[CTA_WARPS];
    __shared__ unsigned long long s_before[CTA_WARPS];
    if (lane == 31) {
        s_warp[warp] = inclusive;
    }
    unsigned long long tile_offset = 0;
    if (SPINE) {
        unsigned long long before = 0;
        for (unsigned t = threadIdx.x; t < blockIdx.x; t += CTA_THREADS) {
            before += tile_offsets[t];
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            before += __shfl_xor_sync(FULL_MASK, before, offset);
        }
        if (lane == 0) {
            s_before[warp] = before;
        }
    } else {
        tile_offset = tile_offsets[blockIdx.x];
    }
    __syncthreads();
    if (SPINE) {
#pragma unroll
        for (int w = 0; w < CTA_WARPS; w++) {
            tile_offset += s_before[w];
        }
    }
    unsigned long long prefix = tile_offset + inclusive - local;
    if (first_value != nullptr) {
        prefix += static_cast<unsigned long long>(*first_value); // the scan continues an earlier one
    }
    for (int w = 0; w < warp; w++) {
        prefix += s_warp[w];
    }
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        size_t idx = base + k;
        if (idx < n) {
            out[idx] = static_cast<TOut>(prefix);
        }
        prefix += values[k];
        if (idx + 1 == n) {
            out[n] = static_cast<TOut>(prefix);
            if (SPINE && total_out != nullptr) {
                *total_out = prefix;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// scatter
// Replaces scatter_particles (vesin/src/cuda/cell_list.cu:392-421); the slot
// inside the cell was already handed out by the histogram, so there is no
// second atomic. Two kernels: indices are scattered, records are gathered.
// ---------------------------------------------------------------------------

/// Step 1: where does point i go? Only its index is scattered (4 bytes per point).
template <bool HALO>
__global__ void __launch_bounds__(CTA_THREADS) scatter_index_kernel(
    const PointSource source, size_t first, size_t last, const int32_t* __restrict__ cell_of, const int32_t* __restrict__ rank,
    const int32_t* __restrict__ cell_start, int32_t* __restrict__ sorted_index, const DeviceHeader* __restrict__ header
) {
    let_next_kernel_start();
    wait_for_previous_kernel();
    size_t i = first + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= last || (header->status & STATUS_ABORT_MASK)) {
        return;
    }
    if (HALO && i >= source.n0) {
        const size_t r = i - source.n0;
        const int k = (r >= source.capacity) ? 1 : 0;
        if (r - k * source.capacity >= message_records(source, k)) {
            return; // empty slot of a halo message
        }
    }
    size_t p = static_cast<size_t>(cell_start[cell_of[i]]) + rank[i];
    sorted_index[p] = static_cast<int32_t>(i);
}

/// Step 2: the records are gathered, one coordinate per thread, so that every
/// store instruction writes one contiguous span whatever the order of the
/// input (a scatter of whole records writes partial sectors all over the
/// arrays when neighbouring points are far apart in the input).
/// Records [first, last). `n_records` (device): number of records, i.e.
/// cell_start[n_cells]; the range may reach past it when the local index space
/// holds empty slots.
template <bool HALO>
__global__ void __launch_bounds__(CTA_THREADS) gather_records_kernel(
    const PointSource source, size_t first, size_t last, const int32_t* __restrict__ n_records, const int32_t* __restrict__ shift,
    SortedPoints sorted, int32_t* __restrict__ sorted_global, DeviceHeader* __restrict__ header
) {
    let_next_kernel_start();
    wait_for_previous_kernel();
    size_t f = 3 * first + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (f >= 3 * last || (header->status & STATUS_ABORT_MASK)) {
        return;
    }
    size_t p = f / 3;
    size_t c = f - 3 * p;
    if (HALO && n_records != nullptr && p >= static_cast<size_t>(*n_records)) {
        return;
    }
    size_t i = static_cast<size_t>(sorted.index[p]);
    sorted.pos[f] = load_coordinate<HALO>(source, i, c);
    sorted.shift[f] = shift[3 * i + c];
    if (c == 0 && sorted_global != nullptr) {
        const long long global = global_index_of<HALO>(source, i);
        if (global < 0 || global > 0x7fffffffll) {
            atomicOr(&header->status, STATUS_INDEX_RANGE);
        }
        sorted_global[p] = static_cast<int32_t>(global);
    }
}

// ---------------------------------------------------------------------------
// cell list of a small system in one launch
// A few thousand points do not fill the GPU; what their build costs is the
// chain of launches. One CTA does what header_init, bin, the scan and the two
// scatter kernels do for large systems: histogram in shared memory, scan,
// scatter, with the same arithmetic per point.
// ---------------------------------------------------------------------------

constexpr int SMALL_FRONT_THREADS = 1024;
constexpr int SMALL_FRONT_MAX_CELLS = 4096;
constexpr size_t SMALL_FRONT_MAX_POINTS = 16384;

__global__ void __launch_bounds__(SMALL_FRONT_THREADS) small_front_kernel(
    const RealView points, size_t n, const GridPlan plan, int32_t* __restrict__ cell_of, int32_t* __restrict__ rank,
    int32_t* __restrict__ shift, int32_t* __restrict__ cell_start, SortedPoints sorted, DeviceHeader* header, const RealView box,
    const bool* periodic, const int speculative, const ExpectedInputs expected
) {
    __shared__ int hist[SMALL_FRONT_MAX_CELLS];
    __shared__ int warp_sums[SMALL_FRONT_THREADS / 32];
    __shared__ unsigned s_status;
    let_next_kernel_start();
    wait_for_previous_kernel();
    const int t = threadIdx.x;
    const int n_cells = plan.n_cells_total;
    if (speculative) {
        // the build starts here: reset the header, then check the plan's assumptions
        reset_header(header, box, periodic, t);
    }
    for (int c = t; c < n_cells; c += SMALL_FRONT_THREADS) {
        hist[c] = 0;
    }
    __syncthreads();
    if (speculative) {
        check_box(header, box, periodic, expected, t);
        __syncthreads();
    }
    // one thread reads the status for all: the binning below may set bits while others still look
    if (t == 0) {
        s_status = *reinterpret_cast<volatile unsigned*>(&header->status);
    }
    __syncthreads();
    if (s_status & STATUS_ABORT_MASK) {
        return;
    }

    // ---- histogram: the value the atomic returns is the slot of the point in its cell ----
    for (size_t i = t; i < n; i += SMALL_FRONT_THREADS) {
        int wrap[3];
        const int linear = locate_point(
            load_real(points, 3 * i + 0), load_real(points, 3 * i + 1), load_real(points, 3 * i + 2), i, plan, header, speculative, wrap
        );
        cell_of[i] = linear;
        rank[i] = atomicAdd(&hist[linear], 1);
        shift[3 * i + 0] = wrap[0];
        shift[3 * i + 1] = wrap[1];
        shift[3 * i + 2] = wrap[2];
    }
    __syncthreads();

    // ---- exclusive scan of the histogram: consecutive cells per thread ----
    const int per_thread = (n_cells + SMALL_FRONT_THREADS - 1) / SMALL_FRONT_THREADS; // at most 4
    const int first = t * per_thread;
    int counts[SMALL_FRONT_MAX_CELLS / SMALL_FRONT_THREADS];
    int mine = 0;
#pragma unroll
    for (int k = 0; k < SMALL_FRONT_MAX_CELLS / SMALL_FRONT_THREADS; k++) {
        const int c = first + k;
        counts[k] = (k < per_thread && c < n_cells) ? hist[c] : 0;
        mine += counts[k];
    }
    const int lane = t & 31;
    const int warp = t >> 5;
    int inclusive = mine;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        const int up = __shfl_up_sync(FULL_MASK, inclusive, offset);
        if (lane >= offset) {
            inclusive += up;
        }
    }
    if (lane == 31) {
        warp_sums[warp] = inclusive;
    }
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; w++) {
        before += warp_sums[w];
    }
    int prefix = before + inclusive - mine;
    __syncthreads(); // every thread has read its counts: the histogram becomes the table of cell starts
#pragma unroll
    for (int k = 0; k < SMALL_FRONT_MAX_CELLS / SMALL_FRONT_THREADS; k++) {
        const int c = first + k;
        if (k < per_thread && c < n_cells) {
            hist[c] = prefix;
            cell_start[c] = prefix;
            prefix += counts[k];
        }
    }
    if (t == SMALL_FRONT_THREADS - 1) {
        cell_start[n_cells] = prefix;
    }
    __syncthreads();

    // ---- scatter into the cell-sorted records (cell_of, rank, shift were written by this thread) ----
    for (size_t i = t; i < n; i += SMALL_FRONT_THREADS) {
        const size_t p = static_cast<size_t>(hist[cell_of[i]]) + rank[i];
        sorted.pos[3 * p + 0] = load_real(points, 3 * i + 0);
        sorted.pos[3 * p + 1] = load_real(points, 3 * i + 1);
        sorted.pos[3 * p + 2] = load_real(points, 3 * i + 2);
        sorted.index[p] = static_cast<int32_t>(i);
        sorted.shift[3 * p + 0] = shift[3 * i + 0];
        sorted.shift[3 * p + 1] = shift[3 * i + 1];
        sorted.shift[3 * p + 2] = shift[3 * i + 2];
    }
}

// ---------------------------------------------------------------------------
// stencil traversal shared by the count and emit passes
// Replaces CellList::foreach_pair (vesin/src/cpu_cell_list.cpp:376-451) and
// the traversal of find_neighbors_cell_list (vesin/src/cuda/cell_list.cu:509-591).
//
// One CTA owns one work unit: a pencil of `plan.pencil` consecutive cells
// along x, whose points ("home points") are one contiguous run of the
// cell-sorted records. The cells of the pencil's stencil are "segments": runs
// of cell-sorted points, each with the image shift q picked up by wrapping
// the cell index. The concatenation of all segments numbers the candidates of
// every home point ("slots"); one bit per slot and per home point is the hit
// mask. Stencils with more than SEG_MAX cells are walked in groups whose slot
// numbering starts on a fresh 32-slot word.
// ---------------------------------------------------------------------------

constexpr int SEG_MAX = 128;
constexpr int TILE_POINTS = 32; // home points handled at once: one per lane

struct SegmentTable {
    /// Image shift of the segment, 21 bits per direction (a stencil never reaches further:
    /// MAX_STENCIL_CELLS), and in the top bit a flag: may a point pair with its own image in
    /// this segment (sorted lists) / does the segment hold owned points (slab decomposition)?
    unsigned long long image[SEG_MAX];
    int start[SEG_MAX];     // first cell-sorted point of the segment
    int slot0[SEG_MAX + 1]; // exclusive prefix of the segment lengths
    int scan_tmp[CTA_WARPS + 1];
};
static_assert(MAX_STENCIL_CELLS <= (1 << 20), "image shifts are stored in 21 bits");

__device__ __forceinline__ unsigned long long pack_segment_image(int q0, int q1, int q2, int flag) {
    return static_cast<unsigned long long>(q0 & 0x1fffff) | (static_cast<unsigned long long>(q1 & 0x1fffff) << 21) |
           (static_cast<unsigned long long>(q2 & 0x1fffff) << 42) | (static_cast<unsigned long long>(flag & 1) << 63);
}
__device__ __forceinline__ void unpack_segment_image(unsigned long long image, int& q0, int& q1, int& q2) {
    // sign extension of 21-bit fields
    q0 = (static_cast<int>(image) << 11) >> 11;
    q1 = (static_cast<int>(image >> 21) << 11) >> 11;
    q2 = (static_cast<int>(image >> 42) << 11) >> 11;
}
__device__ __forceinline__ int segment_flag(unsigned long long image) {
    return static_cast<int>(image >> 63);
}

struct Unit {
    int c0, c1, c2; // first cell of the pencil
    int cells;      // cells in the pencil (the last pencil of a row may be shorter)
    int begin;      // first cell-sorted home point
    int n_home;     // number of home points
    int n_stencil;  // cells in the stencil of this pencil
};

__device__ __forceinline__ Unit unit_of(const GridPlan& plan, const int32_t* __restrict__ cell_start, int u) {
    Unit unit;
    const int pencils_x = (plan.n_cells[0] + plan.pencil - 1) / plan.pencil;
    const int px = u % pencils_x;
    unit.c1 = (u / pencils_x) % plan.n_cells[1];
    unit.c2 = u / (pencils_x * plan.n_cells[1]);
    unit.c0 = px * plan.pencil;
    unit.cells = min(plan.pencil, plan.n_cells[0] - unit.c0);
    const int first = (unit.c2 * plan.n_cells[1] + unit.c1) * plan.n_cells[0] + unit.c0;
    unit.begin = cell_start[first];
    unit.n_home = cell_start[first + unit.cells] - unit.begin;
    unit.n_stencil = (unit.cells + 2 * plan.n_search[0]) * (2 * plan.n_search[1] + 1) * (2 * plan.n_search[2] + 1);
    return unit;
}

/// The unit after `unit` (u + 1) without the divisions of unit_of.
__device__ __forceinline__ void next_unit(const GridPlan& plan, const int32_t* __restrict__ cell_start, Unit& unit) {
    unit.c0 += plan.pencil;
    if (unit.c0 >= plan.n_cells[0]) {
        unit.c0 = 0;
        unit.c1 += 1;
        if (unit.c1 >= plan.n_cells[1]) {
            unit.c1 = 0;
            unit.c2 += 1;
        }
    }
    unit.cells = min(plan.pencil, plan.n_cells[0] - unit.c0);
    const int first = (unit.c2 * plan.n_cells[1] + unit.c1) * plan.n_cells[0] + unit.c0;
    unit.begin = cell_start[first];
    unit.n_home = cell_start[first + unit.cells] - unit.begin;
}

__device__ __forceinline__ bool half_rule(int s0, int s1, int s2) {
    // which of S / -S a half list keeps for a point paired with its own
    // image (vesin/src/cpu_cell_list.cpp:107-132)
    int sum = s0 + s1 + s2;
    if (sum < 0) {
        return false;
    }
    if (sum == 0 && (s2 < 0 || (s2 == 0 && s1 < 0))) {
        return false;
    }
    return true;
}

/// Fill the table for segment group `group` of a unit. Returns the number of
/// slots of the group. Ends with a __syncthreads().
__device__ __forceinline__ int setup_segments(const GridPlan& plan, const int32_t* __restrict__ cell_start, const Unit& unit, int group, SegmentTable& table) {
    int t = threadIdx.x;
    int length = 0;
    if (t < SEG_MAX) {
        int global_t = group * SEG_MAX + t;
        int start = 0;
        int q0 = 0, q1 = 0, q2 = 0;
        int self_ok = 0;
        if (global_t < unit.n_stencil) {
            int w0 = unit.cells + 2 * plan.n_search[0];
            int w1 = 2 * plan.n_search[1] + 1;
            int nb[3] = {
                unit.c0 + (global_t % w0) - plan.n_search[0],
                unit.c1 + ((global_t / w0) % w1) - plan.n_search[1],
                unit.c2 + (global_t / (w0 * w1)) - plan.n_search[2],
            };
            int q[3] = {0, 0, 0};
            bool valid = true;
#pragma unroll
            for (int k = 0; k < 3; k++) {
                if (plan.periodic[k] && k != plan.window_axis) {
                    q[k] = floor_div(nb[k], plan.n_cells[k]);
                    nb[k] -= q[k] * plan.n_cells[k];
                } else if (nb[k] < 0 || nb[k] >= plan.n_cells[k]) {
                    valid = false;
                }
            }
            if (valid) {
                int linear = (nb[2] * plan.n_cells[1] + nb[1]) * plan.n_cells[0] + nb[0];
                start = cell_start[linear];
                length = cell_start[linear + 1] - start;
                q0 = q[0];
                q1 = q[1];
                q2 = q[2];
                // only consulted for a point meeting itself, i.e. in an image
                // of its own cell: the un-shifted copy is the point itself
                bool nonzero = (q0 | q1 | q2) != 0;
                self_ok = nonzero && (plan.full || half_rule(q0, q1, q2));
            }
        }
        table.start[t] = start;
        table.image[t] = pack_segment_image(q0, q1, q2, self_ok);
    }
    int prefix = block_exclusive_scan<SEG_MAX / 32>(length, table.scan_tmp);
    if (t < SEG_MAX) {
        table.slot0[t] = prefix;
    }
    int total = table.scan_tmp[CTA_WARPS];
    if (t == 0) {
        table.slot0[SEG_MAX] = total;
    }
    __syncthreads();
    return total;
}

/// Segment that holds `slot`: last t with slot0[t] <= slot, among the first
/// 2^STEPS segments (entries past the stencil hold the total, so any power of
/// two that covers the stencil will do).
template <int STEPS = 7>
__device__ __forceinline__ int find_segment(const SegmentTable& table, int slot) {
    static_assert((1 << STEPS) <= SEG_MAX, "the table has SEG_MAX entries");
    int lo = 0;
    int hi = 1 << STEPS; // slot0[hi] > slot always holds for slot < total
#pragma unroll
    for (int step = 0; step < STEPS; step++) {
        int mid = (lo + hi) >> 1;
        if (table.slot0[mid] <= slot) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    return lo;
}

/// The reference's pair vector and squared distance, operation for operation:
/// v = (r_j - r_i) + ((S0*H0 + S1*H1) + S2*H2), d2 = (vx*vx + vy*vy) + vz*vz
/// (vesin/src/cpu_cell_list.cpp:135-136, types.hpp:232-243,
/// math.hpp:14-16,111-117). Intrinsics keep the compiler from fusing
/// multiplies and adds, which x86-64 builds of the reference never do.
__device__ __forceinline__ double exact_pair(
    const GridPlan& plan, double rix, double riy, double riz, double rjx, double rjy, double rjz, int s0, int s1, int s2,
    double& vx, double& vy, double& vz
) {
    double f0 = static_cast<double>(s0);
    double f1 = static_cast<double>(s1);
    double f2 = static_cast<double>(s2);
    double shx = __dadd_rn(__dadd_rn(__dmul_rn(f0, plan.H[0][0]), __dmul_rn(f1, plan.H[1][0])), __dmul_rn(f2, plan.H[2][0]));
    double shy = __dadd_rn(__dadd_rn(__dmul_rn(f0, plan.H[0][1]), __dmul_rn(f1, plan.H[1][1])), __dmul_rn(f2, plan.H[2][1]));
    double shz = __dadd_rn(__dadd_rn(__dmul_rn(f0, plan.H[0][2]), __dmul_rn(f1, plan.H[1][2])), __dmul_rn(f2, plan.H[2][2]));
    vx = __dadd_rn(__dsub_rn(rjx, rix), shx);
    vy = __dadd_rn(__dsub_rn(rjy, riy), shy);
    vz = __dadd_rn(__dsub_rn(rjz, riz), shz);
    return __dadd_rn(__dadd_rn(__dmul_rn(vx, vx), __dmul_rn(vy, vy)), __dmul_rn(vz, vz));
}

// ---------------------------------------------------------------------------
// fused pass (unsorted lists): decide and emit in one traversal
//
// Unsorted lists may come in any order, so a block of pairs does not need a
// position computed by a scan: it claims its output range with one atomicAdd
// on a global cursor once it knows how many pairs it holds. That removes the
// hit masks in global memory, the scan and the second traversal.
//
// Half-shell stencil: a unit only looks at the cells "above" its own (rows
// with oz > 0, or oz == 0 and oy > 0, and in its own row the cells at or after
// each home cell), so every unordered pair of images is evaluated once. A
// full list writes (i, j, S, d, v) and (j, i, -S, d, -v); a half list writes
// whichever of the two the reference keeps (i < j, or its rule on S when
// i == j; vesin/src/cpu_cell_list.cpp:101-133). -v is bit-identical to what
// the reference computes for the reversed pair: IEEE subtraction, product and
// sum are odd functions under round-to-nearest.
//
// When the claimed range does not fit the output arrays the block skips its
// stores but the cursor keeps counting: the host then grows the arrays to the
// exact total and runs the pass again.
// ---------------------------------------------------------------------------

// Optional instrumentation (-DVESIN_B200_PHASE_CLOCKS): thread 0 of every CTA of
// the fused pass adds the clock cycles it spends in each phase to a global
// table, read with vesin_b200_debug_phase_clocks(). Off in normal builds.
#ifdef VESIN_B200_PHASE_CLOCKS
__device__ unsigned long long g_phase_clocks[16];
#define PHASE_CLOCK_START() long long phase_last_ = clock64()
#define PHASE_MARK(k)                                                                          \
    do {                                                                                       \
        if (threadIdx.x == 0) {                                                                \
            const long long phase_now_ = clock64();                                            \
            atomicAdd(&g_phase_clocks[k], static_cast<unsigned long long>(phase_now_ - phase_last_)); \
            phase_last_ = phase_now_;                                                          \
        }                                                                                      \
    } while (0)
#else
#define PHASE_CLOCK_START()
#define PHASE_MARK(k)
#endif

constexpr int FUSED_BATCH = 512;
constexpr int DEFAULT_UNIT_RUN = 2; // neighbouring units handled back to back by one CTA (measured: 2 beats 1, 3, 4 and 8)
constexpr int MAX_UNIT_SPLITS = 32; // CTAs that share the candidate batches of one unit (launches of few units)
constexpr int FUSED_WORDS = FUSED_BATCH / 32;
constexpr int FUSED_LIST = 2048;
constexpr int FUSED_TASKS = (TILE_POINTS * FUSED_WORDS + CTA_THREADS - 1) / CTA_THREADS;

/// Shared memory of a CTA of THREADS_ threads that stages BATCH_ candidates at a time and
/// lists up to LIST_ hits per round.
template <int THREADS_, int BATCH_, int LIST_>
struct FusedSharedT {
    static constexpr int THREADS = THREADS_;
    static constexpr int WARPS = THREADS_ / 32;
    static constexpr int BATCH = BATCH_;
    static constexpr int WORDS = BATCH_ / 32;
    static constexpr int LIST = LIST_;
    /// (home point, word) tasks per thread when the hits of a tile are counted
    static constexpr int TASKS = (TILE_POINTS * WORDS + THREADS_ - 1) / THREADS_;
    static_assert(BATCH_ % 32 == 0 && (WORDS & (WORDS - 1)) == 0, "whole words, a power of two of them");
    static_assert(TILE_POINTS * BATCH_ < 65536, "hit counts of a tile are kept in 16 bits");
    static_assert(BATCH_ <= 512 && TILE_POINTS <= 32, "a list entry packs (lane, slot) into 14 bits");

    SegmentTable table;
    // fp32 coordinates of the candidates relative to the unit centre and their squared norm,
    // one array per component so that two candidates fill one packed fp32x2 operand
    alignas(16) float near_x[BATCH]; // read as 16-byte vectors
    alignas(16) float near_y[BATCH];
    alignas(16) float near_z[BATCH];
    alignas(16) float near_n[BATCH];
    double x[BATCH];       // original positions of the candidates
    double y[BATCH];
    double z[BATCH];
    int4 sj[BATCH];        // x, y, z: q - wrap shift of the candidate; w: its index
    double home_pos[3][TILE_POINTS];
    int4 home_sj[TILE_POINTS];   // x, y, z: wrap shift of the home point; w: its index
    unsigned mask[WORDS * TILE_POINTS]; // [word][lane]
    unsigned short list[LIST];          // (home lane << 9) | slot in batch
    unsigned short prefix[THREADS];       // hits of the tasks of the threads before this one in its warp
    alignas(16) double transpose[WARPS][192];         // per warp: 64 shifts, then 64 vectors, on their way to coalesced stores
    unsigned owned_word[WORDS]; // slab decomposition: which slots of a word hold owned points
    unsigned long long claim;
    double centre[3]; // centre of the unit: origin of the fp32 local frame
    int stencil_cached;          // are the packed offsets below usable?
    int stencil_offset[SEG_MAX]; // first SEG_MAX entries of the stencil of a full-length unit, 10 bits per direction
    int next_run[2];  // run of units this CTA takes next (two slots: one is read while the other is written)
    int slab_mode;    // slab decomposition: bit 0 = the unit's points are owned, bit 1 = so are all candidates of the group
};
/// The row kernels of sorted lists: 256 threads, 512 candidates per batch.
using FusedShared = FusedSharedT<CTA_THREADS, FUSED_BATCH, FUSED_LIST>;

/// Shape of the CTAs of the pair kernel of unsorted lists.
template <int THREADS_, int BATCH_, int LIST_, int CTAS_PER_SM_>
struct PairShape {
    using Shared = FusedSharedT<THREADS_, BATCH_, LIST_>;
    static constexpr int THREADS = THREADS_;
    static constexpr int WARPS = THREADS_ / 32;
    static constexpr int BATCH = BATCH_;
    static constexpr int WORDS = BATCH_ / 32;
    static constexpr int LIST = LIST_;
    static constexpr int TASKS = Shared::TASKS;
    static constexpr int CTAS_PER_SM = CTAS_PER_SM_;
    static_assert(THREADS_ >= SEG_MAX, "one thread per stencil segment of a group");
    // 228 KB of shared memory per SM, 1 KB of it reserved per resident CTA
    static_assert((sizeof(Shared) + 1024) * CTAS_PER_SM_ <= 228 * 1024, "CTAS_PER_SM CTAs fit on an SM");
    static_assert(
        offsetof(Shared, near_x) % 16 == 0 && offsetof(Shared, near_y) % 16 == 0 && offsetof(Shared, near_z) % 16 == 0 &&
            offsetof(Shared, near_n) % 16 == 0 && offsetof(Shared, transpose) % 16 == 0 && offsetof(Shared, sj) % 16 == 0 &&
            offsetof(Shared, home_sj) % 16 == 0,
        "members read or written as 16-byte vectors"
    );
};
/// Ordinary units: CTAs of 4 warps with 256 candidates per batch, 8 of them per SM. A barrier
/// holds up 4 warps instead of 8 and twice as many CTAs are there to issue meanwhile: sparse
/// systems (a unit of 30 points with 400 hits) gain 17 %, dense ones 4 %.
using SmallCta = PairShape<128, 256, 1024, 8>;
/// Units next to the halo of a slab (they sort their hits into owned and halo candidates and go
/// over every batch twice): CTAs of 8 warps with 512 candidates per batch, 4 per SM.
using LargeCta = PairShape<CTA_THREADS, FUSED_BATCH, FUSED_LIST, 4>;
static_assert(
    offsetof(FusedShared, near_x) % 16 == 0 && offsetof(FusedShared, near_y) % 16 == 0 && offsetof(FusedShared, near_z) % 16 == 0 &&
        offsetof(FusedShared, near_n) % 16 == 0 && offsetof(FusedShared, transpose) % 16 == 0 && offsetof(FusedShared, sj) % 16 == 0 &&
        offsetof(FusedShared, home_sj) % 16 == 0,
    "members read or written as 16-byte vectors"
);

/// Offset (in cells, relative to the first cell of the unit) of entry `index`
/// of the half-shell stencil of a unit of `cells` cells.
__device__ __forceinline__ void half_stencil_offset(const GridPlan& plan, int cells, int index, int& ox, int& oy, int& oz) {
    const int own_row = cells + plan.n_search[0];
    if (index < own_row) {
        ox = index;
        oy = 0;
        oz = 0;
        return;
    }
    const int row_width = cells + 2 * plan.n_search[0];
    const int rows_y = 2 * plan.n_search[1] + 1;
    const int rest = index - own_row;
    const int row = rest / row_width;
    ox = rest % row_width - plan.n_search[0];
    if (row < plan.n_search[1]) {
        oy = row + 1;
        oz = 0;
    } else {
        const int upper = row - plan.n_search[1];
        oz = 1 + upper / rows_y;
        oy = upper % rows_y - plan.n_search[1];
    }
}

/// Segments of the half-shell stencil of a unit. Order: the unit's own row
/// first (its own cells, then the n_search[0] cells after them), then the rows
/// above. Returns the slots of the group and how many of them belong to the
/// unit's own row; ends with a __syncthreads().
template <class Shared>
__device__ __forceinline__ int setup_half_segments(
    const GridPlan& plan, const int32_t* __restrict__ cell_start, const Unit& unit, int group, Shared& sh, int& home_row_slots
) {
    SegmentTable& table = sh.table;
    const int t = threadIdx.x;
    const int own_row = unit.cells + plan.n_search[0];
    int length = 0;
    if (t < SEG_MAX) {
        const int global_t = group * SEG_MAX + t;
        int start = 0;
        int q0 = 0, q1 = 0, q2 = 0;
        int owned = 1;
        if (global_t < unit.n_stencil) {
            int ox, oy, oz;
            if (group == 0 && unit.cells == plan.pencil && sh.stencil_cached) {
                // the usual unit: offsets decoded once per CTA
                const int packed = sh.stencil_offset[t];
                ox = (packed & 1023) - 512;
                oy = ((packed >> 10) & 1023) - 512;
                oz = (packed >> 20) - 512;
            } else {
                half_stencil_offset(plan, unit.cells, global_t, ox, oy, oz);
            }
            int nb[3] = {unit.c0 + ox, unit.c1 + oy, unit.c2 + oz};
            int q[3] = {0, 0, 0};
            bool valid = true;
            if (plan.window_axis >= 0) {
                // the offset counts layers in space
                const int k = plan.window_axis;
                const int offset = (k == 0) ? ox : ((k == 1) ? oy : oz);
                const int home = (k == 0) ? unit.c0 : ((k == 1) ? unit.c1 : unit.c2);
                nb[k] = window_space_layer(home, plan.n_cells[k]) + offset;
            }
#pragma unroll
            for (int k = 0; k < 3; k++) {
                const bool outside = nb[k] < 0 || nb[k] >= plan.n_cells[k];
                if (plan.periodic[k] && k != plan.window_axis) {
                    if (outside) {
                        q[k] = floor_div(nb[k], plan.n_cells[k]);
                        nb[k] -= q[k] * plan.n_cells[k];
                    }
                } else if (outside) {
                    valid = false;
                }
            }
            if (valid) {
                if (plan.window_axis >= 0) {
                    const int k = plan.window_axis;
                    owned = (nb[k] >= 1 && nb[k] <= plan.n_cells[k] - 2) ? 1 : 0;
                    nb[k] = window_storage_layer(nb[k], plan.n_cells[k]);
                }
                const int linear = (nb[2] * plan.n_cells[1] + nb[1]) * plan.n_cells[0] + nb[0];
                start = cell_start[linear];
                length = cell_start[linear + 1] - start;
                q0 = q[0];
                q1 = q[1];
                q2 = q[2];
            }
        }
        table.start[t] = start;
        table.image[t] = pack_segment_image(q0, q1, q2, owned); // (flag: does the segment hold owned points?)
    }
    const int prefix = block_exclusive_scan<SEG_MAX / 32>(length, table.scan_tmp);
    if (t < SEG_MAX) {
        table.slot0[t] = prefix;
    }
    const int total = table.scan_tmp[CTA_WARPS]; // where block_exclusive_scan leaves the total
    if (t == 0) {
        table.slot0[SEG_MAX] = total;
    }
    __syncthreads();
    // slots of this group that belong to the unit's own row
    home_row_slots = (group == 0) ? table.slot0[min(own_row, SEG_MAX)] : 0;
    return total;
}

/// Decisions of one lane's home point on BITS consecutive candidates of word `w`
/// of the staged batch, starting at bit `first_bit`: fp32 screen of every
/// candidate, the exact fp64 predicate for those too close to the cutoff for
/// fp32. Returns one bit per candidate that is a pair.
template <int BITS, class Shared>
__device__ __forceinline__ unsigned decide_piece(
    const Shared& sh, const GridPlan& plan, int w, int first_bit, int batch0, int home_row_slots, int il, unsigned long long ax2,
    unsigned long long ay2, unsigned long long az2, unsigned long long an2, float cutoff2_lo, float cutoff2_hi, double rix, double riy,
    double riz, int si0, int si1, int si2
) {
    constexpr unsigned ALL = (BITS == 32) ? 0xffffffffu : ((1u << (BITS & 31)) - 1u);
    unsigned inside = 0; // surely inside the cutoff
    unsigned near = 0;   // inside, or too close to the cutoff for fp32
    // four candidates per (broadcast) load, two per packed instruction; every component goes
    // through the same roundings as the scalar expression fma(cx, ax, fma(cy, ay, fma(cz, az, cn + an)))
    const int first_slot = w * 32 + first_bit;
    const ulonglong2* cx = reinterpret_cast<const ulonglong2*>(sh.near_x + first_slot);
    const ulonglong2* cy = reinterpret_cast<const ulonglong2*>(sh.near_y + first_slot);
    const ulonglong2* cz = reinterpret_cast<const ulonglong2*>(sh.near_z + first_slot);
    const ulonglong2* cn = reinterpret_cast<const ulonglong2*>(sh.near_n + first_slot);
#pragma unroll
    for (int k = 0; k < BITS / 4; k++) {
        const ulonglong2 x4 = cx[k];
        const ulonglong2 y4 = cy[k];
        const ulonglong2 z4 = cz[k];
        const ulonglong2 n4 = cn[k];
        float d2[4];
        unpack_f32x2(fma_f32x2(x4.x, ax2, fma_f32x2(y4.x, ay2, fma_f32x2(z4.x, az2, add_f32x2(n4.x, an2)))), d2[0], d2[1]);
        unpack_f32x2(fma_f32x2(x4.y, ax2, fma_f32x2(y4.y, ay2, fma_f32x2(z4.y, az2, add_f32x2(n4.y, an2)))), d2[2], d2[3]);
#pragma unroll
        for (int c = 0; c < 4; c++) {
            if (d2[c] < cutoff2_lo) {
                inside |= 1u << (4 * k + c);
            }
            if (d2[c] <= cutoff2_hi) {
                near |= 1u << (4 * k + c);
            }
        }
    }
    // half shell inside the unit's own row: only slots after the point's own
    unsigned keep = ALL;
    const int piece_slot = batch0 + first_slot;
    if (piece_slot < home_row_slots) {
        const int own = il - piece_slot; // bit of the point itself in this piece
        const unsigned after = (own < 0) ? ALL : ((own >= BITS - 1) ? 0u : ((ALL << (own + 1)) & ALL));
        const int row_bits = home_row_slots - piece_slot; // bits of this piece inside the row
        const unsigned in_row = (row_bits >= BITS) ? ALL : ((1u << row_bits) - 1u);
        keep = (after | ~in_row) & ALL;
    }
    inside &= keep;
    unsigned band = near & keep & ~inside;
    while (band != 0) {
        // the exact fp64 predicate of the reference decides
        const int b = __ffs(band) - 1;
        band &= band - 1;
        const int s = first_slot + b;
        double vx, vy, vz;
        const int4 cand = sh.sj[s];
        const double d2_exact = exact_pair(plan, rix, riy, riz, sh.x[s], sh.y[s], sh.z[s], cand.x + si0, cand.y + si1, cand.z + si2, vx, vy, vz);
        if (d2_exact < plan.cutoff2) {
            inside |= 1u << b;
        }
    }
    return inside;
}

/// Units a launch of the fused pass covers: [begin0, end0) and [begin1, end1).
struct UnitRanges {
    int begin0, end0, begin1, end1;
    /// Launches with far fewer units than CTAs (one small box whose stencil holds many
    /// images): every unit is handed to `splits` CTAs, which share out its candidate batches.
    int splits = 1;
};

template <bool FULL, bool SLAB, class Shape>
__global__ void __launch_bounds__(Shape::THREADS, Shape::CTAS_PER_SM) pairs_kernel(
    const GridPlan plan, const int32_t* __restrict__ cell_start, SortedPoints sorted, PairOutput out, unsigned long long capacity,
    DeviceHeader* header, const int UNIT_RUN, const UnitRanges ranges, unsigned long long* run_cursor, const int follows_pair_kernel
) {
    extern __shared__ __align__(16) unsigned char fused_smem[];
    using Shared = typename Shape::Shared;
    Shared& sh = *reinterpret_cast<Shared*>(fused_smem);

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const float cutoff2_lo = plan.cutoff2_lo;
    const float cutoff2_hi = plan.cutoff2_hi;

    // A slab build launches two pair kernels back to back: the second one (the units next to
    // the halo) needs nothing the first one writes, only what the kernels before both wrote.
    // The first one lets its follower be scheduled once every one of its own blocks has seen
    // those kernels complete (below); the follower then does not wait for it, and its blocks
    // fill the SMs that the first kernel's last runs leave idle.
    if (!follows_pair_kernel) {
        wait_for_previous_kernel();
        let_next_kernel_start();
    }
    if (header->status & STATUS_ABORT_MASK) {
        return; // the plan was refused: the host will redo the build
    }
    PHASE_CLOCK_START();
    if (threadIdx.x == 0) {
        // 10 bits per direction hold the offsets unless the stencil reaches very far
        sh.stencil_cached = (plan.pencil + plan.n_search[0] < 500 && plan.n_search[1] < 500 && plan.n_search[2] < 500) ? 1 : 0;
    }
    if (threadIdx.x < SEG_MAX) {
        // entries beyond the stencil are never read
        int ox, oy, oz;
        half_stencil_offset(plan, plan.pencil, threadIdx.x, ox, oy, oz);
        sh.stencil_offset[threadIdx.x] = ((ox + 512) & 1023) | (((oy + 512) & 1023) << 10) | (((oz + 512) & 1023) << 20);
    }
    __syncthreads();

    // Consecutive units share two thirds of their stencil: a CTA takes runs of
    // UNIT_RUN neighbouring units so that most of its loads hit in L1.
    // Runs are handed out dynamically (the first one is the block index): the run after
    // the current one is fetched while the current one is processed.
    // (the launch covers one or two ranges of units; a run lies inside one range)
    // (with splits > 1 a run is one unit, taken `splits` times: once per share of its batches)
    const int splits = ranges.splits;
    const int n_runs0 = (ranges.end0 - ranges.begin0 + UNIT_RUN - 1) / UNIT_RUN;
    const int n_runs = (n_runs0 + (ranges.end1 - ranges.begin1 + UNIT_RUN - 1) / UNIT_RUN) * splits;
    int claimed = blockIdx.x;
    int run_parity = 0;
    while (claimed < n_runs) {
    if (threadIdx.x == 0) {
        sh.next_run[run_parity] = static_cast<int>(gridDim.x + atomicAdd(run_cursor, 1ull));
    }
    const int run = (splits > 1) ? claimed / splits : claimed;
    const int share = (splits > 1) ? claimed - run * splits : 0;
    int batch_counter = 0;
    const int run_first = (run < n_runs0) ? ranges.begin0 + run * UNIT_RUN : ranges.begin1 + (run - n_runs0) * UNIT_RUN;
    const int run_end = min((run < n_runs0) ? ranges.end0 : ranges.end1, run_first + UNIT_RUN);
    Unit unit = unit_of(plan, cell_start, run_first);
    for (int u = run_first; u < run_end; u++) {
        if (u != run_first) {
            next_unit(plan, cell_start, unit);
        }
        if (unit.n_home == 0) {
            continue;
        }
        {
            const int own_row = unit.cells + plan.n_search[0];
            const int row_width = unit.cells + 2 * plan.n_search[0];
            const int rows_above = plan.n_search[1] + plan.n_search[2] * (2 * plan.n_search[1] + 1);
            unit.n_stencil = own_row + row_width * rows_above;
        }
        const int n_groups = (unit.n_stencil + SEG_MAX - 1) / SEG_MAX;
        const int n_tiles = (unit.n_home + TILE_POINTS - 1) / TILE_POINTS;

        // Slab decomposition: a unit lies in one layer along the cut direction.
        // Full lists: this rank writes (i, j) for its own i. A unit of owned
        // points writes the forward pair of every hit and the reversed pair of
        // hits whose candidate is owned too; a unit of the lower halo layer
        // only writes reversed pairs (towards owned candidates above it); the
        // upper halo layer sees nothing above it. Half lists: every unordered
        // pair is evaluated on exactly one rank with an owned home point, and
        // that rank writes it.
        if (SLAB) {
            const int stored = (plan.window_axis == 0) ? unit.c0 : ((plan.window_axis == 1) ? unit.c1 : unit.c2);
            const int layer = window_space_layer(stored, plan.n_cells[plan.window_axis]);
            const int last = plan.n_cells[plan.window_axis] - 1;
            if (layer == last) {
                continue;
            }
            if (!FULL && layer < 1) {
                continue;
            }
            if (threadIdx.x == 0) {
                sh.slab_mode = (layer >= 1) ? 1 : 0; // read after the barriers of the segment setup
            }
        }

        // centre of the pencil: origin of the fp32 local frame (shared memory: visible after
        // the barriers of the segment setup, and not held in registers across the unit)
        if (threadIdx.x < 3) {
            const int c = threadIdx.x;
            // (along the cut direction of a slab the geometry follows the layer in space)
            const int g0 = (plan.window_axis == 0) ? window_space_layer(unit.c0, plan.n_cells[0]) : unit.c0;
            const int g1 = (plan.window_axis == 1) ? window_space_layer(unit.c1, plan.n_cells[1]) : unit.c1;
            const int g2 = (plan.window_axis == 2) ? window_space_layer(unit.c2, plan.n_cells[2]) : unit.c2;
            sh.centre[c] = plan.origin[c] + (g0 + 0.5 * unit.cells) * plan.cell_vec[0][c] + (g1 + 0.5) * plan.cell_vec[1][c] +
                           (g2 + 0.5) * plan.cell_vec[2][c];
        }

        PHASE_MARK(0); // unit setup
        for (int g = 0; g < n_groups; g++) {
            int home_row_slots;
            const int group_total = setup_half_segments(plan, cell_start, unit, g, sh, home_row_slots);
            PHASE_MARK(1); // segments
            if (SLAB) {
                int segment_ok = 1;
                if (threadIdx.x < SEG_MAX) {
                    const int length = sh.table.slot0[threadIdx.x + 1] - sh.table.slot0[threadIdx.x];
                    segment_ok = (length == 0) || segment_flag(sh.table.image[threadIdx.x]);
                }
                const int all_candidates_owned = __syncthreads_and(segment_ok);
                if (threadIdx.x == 0) {
                    sh.slab_mode = (sh.slab_mode & 1) | ((all_candidates_owned && (sh.slab_mode & 1)) ? 2 : 0);
                }
                // visible after the barrier that ends the staging of the first batch
            }
            for (int batch0 = 0; batch0 < group_total; batch0 += Shape::BATCH) {
                const int batch_slots = min(Shape::BATCH, group_total - batch0);
                const int batch_words = (batch_slots + 31) >> 5;
                if (splits > 1) {
                    // the same decision in every thread of the CTA
                    const bool mine = (batch_counter % splits) == share;
                    batch_counter++;
                    if (!mine) {
                        continue;
                    }
                }

                if (SLAB && FULL) {
                    // which slots of the batch hold owned points: every owned segment marks its range
                    if (threadIdx.x < Shape::WORDS) {
                        sh.owned_word[threadIdx.x] = 0;
                    }
                    __syncthreads();
                    if (threadIdx.x < SEG_MAX && segment_flag(sh.table.image[threadIdx.x])) {
                        const int a = max(sh.table.slot0[threadIdx.x], batch0) - batch0;
                        const int b = min(sh.table.slot0[threadIdx.x + 1], batch0 + batch_slots) - batch0;
                        for (int w = a >> 5; a < b && w <= ((b - 1) >> 5); w++) {
                            const int lo = max(a, 32 * w) - 32 * w;
                            const int hi = min(b, 32 * w + 32) - 32 * w;
                            const unsigned mask = (hi - lo == 32) ? 0xffffffffu : (((1u << (hi - lo)) - 1u) << lo);
                            atomicOr(&sh.owned_word[w], mask);
                        }
                    }
                    // read after the barriers of the first tile
                }
                // ---- stage the candidates: one slot per thread (the segment of a slot is
                //      found by bisection), so all loads of a batch are in flight at once ----
                for (int s = threadIdx.x; s < batch_slots; s += Shape::THREADS) {
                    const int slot = batch0 + s;
                    const int t = (unit.n_stencil <= 32) ? find_segment<5>(sh.table, slot) : find_segment<7>(sh.table, slot);
                    const size_t p = static_cast<size_t>(sh.table.start[t]) + (slot - sh.table.slot0[t]);
                    const double px = sorted.pos[3 * p + 0];
                    const double py = sorted.pos[3 * p + 1];
                    const double pz = sorted.pos[3 * p + 2];
                    int r0, r1, r2;
                    unpack_segment_image(sh.table.image[t], r0, r1, r2);
                    r0 -= sorted.shift[3 * p + 0];
                    r1 -= sorted.shift[3 * p + 1];
                    r2 -= sorted.shift[3 * p + 2];
                    sh.x[s] = px;
                    sh.y[s] = py;
                    sh.z[s] = pz;
                    sh.sj[s] = make_int4(r0, r1, r2, sorted.index[p]);
                    // image of the candidate seen from this unit (most candidates of a large box have none)
                    double ix = px;
                    double iy = py;
                    double iz = pz;
                    if ((r0 | r1 | r2) != 0) {
                        ix += r0 * plan.H[0][0] + r1 * plan.H[1][0] + r2 * plan.H[2][0];
                        iy += r0 * plan.H[0][1] + r1 * plan.H[1][1] + r2 * plan.H[2][1];
                        iz += r0 * plan.H[0][2] + r1 * plan.H[1][2] + r2 * plan.H[2][2];
                    }
                    const float fx = static_cast<float>(ix - sh.centre[0]);
                    const float fy = static_cast<float>(iy - sh.centre[1]);
                    const float fz = static_cast<float>(iz - sh.centre[2]);
                    sh.near_x[s] = fx;
                    sh.near_y[s] = fy;
                    sh.near_z[s] = fz;
                    sh.near_n[s] = fx * fx + fy * fy + fz * fz;
                }
                for (int s = batch_slots + threadIdx.x; s < batch_words * 32; s += Shape::THREADS) {
                    sh.near_x[s] = 0.0f;
                    sh.near_y[s] = 0.0f;
                    sh.near_z[s] = 0.0f;
                    sh.near_n[s] = __int_as_float(0x7f800000); // never a hit
                }

                for (int tile = 0; tile < n_tiles; tile++) {
                    PHASE_MARK(2); // staging (first tile) or the end of the previous tile
                    __syncthreads(); // staging done; previous tile done with mask / list / home
                    PHASE_MARK(3); // wait
                    // A tile with few home points (the overflow of a unit that holds a few more than
                    // 32) gives every home point four lanes: each takes a quarter of every word of
                    // candidates, and a word costs a quarter of what it costs a full tile.
                    const int n_in_tile = min(TILE_POINTS, unit.n_home - tile * TILE_POINTS);
                    const bool narrow = n_in_tile <= TILE_POINTS / 4;
                    const int home_lane = narrow ? (lane >> 2) : lane;
                    const int il = tile * TILE_POINTS + home_lane;
                    const bool valid = home_lane < n_in_tile;
                    // The home points are the first candidates of a unit (its own cells open the
                    // stencil): while they sit in the staged batch they are read from there.
                    const bool home_staged = (g == 0) && (batch0 == 0) && (tile * TILE_POINTS + TILE_POINTS <= Shape::BATCH);
                    // Lanes without a point carry NaN: every comparison fails.
                    const float nan = __int_as_float(0x7fc00000);
                    double rix, riy, riz;
                    int si0, si1, si2, index_i;
                    float xi, yi, zi, an;
                    if (home_staged) {
                        const int slot = valid ? il : 0;
                        rix = sh.x[slot];
                        riy = sh.y[slot];
                        riz = sh.z[slot];
                        const int4 packed = sh.sj[slot]; // own cells have no image shift: q = 0
                        si0 = -packed.x;
                        si1 = -packed.y;
                        si2 = -packed.z;
                        index_i = packed.w;
                        xi = valid ? sh.near_x[slot] : nan;
                        yi = valid ? sh.near_y[slot] : nan;
                        zi = valid ? sh.near_z[slot] : nan;
                        an = sh.near_n[slot];
                    } else {
                        const size_t pi = static_cast<size_t>(unit.begin) + (valid ? il : 0);
                        rix = sorted.pos[3 * pi + 0];
                        riy = sorted.pos[3 * pi + 1];
                        riz = sorted.pos[3 * pi + 2];
                        si0 = sorted.shift[3 * pi + 0];
                        si1 = sorted.shift[3 * pi + 1];
                        si2 = sorted.shift[3 * pi + 2];
                        index_i = sorted.index[pi];
                        xi = valid ? static_cast<float>(rix - (si0 * plan.H[0][0] + si1 * plan.H[1][0] + si2 * plan.H[2][0]) - sh.centre[0]) : nan;
                        yi = valid ? static_cast<float>(riy - (si0 * plan.H[0][1] + si1 * plan.H[1][1] + si2 * plan.H[2][1]) - sh.centre[1]) : nan;
                        zi = valid ? static_cast<float>(riz - (si0 * plan.H[0][2] + si1 * plan.H[1][2] + si2 * plan.H[2][2]) - sh.centre[2]) : nan;
                        an = xi * xi + yi * yi + zi * zi;
                    }
                    if (warp == 0 && (!narrow || (lane & 3) == 0)) {
                        sh.home_pos[0][home_lane] = rix;
                        sh.home_pos[1][home_lane] = riy;
                        sh.home_pos[2][home_lane] = riz;
                        sh.home_sj[home_lane] = make_int4(si0, si1, si2, index_i);
                    }
                    // d2 = |c|^2 + (|i|^2 - 2 c.i): one add and three fused multiply-adds per candidate.
                    const float ax = -2.0f * xi;
                    const float ay = -2.0f * yi;
                    const float az = -2.0f * zi;
                    const unsigned long long ax2 = pack_f32x2(ax, ax);
                    const unsigned long long ay2 = pack_f32x2(ay, ay);
                    const unsigned long long az2 = pack_f32x2(az, az);
                    const unsigned long long an2 = pack_f32x2(an, an);

                    if (narrow) {
                        for (int w = warp; w < batch_words; w += Shape::WARPS) {
                            const int quarter = lane & 3;
                            unsigned word = decide_piece<8>(
                                            sh, plan, w, 8 * quarter, batch0, home_row_slots, il, ax2, ay2, az2, an2, cutoff2_lo, cutoff2_hi, rix, riy, riz,
                                            si0, si1, si2
                                        )
                                        << (8 * quarter);
                            // the four lanes of a home point put their quarters together
                            word |= __shfl_xor_sync(FULL_MASK, word, 1);
                            word |= __shfl_xor_sync(FULL_MASK, word, 2);
                            const unsigned of_home = __shfl_sync(FULL_MASK, word, (lane & 7) * 4);
                            sh.mask[w * TILE_POINTS + lane] = (lane < TILE_POINTS / 4) ? of_home : 0u;
                        }
                    } else if (batch_words <= Shape::WARPS) {
                        // a word of 32 candidates per warp
                        if (warp < batch_words) {
                            sh.mask[warp * TILE_POINTS + lane] = decide_piece<32>(
                                sh, plan, warp, 0, batch0, home_row_slots, il, ax2, ay2, az2, an2, cutoff2_lo, cutoff2_hi, rix, riy, riz, si0, si1, si2
                            );
                        }
                    } else {
                        // more words than warps: halves of words, so that no warp does two words while others do one
                        unsigned short* halves = reinterpret_cast<unsigned short*>(sh.mask);
                        for (int piece = warp; piece < 2 * batch_words; piece += Shape::WARPS) {
                            const int half = (piece >= batch_words) ? 1 : 0;
                            const int w = piece - half * batch_words;
                            halves[2 * (w * TILE_POINTS + lane) + half] = static_cast<unsigned short>(decide_piece<16>(
                                sh, plan, w, 16 * half, batch0, home_row_slots, il, ax2, ay2, az2, an2, cutoff2_lo, cutoff2_hi, rix, riy, riz, si0, si1,
                                si2
                            ));
                        }
                    }
                    PHASE_MARK(4); // home points + decisions
                    __syncthreads();
                    PHASE_MARK(5); // wait

                    // ---- compact the hit bits and write. Tasks = words in [word][lane]
                    // order. One pass writes both orientations (full) or the kept one
                    // (half). A unit of a slab-decomposed full list that touches halo
                    // points sorts its hits by the owner of the candidate: a unit of owned
                    // points writes both orientations of its hits with owned candidates,
                    // then the forward pairs of its hits with halo candidates; a unit of
                    // halo points only has the reversed pairs towards owned candidates ----
                    // (split: the unit or some of its candidates are halo points)
                    const bool split = SLAB && FULL && (sh.slab_mode & 2) == 0;
                    const bool home_owned = !split || (sh.slab_mode & 1) != 0;
                    const int n_passes = (split && home_owned) ? 2 : 1;
                    for (int pass = 0; pass < n_passes; pass++) {
                        const bool write_forward = home_owned;
                        const bool write_reverse = FULL && (!split || pass == 0);
                        const bool only_owned_candidates = split && pass == 0;
                        const bool only_halo_candidates = split && pass == 1;
                        if (pass != 0) {
                            __syncthreads(); // list, claim and scan scratch of the first pass are free again
                        }
                        const int n_tasks = TILE_POINTS * batch_words;
                        // word of hit bits of a task (= word index * 32 + home lane)
                        const auto task_word = [&](int task) -> unsigned {
                            unsigned word = (task < n_tasks) ? sh.mask[task] : 0u;
                            if (SLAB && only_owned_candidates) {
                                word &= sh.owned_word[(task >> 5) & (Shape::WORDS - 1)];
                            }
                            if (SLAB && only_halo_candidates) {
                                word &= ~sh.owned_word[(task >> 5) & (Shape::WORDS - 1)];
                            }
                            return word;
                        };
                        int my_hits = 0;
#pragma unroll
                        for (int k = 0; k < Shape::TASKS; k++) {
                            my_hits += __popc(task_word(threadIdx.x * Shape::TASKS + k));
                        }
                        // scan of the hit counts: inside the warp with shuffles, across warps by
                        // reading the eight warp totals after one barrier
                        int inclusive = my_hits;
#pragma unroll
                        for (int offset = 1; offset < 32; offset <<= 1) {
                            const int up = __shfl_up_sync(FULL_MASK, inclusive, offset);
                            if (lane >= offset) {
                                inclusive += up;
                            }
                        }
                        sh.prefix[threadIdx.x] = static_cast<unsigned short>(inclusive - my_hits);
                        if (lane == 31) {
                            sh.table.scan_tmp[warp] = inclusive;
                        }
                        __syncthreads();
                        int total_hits = 0;
#pragma unroll
                        for (int w = 0; w < Shape::WARPS; w++) {
                            total_hits += sh.table.scan_tmp[w];
                        }
                        if (total_hits == 0) {
                            continue;
                        }
                        const int per_hit = (write_forward ? 1 : 0) + (write_reverse ? 1 : 0);
                        // claim the output range of this block of pairs; the answer is only
                        // needed after the list below has been built
                        const unsigned long long wanted = static_cast<unsigned long long>(total_hits) * per_hit;
                        unsigned long long claimed = 0;
                        if (threadIdx.x == 0) {
                            claimed = atomicAdd(&header->pair_cursor, wanted);
                        }
                        if (capacity == 0) {
                            continue; // counting pass: the host sizes the arrays from the cursor
                        }
                        unsigned long long claim = 0;

                        for (int round0 = 0; round0 < total_hits; round0 += Shape::LIST) {
                            if (round0 != 0) {
                                __syncthreads(); // previous round consumed
                            }
                            const int in_round = min(Shape::LIST, total_hits - round0);
                            {
                                // List of the hits of this round, in task order. Every thread writes the
                                // same number of consecutive entries whatever the hits of its own tasks:
                                // it finds the task that holds its first entry in the scanned counts
                                // (first the warp, then the thread), skips the bits before it and walks
                                // on from there.
                                const int quota = (in_round + Shape::THREADS - 1) / Shape::THREADS;
                                int position = round0 + threadIdx.x * quota;
                                const int stop = min(position + quota, round0 + in_round);
                                if (position < stop) {
                                    int owner_warp = 0;
                                    int before = 0; // hits of the warps before the owner
                                    {
                                        int running = 0;
#pragma unroll
                                        for (int w = 0; w < Shape::WARPS - 1; w++) {
                                            running += sh.table.scan_tmp[w];
                                            if (running <= position) {
                                                owner_warp = w + 1;
                                                before = running;
                                            }
                                        }
                                    }
                                    const int target = position - before;
                                    const unsigned short* local = sh.prefix + owner_warp * 32;
                                    int lo = 0;
                                    int hi = 32;
#pragma unroll
                                    for (int step = 0; step < 5; step++) {
                                        const int mid = (lo + hi) >> 1;
                                        if (static_cast<int>(local[mid]) <= target) {
                                            lo = mid;
                                        } else {
                                            hi = mid;
                                        }
                                    }
                                    int skip = target - static_cast<int>(local[lo]);
                                    lo += owner_warp * 32;
                                    int task = lo * Shape::TASKS;
                                    unsigned word = task_word(task);
#pragma unroll
                                    for (int k = 1; k < Shape::TASKS; k++) {
                                        const int count = __popc(word);
                                        if (skip >= count) {
                                            skip -= count;
                                            task++;
                                            word = task_word(task);
                                        }
                                    }
                                    word &= 0xffffffffu << select_bit(word, skip);
                                    for (; position < stop; position++) {
                                        while (word == 0 && task + 1 < n_tasks) {
                                            task++;
                                            word = task_word(task);
                                        }
                                        const int bit = __ffs(word) - 1;
                                        word &= word - 1;
                                        sh.list[position - round0] =
                                            static_cast<unsigned short>(((task & 31) << 9) | ((task >> 5) << 5) | (bit & 31));
                                    }
                                }
                            }
                            if (round0 == 0 && threadIdx.x == 0) {
                                sh.claim = (claimed + wanted <= capacity) ? claimed : ~0ull;
                            }
                            __syncthreads();
                            PHASE_MARK(7); // list of hits
                            if (round0 == 0) {
                                claim = sh.claim;
                            }
                            if (claim == ~0ull) {
                                break; // counted, not written: the host will grow the arrays
                            }

                            // both orientations side by side when the claim and the arrays allow it
                            // (a claim on an odd element is moved on by one, see store_both; plain full
                            // lists only ever claim even blocks)
                            const bool interleave = FULL && write_forward && write_reverse && out.interleave_ok && (SLAB || (claim & 1ull) == 0);
                            const unsigned long long moved_on = SLAB ? (claim & 1ull) : 0ull;
                            for (int chunk0 = warp * 32; chunk0 < in_round; chunk0 += Shape::WARPS * 32) {
                                const int n_valid = min(32, in_round - chunk0);
                                double vx = 0, vy = 0, vz = 0, d = 0;
                                int h = 0, s = 0;
                                if (lane < n_valid) {
                                    const unsigned entry = sh.list[chunk0 + lane];
                                    h = entry >> 9;
                                    s = entry & 511;
                                }
                                const int4 cand = sh.sj[s];
                                const int4 home = sh.home_sj[h];
                                int s0 = cand.x + home.x;
                                int s1 = cand.y + home.y;
                                int s2 = cand.z + home.z;
                                double d2;
                                if (__any_sync(0xffffffffu, (s0 | s1 | s2) != 0)) {
                                    d2 = exact_pair(
                                        plan, sh.home_pos[0][h], sh.home_pos[1][h], sh.home_pos[2][h], sh.x[s], sh.y[s], sh.z[s], s0, s1, s2,
                                        vx, vy, vz
                                    );
                                } else {
                                    // no image shift in this chunk: the shift term is the signed zero the
                                    // reference's arithmetic gives for S = 0
                                    vx = __dadd_rn(__dsub_rn(sh.x[s], sh.home_pos[0][h]), plan.zero_shift[0]);
                                    vy = __dadd_rn(__dsub_rn(sh.y[s], sh.home_pos[1][h]), plan.zero_shift[1]);
                                    vz = __dadd_rn(__dsub_rn(sh.z[s], sh.home_pos[2][h]), plan.zero_shift[2]);
                                    d2 = __dadd_rn(__dadd_rn(__dmul_rn(vx, vx), __dmul_rn(vy, vy)), __dmul_rn(vz, vz));
                                }
                                d = __dsqrt_rn(d2);
                                unsigned long long index_i = static_cast<unsigned long long>(home.w);
                                unsigned long long index_j = static_cast<unsigned long long>(cand.w);
                                if (interleave) {
                                    int tail_lane = -1;
                                    if (SLAB && moved_on != 0 && round0 + chunk0 + n_valid == total_hits) {
                                        tail_lane = n_valid - 1; // the last hit of the block is in this chunk
                                    }
                                    store_both(
                                        sh.transpose[warp], out, lane, claim + moved_on + 2ull * (round0 + chunk0), n_valid, index_i, index_j, s0, s1, s2, d,
                                        vx, vy, vz, tail_lane, claim
                                    );
                                    continue;
                                }
                                const unsigned long long first = claim + round0 + chunk0;
                                if (FULL) {
                                    if (write_forward) {
                                        store_pairs(sh.transpose[warp], out, lane, first, n_valid, index_i, index_j, s0, s1, s2, d, vx, vy, vz);
                                    }
                                    if (write_reverse) {
                                        store_pairs(
                                            sh.transpose[warp], out, lane, first + (write_forward ? total_hits : 0), n_valid, index_j, index_i, -s0, -s1, -s2,
                                            d, -vx, -vy, -vz
                                        );
                                    }
                                } else {
                                    // the orientation the reference's half list keeps
                                    const bool forward = (index_i < index_j) || (index_i == index_j && half_rule(s0, s1, s2));
                                    if (!forward) {
                                        const unsigned long long swap = index_i;
                                        index_i = index_j;
                                        index_j = swap;
                                        s0 = -s0;
                                        s1 = -s1;
                                        s2 = -s2;
                                        vx = -vx;
                                        vy = -vy;
                                        vz = -vz;
                                    }
                                    store_pairs(sh.transpose[warp], out, lane, first, n_valid, index_i, index_j, s0, s1, s2, d, vx, vy, vz);
                                }
                            }
                            PHASE_MARK(8); // emission
                        }
                    }
                }
                __syncthreads();
                PHASE_MARK(9); // wait
            }
        }
    }
    __syncthreads(); // next_run is visible; nobody reads the other slot any more
    claimed = sh.next_run[run_parity];
    run_parity ^= 1;
    }
}

// ---------------------------------------------------------------------------
// sorted lists: one row per point, rows in index order
// Replaces find_neighbors_cell_list + sort_pairs (vesin/src/vesin_cuda.cpp:188-291,
// vesin/src/cuda/sort_pairs.cu:63-202: a bitonic network over all pairs in
// global memory) and GrowableNeighborList::sort (vesin/src/cpu_cell_list.cpp:634-730).
//
// A row can only be written by one CTA if that CTA sees every pair of the
// point, so the two passes walk the FULL stencil of a unit (every pair of a
// full list is decided twice, once from each end). Pass 1 decides with the
// machinery of the fused pass (packed fp32 screen, exact fp64 band) and leaves
// one hit word per (point, 32 candidates) in global memory plus the number of
// pairs of every point; a scan turns the counts into row starts; pass 2 walks
// the hit words, so both passes agree by construction, and writes every row
// in the order the candidates were staged.
// ---------------------------------------------------------------------------

struct RowShared {
    FusedShared staged;
    unsigned long long home_row[TILE_POINTS]; // where the row of a home point continues
    int row_offset[TILE_POINTS + 1];          // list position where the hits of each home point start
    int tile_hits[TILE_POINTS];               // pass 1: hits of the home points of the tile in the current batch
    unsigned long long mask_base;
};

/// Does the pair (home point, candidate) belong to the list, as far as indices
/// and shifts decide? Full lists: everything but the point itself. Half lists:
/// the rule of the reference (vesin/src/cpu_cell_list.cpp:101-133).
template <bool FULL>
__device__ __forceinline__ bool row_keeps(const int4& home, const int4& candidate) {
    const int s0 = candidate.x + home.x;
    const int s1 = candidate.y + home.y;
    const int s2 = candidate.z + home.z;
    if (candidate.w != home.w) {
        return FULL || candidate.w > home.w;
    }
    if ((s0 | s1 | s2) == 0) {
        return false; // the point itself
    }
    return FULL || half_rule(s0, s1, s2);
}

/// Words of hit bits one home point of the unit needs: every segment group
/// starts on a fresh word. Leaves the table of the LAST group in place.
__device__ __forceinline__ int row_words_of_unit(
    const GridPlan& plan, const int32_t* __restrict__ cell_start, const Unit& unit, int n_groups, SegmentTable& table, int& last_total
) {
    int words = 0;
    for (int g = 0; g < n_groups; g++) {
        last_total = setup_segments(plan, cell_start, unit, g, table);
        words += (last_total + 31) >> 5;
    }
    return words;
}

/// Stage `batch_slots` candidates starting at slot `batch0` of the current
/// segment group: original positions and (shift part, index) for the exact
/// arithmetic and the output, and, with NEAR, fp32 coordinates relative to the
/// unit centre for the screen.
template <bool NEAR>
__device__ __forceinline__ void stage_row_batch(
    FusedShared& sh, const GridPlan& plan, const SortedPoints& sorted, int n_stencil, int batch0, int batch_slots
) {
    for (int s = threadIdx.x; s < batch_slots; s += CTA_THREADS) {
        const int slot = batch0 + s;
        const int t = (n_stencil <= 32) ? find_segment<5>(sh.table, slot) : find_segment<7>(sh.table, slot);
        const size_t p = static_cast<size_t>(sh.table.start[t]) + (slot - sh.table.slot0[t]);
        const double px = sorted.pos[3 * p + 0];
        const double py = sorted.pos[3 * p + 1];
        const double pz = sorted.pos[3 * p + 2];
        int r0, r1, r2;
        unpack_segment_image(sh.table.image[t], r0, r1, r2);
        r0 -= sorted.shift[3 * p + 0];
        r1 -= sorted.shift[3 * p + 1];
        r2 -= sorted.shift[3 * p + 2];
        sh.x[s] = px;
        sh.y[s] = py;
        sh.z[s] = pz;
        sh.sj[s] = make_int4(r0, r1, r2, sorted.index[p]);
        if (NEAR) {
            double ix = px;
            double iy = py;
            double iz = pz;
            if ((r0 | r1 | r2) != 0) {
                ix += r0 * plan.H[0][0] + r1 * plan.H[1][0] + r2 * plan.H[2][0];
                iy += r0 * plan.H[0][1] + r1 * plan.H[1][1] + r2 * plan.H[2][1];
                iz += r0 * plan.H[0][2] + r1 * plan.H[1][2] + r2 * plan.H[2][2];
            }
            const float fx = static_cast<float>(ix - sh.centre[0]);
            const float fy = static_cast<float>(iy - sh.centre[1]);
            const float fz = static_cast<float>(iz - sh.centre[2]);
            sh.near_x[s] = fx;
            sh.near_y[s] = fy;
            sh.near_z[s] = fz;
            sh.near_n[s] = fx * fx + fy * fy + fz * fz;
        }
    }
    if (NEAR) {
        const int batch_words = (batch_slots + 31) >> 5;
        for (int s = batch_slots + threadIdx.x; s < batch_words * 32; s += CTA_THREADS) {
            sh.near_x[s] = 0.0f;
            sh.near_y[s] = 0.0f;
            sh.near_z[s] = 0.0f;
            sh.near_n[s] = __int_as_float(0x7f800000); // never a hit
        }
    }
}

template <bool FULL>
__global__ void __launch_bounds__(CTA_THREADS, 4) row_count_kernel(
    const GridPlan plan, const int32_t* __restrict__ cell_start, SortedPoints sorted, uint32_t* __restrict__ masks,
    unsigned long long mask_capacity, unsigned long long* __restrict__ unit_mask_base, uint32_t* __restrict__ unit_words,
    uint32_t* __restrict__ row_count, DeviceHeader* header
) {
    extern __shared__ __align__(16) unsigned char row_smem[];
    RowShared& rows = *reinterpret_cast<RowShared*>(row_smem);
    FusedShared& sh = rows.staged;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const float cutoff2_lo = plan.cutoff2_lo;
    const float cutoff2_hi = plan.cutoff2_hi;
    if (header->status & STATUS_ABORT_MASK) {
        return;
    }
    if (threadIdx.x < TILE_POINTS) {
        rows.tile_hits[threadIdx.x] = 0;
    }

    for (int u = blockIdx.x; u < plan.n_units; u += gridDim.x) {
        const Unit unit = unit_of(plan, cell_start, u);
        if (unit.n_home == 0) {
            continue;
        }
        const int n_groups = (unit.n_stencil + SEG_MAX - 1) / SEG_MAX;
        const int n_tiles = (unit.n_home + TILE_POINTS - 1) / TILE_POINTS;
        if (threadIdx.x < 3) {
            const int c = threadIdx.x;
            sh.centre[c] = plan.origin[c] + (unit.c0 + 0.5 * unit.cells) * plan.cell_vec[0][c] + (unit.c1 + 0.5) * plan.cell_vec[1][c] +
                           (unit.c2 + 0.5) * plan.cell_vec[2][c];
        }

        int group_total = 0;
        const int words = row_words_of_unit(plan, cell_start, unit, n_groups, sh.table, group_total);
        // claim the storage of the hit words: n_tiles blocks of `words` x 32 lanes
        if (threadIdx.x == 0) {
            const unsigned long long need = static_cast<unsigned long long>(n_tiles) * words * TILE_POINTS;
            unsigned long long base = atomicAdd(&header->mask_cursor, need);
            if (base + need > mask_capacity) {
                atomicOr(&header->status, STATUS_MASK_OVERFLOW);
                base = ~0ull;
            } else {
                unit_mask_base[u] = base;
                unit_words[u] = static_cast<uint32_t>(words);
            }
            rows.mask_base = base;
        }
        __syncthreads();
        const unsigned long long base = rows.mask_base;
        if (base == ~0ull) {
            __syncthreads();
            continue; // the host grows the storage and runs the pass again
        }

        // the unit's own cells open the entries own_entry ... of the stencil: the slot of a home
        // point among the candidates is the slot of its first cell plus its number in the unit
        const int own_entry = plan.n_search[0] + (unit.cells + 2 * plan.n_search[0]) * (plan.n_search[1] + (2 * plan.n_search[1] + 1) * plan.n_search[2]);
        const int own_group = own_entry / SEG_MAX;
        const bool own_straddles = (own_entry % SEG_MAX) + unit.cells > SEG_MAX;
        int word_base = 0;
        for (int g = 0; g < n_groups; g++) {
            if (n_groups > 1) {
                group_total = setup_segments(plan, cell_start, unit, g, sh.table);
            }
            const int own_slot0 = (g == own_group) ? sh.table.slot0[own_entry % SEG_MAX] : 0;
            for (int batch0 = 0; batch0 < group_total; batch0 += FUSED_BATCH) {
                const int batch_slots = min(FUSED_BATCH, group_total - batch0);
                const int batch_words = (batch_slots + 31) >> 5;
                stage_row_batch<true>(sh, plan, sorted, unit.n_stencil, batch0, batch_slots);

                for (int tile = 0; tile < n_tiles; tile++) {
                    __syncthreads(); // staging done; previous tile done with the hit words and the home points
                    const int il = tile * TILE_POINTS + lane;
                    const bool valid = il < unit.n_home;
                    const size_t pi = static_cast<size_t>(unit.begin) + (valid ? il : 0);
                    const double rix = sorted.pos[3 * pi + 0];
                    const double riy = sorted.pos[3 * pi + 1];
                    const double riz = sorted.pos[3 * pi + 2];
                    const int si0 = sorted.shift[3 * pi + 0];
                    const int si1 = sorted.shift[3 * pi + 1];
                    const int si2 = sorted.shift[3 * pi + 2];
                    // lanes without a point carry NaN: every comparison fails
                    const float nan = __int_as_float(0x7fc00000);
                    const float xi = valid ? static_cast<float>(rix - (si0 * plan.H[0][0] + si1 * plan.H[1][0] + si2 * plan.H[2][0]) - sh.centre[0]) : nan;
                    const float yi = valid ? static_cast<float>(riy - (si0 * plan.H[0][1] + si1 * plan.H[1][1] + si2 * plan.H[2][1]) - sh.centre[1]) : nan;
                    const float zi = valid ? static_cast<float>(riz - (si0 * plan.H[0][2] + si1 * plan.H[1][2] + si2 * plan.H[2][2]) - sh.centre[2]) : nan;
                    const float an = xi * xi + yi * yi + zi * zi;
                    if (warp == 0) {
                        sh.home_sj[lane] = make_int4(si0, si1, si2, sorted.index[pi]);
                    }
                    const float ax = -2.0f * xi;
                    const float ay = -2.0f * yi;
                    const float az = -2.0f * zi;
                    const unsigned long long ax2 = pack_f32x2(ax, ax);
                    const unsigned long long ay2 = pack_f32x2(ay, ay);
                    const unsigned long long az2 = pack_f32x2(az, az);
                    const unsigned long long an2 = pack_f32x2(an, an);
                    // (no half shell here: home_row_slots = 0 keeps every candidate)
                    if (batch_words <= CTA_WARPS) {
                        if (warp < batch_words) {
                            sh.mask[warp * TILE_POINTS + lane] =
                                decide_piece<32>(sh, plan, warp, 0, batch0, 0, il, ax2, ay2, az2, an2, cutoff2_lo, cutoff2_hi, rix, riy, riz, si0, si1, si2);
                        }
                    } else {
                        unsigned short* halves = reinterpret_cast<unsigned short*>(sh.mask);
                        for (int piece = warp; piece < 2 * batch_words; piece += CTA_WARPS) {
                            const int half = (piece >= batch_words) ? 1 : 0;
                            const int w = piece - half * batch_words;
                            halves[2 * (w * TILE_POINTS + lane) + half] = static_cast<unsigned short>(decide_piece<16>(
                                sh, plan, w, 16 * half, batch0, 0, il, ax2, ay2, az2, an2, cutoff2_lo, cutoff2_hi, rix, riy, riz, si0, si1, si2
                            ));
                        }
                    }
                    __syncthreads();
                    // ---- indices and shifts have their say on the hits; the words go to global
                    //      memory as [tile][word][lane], the counts to the rows. A thread meets the
                    //      same home point in all of its tasks (256 is a multiple of 32). ----
                    uint32_t* mask_tile = masks + base + (static_cast<unsigned long long>(tile) * words + word_base + (batch0 >> 5)) * TILE_POINTS;
                    const int4 home = sh.home_sj[lane];
                    // full lists: the only candidate to drop is the point itself, whose slot is known
                    const int self_bit = (g == own_group) ? own_slot0 + tile * TILE_POINTS + lane - batch0 : -1;
                    int my_hits = 0;
                    for (int task = threadIdx.x; task < batch_words * TILE_POINTS; task += CTA_THREADS) {
                        unsigned word = sh.mask[task];
                        unsigned kept = word;
                        const int slot0 = (task >> 5) << 5;
                        if (FULL && !own_straddles) {
                            if (self_bit >= slot0 && self_bit < slot0 + 32) {
                                kept &= ~(1u << (self_bit - slot0));
                            }
                        } else {
                            kept = 0;
                            while (word != 0) {
                                const int b = __ffs(word) - 1;
                                word &= word - 1;
                                if (row_keeps<FULL>(home, sh.sj[slot0 + b])) {
                                    kept |= 1u << b;
                                }
                            }
                        }
                        mask_tile[task] = kept;
                        my_hits += __popc(kept);
                    }
                    if (my_hits != 0) {
                        atomicAdd(&rows.tile_hits[lane], my_hits);
                    }
                    __syncthreads();
                    if (threadIdx.x < TILE_POINTS) {
                        const int hits = rows.tile_hits[threadIdx.x];
                        if (hits != 0) {
                            atomicAdd(&row_count[sh.home_sj[threadIdx.x].w], static_cast<uint32_t>(hits));
                            rows.tile_hits[threadIdx.x] = 0;
                        }
                    }
                }
                __syncthreads();
            }
            word_base += (group_total + 31) >> 5;
        }
    }
}

/// 12-byte element at a 4-byte aligned address: one 8-byte and one 4-byte store.
template <typename T>
__device__ __forceinline__ void store_triple_32(T* base, unsigned long long element, T a, T b, T c) {
    static_assert(sizeof(T) == 4, "int32 shifts or float vectors");
    T* dst = base + 3 * element;
    struct alignas(8) Two {
        T x, y;
    };
    // (streaming stores, like every store of a list: see emit.cuh)
    static_assert(sizeof(Two) == sizeof(float2), "stored as one 8-byte word");
    float2 pair;
    if ((element & 1ull) == 0) {
        const Two two{a, b};
        memcpy(&pair, &two, sizeof(pair));
        __stcs(reinterpret_cast<float2*>(dst), pair);
        __stcs(dst + 2, c);
    } else {
        const Two two{b, c};
        memcpy(&pair, &two, sizeof(pair));
        __stcs(dst, a);
        __stcs(reinterpret_cast<float2*>(dst + 1), pair);
    }
}

/// 24-byte element at an 8-byte aligned address: one 16-byte and one 8-byte store.
__device__ __forceinline__ void store_triple_64(double* base, unsigned long long element, double a, double b, double c) {
    double* dst = base + 3 * element;
    if ((element & 1ull) == 0) {
        __stcs(reinterpret_cast<double2*>(dst), make_double2(a, b));
        __stcs(dst + 2, c);
    } else {
        __stcs(dst, a);
        __stcs(reinterpret_cast<double2*>(dst + 1), make_double2(b, c));
    }
}

__global__ void __launch_bounds__(CTA_THREADS, 4) row_emit_kernel(
    const GridPlan plan, const int32_t* __restrict__ cell_start, SortedPoints sorted, const uint32_t* __restrict__ masks,
    const unsigned long long* __restrict__ unit_mask_base, const uint32_t* __restrict__ unit_words,
    const unsigned long long* __restrict__ row_start, uint32_t* __restrict__ row_fill, PairOutput out
) {
    extern __shared__ __align__(16) unsigned char row_smem[];
    RowShared& rows = *reinterpret_cast<RowShared*>(row_smem);
    FusedShared& sh = rows.staged;
    static_assert(FUSED_WORDS == 16 && FUSED_TASKS == 2, "tasks are (home point, word) pairs: home = task >> 4");

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    for (int u = blockIdx.x; u < plan.n_units; u += gridDim.x) {
        const Unit unit = unit_of(plan, cell_start, u);
        if (unit.n_home == 0) {
            continue;
        }
        const int n_groups = (unit.n_stencil + SEG_MAX - 1) / SEG_MAX;
        const int n_tiles = (unit.n_home + TILE_POINTS - 1) / TILE_POINTS;
        const unsigned long long base = unit_mask_base[u];
        const int words = static_cast<int>(unit_words[u]);

        int word_base = 0;
        for (int g = 0; g < n_groups; g++) {
            const int group_total = setup_segments(plan, cell_start, unit, g, sh.table);
            for (int batch0 = 0; batch0 < group_total; batch0 += FUSED_BATCH) {
                const int batch_slots = min(FUSED_BATCH, group_total - batch0);
                const int batch_words = (batch_slots + 31) >> 5;
                stage_row_batch<false>(sh, plan, sorted, unit.n_stencil, batch0, batch_slots);

                for (int tile = 0; tile < n_tiles; tile++) {
                    __syncthreads(); // staging done; previous tile done with the shared arrays
                    if (threadIdx.x < TILE_POINTS) {
                        const int il = tile * TILE_POINTS + threadIdx.x;
                        if (il < unit.n_home) {
                            const size_t pi = static_cast<size_t>(unit.begin) + il;
                            const int index_i = sorted.index[pi];
                            sh.home_pos[0][threadIdx.x] = sorted.pos[3 * pi + 0];
                            sh.home_pos[1][threadIdx.x] = sorted.pos[3 * pi + 1];
                            sh.home_pos[2][threadIdx.x] = sorted.pos[3 * pi + 2];
                            sh.home_sj[threadIdx.x] = make_int4(sorted.shift[3 * pi + 0], sorted.shift[3 * pi + 1], sorted.shift[3 * pi + 2], index_i);
                            rows.home_row[threadIdx.x] = row_start[index_i] + row_fill[index_i];
                        }
                    }
                    // hit words of the tile, transposed to [home point][word] so that the hits of a
                    // point are consecutive tasks; words past the batch hold nothing
                    const uint32_t* mask_tile = masks + base + (static_cast<unsigned long long>(tile) * words + word_base + (batch0 >> 5)) * TILE_POINTS;
                    for (int k = threadIdx.x; k < FUSED_WORDS * TILE_POINTS; k += CTA_THREADS) {
                        const int w = k >> 5;
                        sh.mask[(k & 31) * FUSED_WORDS + w] = (w < batch_words) ? mask_tile[k] : 0u;
                    }
                    __syncthreads();

                    // ---- scan of the hit counts of the tasks (two consecutive tasks per thread) ----
                    const unsigned word_a = sh.mask[2 * threadIdx.x];
                    const unsigned word_b = sh.mask[2 * threadIdx.x + 1];
                    const int my_hits = __popc(word_a) + __popc(word_b);
                    int inclusive = my_hits;
#pragma unroll
                    for (int offset = 1; offset < 32; offset <<= 1) {
                        const int up = __shfl_up_sync(FULL_MASK, inclusive, offset);
                        if (lane >= offset) {
                            inclusive += up;
                        }
                    }
                    sh.prefix[threadIdx.x] = static_cast<unsigned short>(inclusive - my_hits);
                    if (lane == 31) {
                        sh.table.scan_tmp[warp] = inclusive;
                    }
                    __syncthreads();
                    int total_hits = 0;
                    int before_warp = 0;
#pragma unroll
                    for (int w = 0; w < CTA_WARPS; w++) {
                        const int sum = sh.table.scan_tmp[w];
                        if (w < warp) {
                            before_warp += sum;
                        }
                        total_hits += sum;
                    }
                    // the thread that owns the first task of a home point knows where its hits start
                    if ((threadIdx.x & 7) == 0) {
                        rows.row_offset[threadIdx.x >> 3] = before_warp + inclusive - my_hits;
                    }
                    if (threadIdx.x == 0) {
                        rows.row_offset[TILE_POINTS] = total_hits;
                    }

                    for (int round0 = 0; round0 < total_hits; round0 += FUSED_LIST) {
                        if (round0 != 0) {
                            __syncthreads(); // previous round consumed
                        }
                        const int in_round = min(FUSED_LIST, total_hits - round0);
                        {
                            // every thread writes the same number of consecutive list entries (see the fused pass)
                            const int quota = (in_round + CTA_THREADS - 1) / CTA_THREADS;
                            int position = round0 + threadIdx.x * quota;
                            const int stop = min(position + quota, round0 + in_round);
                            if (position < stop) {
                                int owner_warp = 0;
                                int before = 0;
                                {
                                    int running = 0;
#pragma unroll
                                    for (int w = 0; w < CTA_WARPS - 1; w++) {
                                        running += sh.table.scan_tmp[w];
                                        if (running <= position) {
                                            owner_warp = w + 1;
                                            before = running;
                                        }
                                    }
                                }
                                const int target = position - before;
                                const unsigned short* local = sh.prefix + owner_warp * 32;
                                int lo = 0;
                                int hi = 32;
#pragma unroll
                                for (int step = 0; step < 5; step++) {
                                    const int mid = (lo + hi) >> 1;
                                    if (static_cast<int>(local[mid]) <= target) {
                                        lo = mid;
                                    } else {
                                        hi = mid;
                                    }
                                }
                                int skip = target - static_cast<int>(local[lo]);
                                lo += owner_warp * 32;
                                int task = lo * 2;
                                unsigned word = sh.mask[task];
                                {
                                    const int count = __popc(word);
                                    if (skip >= count) {
                                        skip -= count;
                                        task++;
                                        word = sh.mask[task];
                                    }
                                }
                                word &= 0xffffffffu << select_bit(word, skip);
                                for (; position < stop; position++) {
                                    while (word == 0 && task + 1 < FUSED_WORDS * TILE_POINTS) {
                                        task++;
                                        word = sh.mask[task];
                                    }
                                    const int bit = __ffs(word) - 1;
                                    word &= word - 1;
                                    // (home point << 9) | slot in the batch
                                    sh.list[position - round0] = static_cast<unsigned short>(((task >> 4) << 9) | ((task & 15) << 5) | (bit & 31));
                                }
                            }
                        }
                        __syncthreads();

                        for (int chunk0 = warp * 32; chunk0 < in_round; chunk0 += CTA_WARPS * 32) {
                            if (chunk0 + lane >= in_round) {
                                continue;
                            }
                            const unsigned entry = sh.list[chunk0 + lane];
                            const int h = entry >> 9;
                            const int s = entry & 511;
                            const int4 cand = sh.sj[s];
                            const int4 home = sh.home_sj[h];
                            const int s0 = cand.x + home.x;
                            const int s1 = cand.y + home.y;
                            const int s2 = cand.z + home.z;
                            double vx, vy, vz;
                            const double d2 = exact_pair(
                                plan, sh.home_pos[0][h], sh.home_pos[1][h], sh.home_pos[2][h], sh.x[s], sh.y[s], sh.z[s], s0, s1, s2, vx, vy, vz
                            );
                            const unsigned long long dest = rows.home_row[h] + static_cast<unsigned long long>(round0 + chunk0 + lane - rows.row_offset[h]);
                            __stcs(
                                reinterpret_cast<ulonglong2*>(out.pairs) + dest,
                                make_ulonglong2(static_cast<unsigned long long>(home.w), static_cast<unsigned long long>(cand.w))
                            );
                            if (out.shifts != nullptr) {
                                store_triple_32(out.shifts, dest, s0, s1, s2);
                            }
                            if (out.values_float) {
                                if (out.distances != nullptr) {
                                    __stcs(reinterpret_cast<float*>(out.distances) + dest, static_cast<float>(__dsqrt_rn(d2)));
                                }
                                if (out.vectors != nullptr) {
                                    store_triple_32(
                                        reinterpret_cast<float*>(out.vectors), dest, static_cast<float>(vx), static_cast<float>(vy), static_cast<float>(vz)
                                    );
                                }
                            } else {
                                if (out.distances != nullptr) {
                                    __stcs(out.distances + dest, __dsqrt_rn(d2));
                                }
                                if (out.vectors != nullptr) {
                                    store_triple_64(out.vectors, dest, vx, vy, vz);
                                }
                            }
                        }
                    }
                    __syncthreads();
                    if (threadIdx.x < TILE_POINTS && tile * TILE_POINTS + threadIdx.x < unit.n_home) {
                        const int hits = rows.row_offset[threadIdx.x + 1] - rows.row_offset[threadIdx.x];
                        if (hits != 0) {
                            row_fill[sh.home_sj[threadIdx.x].w] += static_cast<uint32_t>(hits);
                        }
                    }
                }
                __syncthreads();
            }
            word_base += (group_total + 31) >> 5;
        }
    }
}

// ---------------------------------------------------------------------------
// canonical order inside the rows
// A list sorted by the first index becomes THE canonical list (rows ordered by
// second index, then by shift) when every row is sorted. Rows are short (tens
// to hundreds of pairs), so a warp ranks the pairs of a row against each other
// (the rank of a pair is the number of pairs of the row that come before it)
// and copies every pair to its place in a second set of arrays. No counterpart
// in the reference, whose device sort stops at the first index
// (vesin/src/cuda/sort_pairs.cu:3-12).
// ---------------------------------------------------------------------------

__device__ __forceinline__ bool shift_before(const int32_t* __restrict__ shifts, unsigned long long a, unsigned long long b) {
    if (shifts == nullptr) {
        return false;
    }
#pragma unroll
    for (int c = 0; c < 3; c++) {
        const int sa = shifts[3 * a + c];
        const int sb = shifts[3 * b + c];
        if (sa != sb) {
            return sa < sb;
        }
    }
    return false;
}

constexpr int ROW_SORT_STAGED = 512; // second indices of a row a warp keeps in shared memory

/// One pair of a list on its way from one place to another.
template <bool FLOAT>
struct PairInFlight {
    ulonglong2 pair;
    int s0, s1, s2;
    typename std::conditional<FLOAT, float, double>::type d, vx, vy, vz;
};

template <bool FLOAT>
__device__ __forceinline__ PairInFlight<FLOAT> load_pair(const PairOutput& in, unsigned long long from) {
    using Real = typename std::conditional<FLOAT, float, double>::type;
    PairInFlight<FLOAT> p{};
    p.pair = __ldcs(reinterpret_cast<const ulonglong2*>(in.pairs) + from);
    if (in.shifts != nullptr) {
        p.s0 = __ldcs(in.shifts + 3 * from + 0);
        p.s1 = __ldcs(in.shifts + 3 * from + 1);
        p.s2 = __ldcs(in.shifts + 3 * from + 2);
    }
    if (in.distances != nullptr) {
        p.d = __ldcs(reinterpret_cast<const Real*>(in.distances) + from);
    }
    if (in.vectors != nullptr) {
        const Real* v = reinterpret_cast<const Real*>(in.vectors) + 3 * from;
        p.vx = __ldcs(v);
        p.vy = __ldcs(v + 1);
        p.vz = __ldcs(v + 2);
    }
    return p;
}

template <bool FLOAT>
__device__ __forceinline__ void store_pair(const PairOutput& out, unsigned long long to, const PairInFlight<FLOAT>& p) {
    __stcs(reinterpret_cast<ulonglong2*>(out.pairs) + to, p.pair);
    if (out.shifts != nullptr) {
        store_triple_32(out.shifts, to, p.s0, p.s1, p.s2);
    }
    if (FLOAT) {
        if (out.distances != nullptr) {
            __stcs(reinterpret_cast<float*>(out.distances) + to, static_cast<float>(p.d));
        }
        if (out.vectors != nullptr) {
            store_triple_32(reinterpret_cast<float*>(out.vectors), to, static_cast<float>(p.vx), static_cast<float>(p.vy), static_cast<float>(p.vz));
        }
    } else {
        if (out.distances != nullptr) {
            __stcs(out.distances + to, static_cast<double>(p.d));
        }
        if (out.vectors != nullptr) {
            store_triple_64(out.vectors, to, static_cast<double>(p.vx), static_cast<double>(p.vy), static_cast<double>(p.vz));
        }
    }
}

/// A warp per row: every pair of the row is ranked against the others by (second index,
/// shift) and copied to its place in `out`. Rows of up to ROW_SORT_STAGED pairs keep their
/// second indices in shared memory; a lane takes three pairs per pass, starts the loads of
/// everything it will copy, ranks both pairs against the row while the loads are in flight
/// (four comparisons per 16-byte load and pair), then stores. DUPLICATES = false: the caller
/// knows that no second index comes twice in a row (no lattice vector shorter than twice the
/// cutoff), so the comparisons of shifts are left out altogether.
template <bool DUPLICATES, bool FLOAT>
__global__ void __launch_bounds__(CTA_THREADS, 3) row_sort_kernel(
    const unsigned long long* __restrict__ row_start, size_t n_rows, PairOutput in, PairOutput out
) {
    __shared__ __align__(16) unsigned row_keys[CTA_WARPS][ROW_SORT_STAGED];
    constexpr int PER_LANE = 3; // a row of up to 96 pairs is one pass
    const int lane = threadIdx.x & 31;
    unsigned* keys = row_keys[threadIdx.x >> 5];
    const size_t warps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
    for (size_t row = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; row < n_rows; row += warps) {
        const unsigned long long begin = row_start[row];
        const unsigned long long length = row_start[row + 1] - begin;
        if (length <= ROW_SORT_STAGED) {
            // indices fit 31 bits: the low words of the second indices of the row, padded with
            // the largest key to a multiple of four
            const int n = static_cast<int>(length);
            const int n4 = (n + 3) >> 2;
            __syncwarp();
            for (int e = lane; e < 4 * n4; e += 32) {
                keys[e] = (e < n) ? static_cast<unsigned>(in.pairs[2 * (begin + e) + 1]) : 0xffffffffu;
            }
            __syncwarp();
            const uint4* four = reinterpret_cast<const uint4*>(keys);
            for (int base = 0; base < n; base += 32 * PER_LANE) {
                // pairs base + lane + 32 m of the row
                PairInFlight<FLOAT> moving[PER_LANE];
                unsigned key[PER_LANE];
                int smaller[PER_LANE];
                int equal[PER_LANE];
#pragma unroll
                for (int m = 0; m < PER_LANE; m++) {
                    const int e = base + lane + 32 * m;
                    smaller[m] = 0;
                    equal[m] = 0;
                    key[m] = (e < n) ? keys[e] : 0u;
                    if (e < n) {
                        moving[m] = load_pair<FLOAT>(in, begin + e);
                    }
                }
                for (int k = 0; k < n4; k++) {
                    const uint4 others = four[k]; // the same address for every lane
#pragma unroll
                    for (int m = 0; m < PER_LANE; m++) {
                        smaller[m] += (others.x < key[m]) + (others.y < key[m]) + (others.z < key[m]) + (others.w < key[m]);
                        if (DUPLICATES) {
                            equal[m] += (others.x == key[m]) + (others.y == key[m]) + (others.z == key[m]) + (others.w == key[m]);
                        }
                    }
                }
#pragma unroll
                for (int m = 0; m < PER_LANE; m++) {
                    const int e = base + lane + 32 * m;
                    if (e >= n) {
                        continue;
                    }
                    const unsigned long long mine = begin + e;
                    unsigned long long rank = static_cast<unsigned long long>(smaller[m]);
                    if (DUPLICATES && equal[m] > 1) {
                        // the same second index several times in the row (periodic images): shifts decide
                        for (int k = 0; k < n; k++) {
                            if (keys[k] == key[m] && k != e &&
                                (shift_before(in.shifts, begin + k, mine) || (k < e && !shift_before(in.shifts, mine, begin + k)))) {
                                rank++;
                            }
                        }
                    }
                    store_pair<FLOAT>(out, begin + rank, moving[m]);
                }
            }
        } else {
            for (unsigned long long e = lane; e < length; e += 32) {
                const unsigned long long mine = begin + e;
                const unsigned long long j = in.pairs[2 * mine + 1];
                unsigned long long rank = 0;
                for (unsigned long long k = 0; k < length; k++) {
                    const unsigned long long other = in.pairs[2 * (begin + k) + 1]; // the same address for every lane
                    if (other < j || (other == j && (shift_before(in.shifts, begin + k, mine) || (k < e && !shift_before(in.shifts, mine, begin + k))))) {
                        rank++;
                    }
                }
                store_pair<FLOAT>(out, begin + rank, load_pair<FLOAT>(in, mine));
            }
        }
    }
}

} // namespace
#ifdef VESIN_B200_PHASE_CLOCKS
extern "C" __attribute__((visibility("default"))) void vesin_b200_debug_phase_clocks(unsigned long long* out, int reset) {
    cudaMemcpyFromSymbol(out, g_phase_clocks, sizeof(g_phase_clocks));
    if (reset) {
        const unsigned long long zeros[16] = {0};
        cudaMemcpyToSymbol(g_phase_clocks, zeros, sizeof(zeros));
    }
}
#endif
namespace {
/// Launch as a link of the chain of a build (see let_next_kernel_start).
template <typename... KernelArgs, typename... Args>
void launch_chained(void (*kernel)(KernelArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(block);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

int pair_grid(int n_units, int per_sm) {
    int device = 0;
    int sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    }
    long long cap = static_cast<long long>(sms) * per_sm;
    return static_cast<int>(n_units < cap ? n_units : cap);
}

} // namespace

// ---------------------------------------------------------------------------
// launch wrappers
// ---------------------------------------------------------------------------

void configure_kernels() {
    cudaFuncSetAttribute(row_count_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(RowShared)));
    cudaFuncSetAttribute(row_count_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(RowShared)));
    cudaFuncSetAttribute(row_emit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(RowShared)));
    cudaFuncSetAttribute(pairs_kernel<false, false, SmallCta>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(SmallCta::Shared)));
    cudaFuncSetAttribute(pairs_kernel<true, false, SmallCta>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(SmallCta::Shared)));
    cudaFuncSetAttribute(pairs_kernel<false, true, LargeCta>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(LargeCta::Shared)));
    cudaFuncSetAttribute(pairs_kernel<true, true, LargeCta>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(LargeCta::Shared)));
}

static ExpectedInputs expected_inputs(const double box[9], const bool periodic[3]) {
    ExpectedInputs expected;
    for (int k = 0; k < 9; k++) {
        expected.box[k] = box[k];
    }
    for (int k = 0; k < 3; k++) {
        expected.periodic[k] = periodic[k] ? 1 : 0;
    }
    return expected;
}

static unsigned header_blocks(size_t n_zero) {
    size_t blocks = (n_zero + CTA_THREADS * 4 - 1) / (CTA_THREADS * 4);
    return static_cast<unsigned>(std::max<size_t>(1, std::min<size_t>(blocks, 148 * 4)));
}

void launch_header_init(DeviceHeader* header, RealView box, const bool* periodic, cudaStream_t stream) {
    header_init_kernel<<<1, CTA_THREADS, 0, stream>>>(header, box, periodic, nullptr, 0, 0, ExpectedInputs{});
}

void launch_header_reset(DeviceHeader* header, int32_t* zero, size_t n_zero, cudaStream_t stream) {
    header_init_kernel<<<header_blocks(n_zero), CTA_THREADS, 0, stream>>>(header, RealView{nullptr, 0}, nullptr, zero, n_zero, 0, ExpectedInputs{});
}

void launch_header_init_speculative(
    DeviceHeader* header, RealView box, const bool* periodic, int32_t* zero, size_t n_zero, const double expected_box[9],
    const bool expected_periodic[3], cudaStream_t stream
) {
    header_init_kernel<<<header_blocks(n_zero), CTA_THREADS, 0, stream>>>(
        header, box, periodic, zero, n_zero, 1, expected_inputs(expected_box, expected_periodic)
    );
}

void launch_bounds(const PointSource& source, DeviceHeader* header, cudaStream_t stream) {
    const size_t n = source.n_index();
    if (n == 0) {
        return;
    }
    // every block ends with seven atomics on the same few words of the header: few blocks,
    // eight points or more per thread
    size_t blocks = (n + 8 * CTA_THREADS - 1) / (8 * CTA_THREADS);
    blocks = std::max<size_t>(1, std::min<size_t>(blocks, 148 * 2));
    if (source.message[0] != nullptr) {
        bounds_kernel<true><<<static_cast<unsigned>(blocks), CTA_THREADS, 0, stream>>>(source, n, header);
    } else {
        bounds_kernel<false><<<static_cast<unsigned>(blocks), CTA_THREADS, 0, stream>>>(source, n, header);
    }
}

void launch_bin(
    const PointSource& source, size_t first, size_t last, const GridPlan& plan, int32_t* cell_of, int32_t* rank, int32_t* shift,
    int32_t* cell_count, DeviceHeader* header, bool check_points, bool chained, cudaStream_t stream
) {
    if (last <= first) {
        return;
    }
    const unsigned blocks = static_cast<unsigned>((last - first + CTA_THREADS - 1) / CTA_THREADS);
    const int check = check_points ? 1 : 0;
    const bool halo = source.message[0] != nullptr && source.capacity > 0;
    if (halo && chained) {
        launch_chained(bin_kernel<true>, blocks, CTA_THREADS, 0, stream, source, first, last, plan, cell_of, rank, shift, cell_count, header, check);
    } else if (halo) {
        bin_kernel<true><<<blocks, CTA_THREADS, 0, stream>>>(source, first, last, plan, cell_of, rank, shift, cell_count, header, check);
    } else if (chained) {
        launch_chained(bin_kernel<false>, blocks, CTA_THREADS, 0, stream, source, first, last, plan, cell_of, rank, shift, cell_count, header, check);
    } else {
        bin_kernel<false><<<blocks, CTA_THREADS, 0, stream>>>(source, first, last, plan, cell_of, rank, shift, cell_count, header, check);
    }
}

size_t scan_tmp_bytes(size_t n) {
    size_t tiles = (n + SCAN_TILE - 1) / SCAN_TILE;
    return (tiles + 1) * sizeof(unsigned long long);
}

template <typename TIn, typename TOut>
static void launch_scan(
    const TIn* counts, TOut* starts, size_t n, void* tmp, unsigned long long* total, cudaStream_t stream, const TOut* first_value = nullptr
) {
    auto* tile_sums = static_cast<unsigned long long*>(tmp);
    size_t tiles = (n + SCAN_TILE - 1) / SCAN_TILE;
    launch_chained(scan_tile_sums_kernel<TIn>, static_cast<unsigned>(tiles), CTA_THREADS, 0, stream, counts, n, tile_sums);
    if (tiles <= 2048) {
        // short spine: every block of the second kernel adds up the tile sums before it
        launch_chained(
            scan_apply_kernel<TIn, TOut, true>, static_cast<unsigned>(tiles), CTA_THREADS, 0, stream, counts, starts, n, tile_sums, total, first_value
        );
    } else {
        scan_spine_kernel<<<1, CTA_THREADS, 0, stream>>>(tile_sums, tiles, total);
        scan_apply_kernel<TIn, TOut, false><<<static_cast<unsigned>(tiles), CTA_THREADS, 0, stream>>>(counts, starts, n, tile_sums, nullptr, first_value);
    }
}

void launch_scan_cells(const int32_t* counts, int32_t* starts, size_t n, void* tmp, cudaStream_t stream, const int32_t* first_value) {
    launch_scan<int32_t, int32_t>(counts, starts, n, tmp, nullptr, stream, first_value);
}

void launch_scan_rows(
    const uint32_t* counts, unsigned long long* starts, size_t n, void* tmp, unsigned long long* total, cudaStream_t stream
) {
    launch_scan<uint32_t, unsigned long long>(counts, starts, n, tmp, total, stream);
}

void launch_scatter(
    const PointSource& source, const int32_t* cell_of, const int32_t* rank, const int32_t* shift, const int32_t* cell_start,
    size_t n_cells, SortedPoints sorted, int32_t* sorted_global, DeviceHeader* header, cudaStream_t stream, size_t first, size_t last
) {
    if (last == static_cast<size_t>(-1)) {
        last = source.n_index();
    }
    if (last <= first) {
        return;
    }
    // local indices [first, last) go to records [first, last) at most: cells are filled in the order
    // of the local indices' segments (see the slab build), or the range is everything
    const size_t n = last - first;
    const unsigned index_blocks = static_cast<unsigned>((n + CTA_THREADS - 1) / CTA_THREADS);
    const unsigned record_blocks = static_cast<unsigned>((3 * n + CTA_THREADS - 1) / CTA_THREADS);
    // records below source.n0 are the points of the caller's array: all there; further on the
    // local index space may hold empty slots and the number of records (known once every cell
    // has its start) bounds the range
    const int32_t* n_records = (last <= source.n0) ? nullptr : cell_start + n_cells;
    const DeviceHeader* read_header = header;
    if (source.message[0] != nullptr && source.capacity > 0) {
        launch_chained(scatter_index_kernel<true>, index_blocks, CTA_THREADS, 0, stream, source, first, last, cell_of, rank, cell_start, sorted.index, read_header);
        launch_chained(gather_records_kernel<true>, record_blocks, CTA_THREADS, 0, stream, source, first, last, n_records, shift, sorted, sorted_global, header);
    } else {
        launch_chained(scatter_index_kernel<false>, index_blocks, CTA_THREADS, 0, stream, source, first, last, cell_of, rank, cell_start, sorted.index, read_header);
        launch_chained(gather_records_kernel<false>, record_blocks, CTA_THREADS, 0, stream, source, first, last, n_records, shift, sorted, sorted_global, header);
    }
}

void launch_count(
    const GridPlan& plan, const int32_t* cell_start, SortedPoints sorted, uint32_t* masks, unsigned long long mask_capacity,
    unsigned long long* unit_mask_base, uint32_t* unit_words, uint32_t* row_count, DeviceHeader* header, cudaStream_t stream
) {
    const int grid = pair_grid(plan.n_units, 4);
    if (plan.full) {
        row_count_kernel<true><<<grid, CTA_THREADS, sizeof(RowShared), stream>>>(
            plan, cell_start, sorted, masks, mask_capacity, unit_mask_base, unit_words, row_count, header
        );
    } else {
        row_count_kernel<false><<<grid, CTA_THREADS, sizeof(RowShared), stream>>>(
            plan, cell_start, sorted, masks, mask_capacity, unit_mask_base, unit_words, row_count, header
        );
    }
}

void launch_emit(
    const GridPlan& plan, const int32_t* cell_start, SortedPoints sorted, const uint32_t* masks, const unsigned long long* unit_mask_base,
    const uint32_t* unit_words, const unsigned long long* row_start, uint32_t* row_fill, PairOutput out, cudaStream_t stream
) {
    const int grid = pair_grid(plan.n_units, 4);
    row_emit_kernel<<<grid, CTA_THREADS, sizeof(RowShared), stream>>>(
        plan, cell_start, sorted, masks, unit_mask_base, unit_words, row_start, row_fill, out
    );
}

void launch_sort_rows(
    const unsigned long long* row_start, size_t n_rows, PairOutput in, PairOutput out, bool duplicates_possible, cudaStream_t stream
) {
    if (n_rows == 0) {
        return;
    }
    // a warp per row, eight rows per CTA
    const size_t blocks = std::min<size_t>((n_rows + CTA_WARPS - 1) / CTA_WARPS, 148 * 64);
    const auto launch = [&](auto kernel) { kernel<<<static_cast<unsigned>(blocks), CTA_THREADS, 0, stream>>>(row_start, n_rows, in, out); };
    if (in.values_float) {
        duplicates_possible ? launch(row_sort_kernel<true, true>) : launch(row_sort_kernel<false, true>);
    } else {
        duplicates_possible ? launch(row_sort_kernel<true, false>) : launch(row_sort_kernel<false, false>);
    }
}

void launch_pairs(
    const GridPlan& plan, const int32_t* cell_start, SortedPoints sorted, PairOutput out, unsigned long long capacity,
    DeviceHeader* header, cudaStream_t stream, size_t n_records, int part
) {
    // as many CTAs as are resident (by registers and shared memory), which take
    // runs of units from a shared counter; small systems give every unit its own CTA
    // instead of runs of neighbouring units
    int sms = 148;
    {
        int device = 0;
        if (cudaGetDevice(&device) == cudaSuccess) {
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        }
    }
    // paired stores of full lists: 32 bytes of indices, 16 of distances / vectors, 8 of shifts
    // (half of that for float values); null arrays are not written
    const auto aligned = [](const void* pointer, uintptr_t bytes) { return reinterpret_cast<uintptr_t>(pointer) % bytes == 0; };
    const uintptr_t value_bytes = out.values_float ? 8 : 16;
    out.interleave_ok = aligned(out.pairs, 32) && aligned(out.shifts, 8) && aligned(out.distances, value_bytes) && aligned(out.vectors, value_bytes);

    const auto launch = [&](auto shape, auto kernel, UnitRanges ranges, unsigned long long* run_cursor, bool follows = false) {
        using Shape = decltype(shape);
        const int per_sm = Shape::CTAS_PER_SM;
        const size_t smem = sizeof(typename Shape::Shared);
        const int n_units = (ranges.end0 - ranges.begin0) + (ranges.end1 - ranges.begin1);
        if (n_units <= 0) {
            return;
        }
        // at least 8 runs per CTA, so that the last runs do not leave most of the GPU idle
        const int unit_run = std::max(1, std::min(DEFAULT_UNIT_RUN, n_units / (sms * 4 * 8)));
        int runs = (ranges.end0 - ranges.begin0 + unit_run - 1) / unit_run + (ranges.end1 - ranges.begin1 + unit_run - 1) / unit_run;
        // A handful of units whose stencils hold many batches of candidates (a small box with
        // many images): several CTAs share the batches of a unit.
        if (unit_run == 1 && runs * 2 <= sms * per_sm && plan.n_cells_total > 0 && n_records > 0) {
            const int row_width = plan.pencil + 2 * plan.n_search[0];
            const int rows_above = plan.n_search[1] + plan.n_search[2] * (2 * plan.n_search[1] + 1);
            const double stencil_cells = static_cast<double>(plan.pencil + plan.n_search[0]) + static_cast<double>(row_width) * rows_above;
            const double per_cell = static_cast<double>(n_records) / static_cast<double>(plan.n_cells_total);
            const double batches = std::ceil(stencil_cells * per_cell / Shape::BATCH);
            const int wanted = std::min(MAX_UNIT_SPLITS, (sms * per_sm) / runs);
            ranges.splits = std::max(1, static_cast<int>(std::min<double>(wanted, batches)));
            runs *= ranges.splits;
        }
        const int grid = pair_grid(runs, per_sm);
        launch_chained(
            kernel, grid, Shape::THREADS, smem, stream, plan, cell_start, sorted, out, capacity, header, unit_run, ranges, run_cursor, follows ? 1 : 0
        );
    };
    const UnitRanges all{0, plan.n_units, 0, 0};
    if (plan.window_axis < 0) {
        if (plan.full) {
            launch(SmallCta{}, pairs_kernel<true, false, SmallCta>, all, &header->run_cursor);
        } else {
            launch(SmallCta{}, pairs_kernel<false, false, SmallCta>, all, &header->run_cursor);
        }
    } else if (plan.window_axis == 2) {
        // Slab cut along the last direction: a layer of cells is a contiguous range of units.
        // Units whose whole stencil holds owned points are ordinary units: they take the
        // plain kernel. Half lists: every owned layer (a unit pairs with the layer above it;
        // the pairs with halo points above are this rank's too). Full lists: the lower halo
        // layer and the last owned layer write one orientation of some of
        // their pairs only: they go to the slab kernel, launched behind the plain one (whose
        // tail its blocks fill, see the top of the kernel) so that the blocks of odd length it
        // may claim move few of the plain kernel's blocks off their alignment.
        // (layers are stored as: owned layers, upper halo layer, lower halo layer)
        // The units below the last owned layer need nothing from the halo: a caller may launch
        // them (PAIR_PART_INTERIOR) while the halo is still on its way, and the rest
        // (PAIR_PART_BOUNDARY) once it has been sorted in. The two parts take their runs from
        // two counters.
        const int per_layer = plan.n_units / plan.n_cells[2];
        const int owned_layers = plan.n_cells[2] - 2;
        const int interior_end = per_layer * (owned_layers - 1);
        if (!plan.full) {
            if (part == PAIR_PART_ALL) {
                launch(SmallCta{}, pairs_kernel<false, false, SmallCta>, UnitRanges{0, per_layer * owned_layers, 0, 0}, &header->run_cursor);
            } else if (part == PAIR_PART_INTERIOR) {
                launch(SmallCta{}, pairs_kernel<false, false, SmallCta>, UnitRanges{0, interior_end, 0, 0}, &header->run_cursor);
            } else {
                launch(SmallCta{}, pairs_kernel<false, false, SmallCta>, UnitRanges{interior_end, per_layer * owned_layers, 0, 0}, &header->mask_cursor);
            }
        } else {
            if (part != PAIR_PART_BOUNDARY) {
                launch(SmallCta{}, pairs_kernel<true, false, SmallCta>, UnitRanges{0, interior_end, 0, 0}, &header->run_cursor);
            }
            if (part != PAIR_PART_INTERIOR) {
                launch(
                    LargeCta{}, pairs_kernel<true, true, LargeCta>,
                    UnitRanges{interior_end, per_layer * owned_layers, per_layer * (owned_layers + 1), per_layer * (owned_layers + 2)},
                    &header->mask_cursor, /*follows=*/part == PAIR_PART_ALL && owned_layers > 1
                );
            }
        }
    } else if (plan.full) {
        launch(LargeCta{}, pairs_kernel<true, true, LargeCta>, all, &header->run_cursor);
    } else {
        launch(LargeCta{}, pairs_kernel<false, true, LargeCta>, all, &header->run_cursor);
    }
}

bool pairs_have_interior(const GridPlan& plan) {
    return plan.window_axis == 2 && plan.n_cells[2] - 2 > 1;
}

// ---------------------------------------------------------------------------
// checksum of a list
// Lists of the same system built by different decompositions (one GPU, slabs
// over several GPUs, the CPU reference) hold the same rows in different orders;
// a sum of per-row hashes compares them without sorting 10^8 rows.
// ---------------------------------------------------------------------------

namespace {

__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdull;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ull;
    x ^= x >> 33;
    return x;
}

__global__ void __launch_bounds__(CTA_THREADS) checksum_kernel(
    const unsigned long long* __restrict__ pairs, const int32_t* __restrict__ shifts, const double* __restrict__ distances,
    const int values_float, size_t n, unsigned long long* __restrict__ result
) {
    unsigned long long h0 = 0, h1 = 0, h2 = 0;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t r = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; r < n; r += stride) {
        const ulonglong2 ij = reinterpret_cast<const ulonglong2*>(pairs)[r];
        unsigned long long key = ij.x * 0x9e3779b97f4a7c15ull + ij.y * 0xc2b2ae3d27d4eb4full;
        if (shifts != nullptr) {
            key += static_cast<unsigned long long>(static_cast<unsigned>(shifts[3 * r + 0])) * 0x165667b19e3779f9ull;
            key += static_cast<unsigned long long>(static_cast<unsigned>(shifts[3 * r + 1])) * 0x27d4eb2f165667c5ull;
            key += static_cast<unsigned long long>(static_cast<unsigned>(shifts[3 * r + 2])) * 0x85ebca77c2b2ae63ull;
        }
        unsigned long long value_bits = 0;
        if (distances != nullptr) {
            value_bits = values_float ? static_cast<unsigned long long>(__float_as_uint(reinterpret_cast<const float*>(distances)[r]))
                                      : static_cast<unsigned long long>(__double_as_longlong(distances[r]));
        }
        h0 += mix64(key);
        h1 += mix64(key ^ 0x5555555555555555ull);
        h2 += mix64(key + value_bits * 0xd6e8feb86659fd93ull);
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        h0 += __shfl_xor_sync(FULL_MASK, h0, offset);
        h1 += __shfl_xor_sync(FULL_MASK, h1, offset);
        h2 += __shfl_xor_sync(FULL_MASK, h2, offset);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(&result[0], h0);
        atomicAdd(&result[1], h1);
        atomicAdd(&result[2], h2);
    }
}

} // namespace

void launch_checksum(
    const unsigned long long* pairs, const int32_t* shifts, const double* distances, int values_float, size_t n, unsigned long long* result,
    cudaStream_t stream
) {
    cudaMemsetAsync(result, 0, 4 * sizeof(unsigned long long), stream);
    if (n != 0) {
        const size_t blocks = std::min<size_t>((n + CTA_THREADS - 1) / CTA_THREADS, 148 * 8);
        checksum_kernel<<<static_cast<unsigned>(blocks), CTA_THREADS, 0, stream>>>(pairs, shifts, distances, values_float, n, result);
    }
}

bool small_front_fits(size_t n_points, const GridPlan& plan) {
    return n_points != 0 && n_points <= SMALL_FRONT_MAX_POINTS && plan.n_cells_total <= SMALL_FRONT_MAX_CELLS;
}

void launch_small_front(
    RealView points, size_t n, const GridPlan& plan, int32_t* cell_of, int32_t* rank, int32_t* shift, int32_t* cell_start,
    SortedPoints sorted, DeviceHeader* header, RealView box, const bool* periodic, bool speculative, const double expected_box[9],
    const bool expected_periodic[3], cudaStream_t stream
) {
    small_front_kernel<<<1, SMALL_FRONT_THREADS, 0, stream>>>(
        points, n, plan, cell_of, rank, shift, cell_start, sorted, header, box, periodic, speculative ? 1 : 0,
        expected_inputs(expected_box, expected_periodic)
    );
}

void launch_scan_units(
    const unsigned long long* counts, unsigned long long* starts, size_t n, void* tmp, unsigned long long* total, cudaStream_t stream
) {
    launch_scan<unsigned long long, unsigned long long>(counts, starts, n, tmp, total, stream);
}

} // namespace vb200
