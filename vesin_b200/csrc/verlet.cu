// Verlet-skin cache on the device.
//
// With `skin > 0` the reference keeps, per list, the candidate pairs found at
// cutoff + skin and re-filters them at the cutoff on every call while no point
// has moved more than skin / 2 since the candidates were built
// (vesin/src/verlet_cuda.cpp:151-322, vesin/src/cuda/verlet.cu:8-91; CPU:
// vesin/src/verlet.cpp:82-191). The result of every call is the exact list at
// `cutoff`; the cache only saves work. Here:
//   * candidates are a HALF list at cutoff + skin (a full list writes both
//     orientations of every kept pair), compacted to 12-byte records: the two
//     points as positions in the cell-sorted order of the build that found them
//     and the three shift components in 10 bits each. Every call copies the
//     current points into that order first (one pass), so that the filter's
//     gathers stay inside a few neighbouring cells and are served by L1,
//     whatever the order of the caller's array;
//   * one kernel checks the displacements of all points against the threshold,
//     which shrinks by half the displacement of the box corners when the box
//     has changed (vesin/src/verlet_cuda.cpp:23-48,166-178), and compares the
//     periodicity flags; it leaves a flag in device memory;
//   * the filter streams over the records, evaluates the reference's exact
//     fp64 arithmetic on the current positions, gathers the kept pairs per
//     CTA and writes them 256 at a time through the coalesced stores of the
//     pair kernels, into ranges claimed from a cursor (one atomic per 256
//     pairs: the cursor is a single word).
//     It does nothing when the check kernel raised the flag, so check and
//     filter are queued back to back and the host reads both results at once.
#include "kernels.cuh"

#include "emit.cuh"

namespace vb200 {

namespace {

constexpr int VERLET_THREADS = 256;
constexpr int VERLET_WARPS = VERLET_THREADS / 32;
constexpr unsigned FULL_MASK = 0xffffffffu;
constexpr int SHIFT_BIAS = 512; // a shift component is stored as value + 512 in 10 bits

__device__ __forceinline__ double load_value(const RealView& view, size_t k) {
    return view.is_float ? static_cast<double>(static_cast<const float*>(view.data)[k]) : static_cast<const double*>(view.data)[k];
}

// ---------------------------------------------------------------------------
// candidates -> records
// ---------------------------------------------------------------------------

/// rank_of[i] = position of point i in the cell-sorted order.
__global__ void __launch_bounds__(VERLET_THREADS) verlet_rank_kernel(const int32_t* __restrict__ sorted_index, size_t n, uint32_t* __restrict__ rank_of) {
    const size_t p = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (p < n) {
        rank_of[sorted_index[p]] = static_cast<uint32_t>(p);
    }
}

__global__ void __launch_bounds__(VERLET_THREADS) verlet_pack_kernel(
    const unsigned long long* __restrict__ pairs, const int32_t* __restrict__ shifts, size_t n, const uint32_t* __restrict__ rank_of,
    uint32_t* __restrict__ records, VerletState* state
) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t r = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; r < n; r += stride) {
        const ulonglong2 ij = reinterpret_cast<const ulonglong2*>(pairs)[r];
        const int s0 = shifts[3 * r + 0];
        const int s1 = shifts[3 * r + 1];
        const int s2 = shifts[3 * r + 2];
        if (s0 < -SHIFT_BIAS || s0 >= SHIFT_BIAS || s1 < -SHIFT_BIAS || s1 >= SHIFT_BIAS || s2 < -SHIFT_BIAS || s2 >= SHIFT_BIAS) {
            state->unpackable = 1; // the host keeps rebuilding lists of this system
        }
        records[3 * r + 0] = rank_of[ij.x];
        records[3 * r + 1] = rank_of[ij.y];
        records[3 * r + 2] = static_cast<uint32_t>(s0 + SHIFT_BIAS) | (static_cast<uint32_t>(s1 + SHIFT_BIAS) << 10) |
                             (static_cast<uint32_t>(s2 + SHIFT_BIAS) << 20);
    }
}

/// The current points in the cell-sorted order of the candidates' build, one
/// 32-byte row per point: x, y, z as doubles and the caller's index of the
/// point (raw bits). The filter fetches a point with ONE 32-byte load; its
/// gathers touch a different cache line per lane, so the number of load
/// instructions is what they cost.
__global__ void __launch_bounds__(VERLET_THREADS) verlet_positions_kernel(
    const RealView points, const int32_t* __restrict__ sorted_index, size_t n, double* __restrict__ positions, const VerletState* state
) {
    if (*reinterpret_cast<const volatile int*>(&state->stale)) {
        return;
    }
    const size_t f = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (f >= 4 * n) {
        return;
    }
    const size_t p = f >> 2;
    const size_t c = f & 3;
    const int32_t index = sorted_index[p];
    positions[f] = (c == 3) ? __longlong_as_double(static_cast<long long>(index)) : load_value(points, 3 * static_cast<size_t>(index) + c);
}

/// One row of `positions` (32-byte aligned): a single 256-bit load.
__device__ __forceinline__ void load_row(const double* __restrict__ positions, uint32_t p, double& x, double& y, double& z, long long& index) {
    long long a, b, c;
    asm("ld.global.v4.b64 {%0, %1, %2, %3}, [%4];" : "=l"(a), "=l"(b), "=l"(c), "=l"(index) : "l"(positions + 4 * static_cast<size_t>(p)));
    x = __longlong_as_double(a);
    y = __longlong_as_double(b);
    z = __longlong_as_double(c);
}

// ---------------------------------------------------------------------------
// are the candidates still good for these points and this box?
// ---------------------------------------------------------------------------

__global__ void __launch_bounds__(VERLET_THREADS) verlet_check_kernel(
    const RealView points, const RealView reference_points, size_t n, const RealView box, const bool* __restrict__ periodic,
    const double* __restrict__ reference_box, const unsigned char* __restrict__ reference_periodic, double skin, VerletState* state
) {
    __shared__ double threshold2;
    __shared__ int stale;
    if (threadIdx.x == 0) {
        // displacement of the corners of the box since the candidates were built: the two largest add up
        double first = 0.0, second = 0.0;
        for (int corner = 0; corner < 8; corner++) {
            const double b0 = (corner & 1) ? 1.0 : 0.0;
            const double b1 = (corner & 2) ? 1.0 : 0.0;
            const double b2 = (corner & 4) ? 1.0 : 0.0;
            double delta = 0.0;
            for (int c = 0; c < 3; c++) {
                const double now = load_value(box, c) * b0 + load_value(box, c + 3) * b1 + load_value(box, c + 6) * b2;
                const double then = reference_box[c] * b0 + reference_box[c + 3] * b1 + reference_box[c + 6] * b2;
                delta += (now - then) * (now - then);
            }
            if (delta > first) {
                second = first;
                first = delta;
            } else if (delta > second) {
                second = delta;
            }
        }
        const double corners = sqrt(first) + sqrt(second);
        bool same_periodicity = true;
        for (int k = 0; k < 3; k++) {
            same_periodicity = same_periodicity && ((periodic[k] ? 1 : 0) == (reference_periodic[k] ? 1 : 0));
        }
        // (a NaN in the box fails the comparison: the build that follows reports it)
        stale = !(corners < skin) || !same_periodicity;
        const double half = 0.5 * (skin - corners);
        threshold2 = half * half;
    }
    __syncthreads();
    if (stale) {
        if (threadIdx.x == 0 && blockIdx.x == 0) {
            state->stale = 1;
        }
        return;
    }
    const double limit = threshold2;
    bool moved = false;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const double dx = load_value(points, 3 * i + 0) - load_value(reference_points, 3 * i + 0);
        const double dy = load_value(points, 3 * i + 1) - load_value(reference_points, 3 * i + 1);
        const double dz = load_value(points, 3 * i + 2) - load_value(reference_points, 3 * i + 2);
        // written so that a non-finite coordinate counts as "moved": the rebuild reports it
        moved = moved || !(dx * dx + dy * dy + dz * dz <= limit);
    }
    if (__any_sync(FULL_MASK, moved) && (threadIdx.x & 31) == 0) {
        state->stale = 1;
    }
}

// ---------------------------------------------------------------------------
// filter
// ---------------------------------------------------------------------------

constexpr int FILTER_CHUNK = VERLET_THREADS; // kept records written per claim: 32 per warp

struct FilterShared {
    alignas(16) double transpose[VERLET_WARPS][TRANSPOSE_DOUBLES];
    uint32_t kept[2 * FILTER_CHUNK][3]; // records waiting to be written
    double H[9];
    int n_kept;
    unsigned long long claim;
};

/// The reference's pair vector and squared distance for a record on the
/// current positions, operation for operation (vesin/src/cpu_cell_list.cpp:135-136,
/// types.hpp:232-243).
__device__ __forceinline__ double record_pair(
    const double* __restrict__ positions, const double* H, uint32_t i, uint32_t j, int s0, int s1, int s2, double& vx, double& vy, double& vz,
    long long& index_i, long long& index_j
) {
    const double f0 = static_cast<double>(s0);
    const double f1 = static_cast<double>(s1);
    const double f2 = static_cast<double>(s2);
    const double shx = __dadd_rn(__dadd_rn(__dmul_rn(f0, H[0]), __dmul_rn(f1, H[3])), __dmul_rn(f2, H[6]));
    const double shy = __dadd_rn(__dadd_rn(__dmul_rn(f0, H[1]), __dmul_rn(f1, H[4])), __dmul_rn(f2, H[7]));
    const double shz = __dadd_rn(__dadd_rn(__dmul_rn(f0, H[2]), __dmul_rn(f1, H[5])), __dmul_rn(f2, H[8]));
    double rix, riy, riz, rjx, rjy, rjz;
    load_row(positions, i, rix, riy, riz, index_i);
    load_row(positions, j, rjx, rjy, rjz, index_j);
    vx = __dadd_rn(__dsub_rn(rjx, rix), shx);
    vy = __dadd_rn(__dsub_rn(rjy, riy), shy);
    vz = __dadd_rn(__dsub_rn(rjz, riz), shz);
    return __dadd_rn(__dadd_rn(__dmul_rn(vx, vx), __dmul_rn(vy, vy)), __dmul_rn(vz, vz));
}

/// The CTA writes the first `n_write` kept records (warp w takes entries
/// 32 w ... 32 w + 31) into one range claimed from the cursor; a range past the
/// capacity is counted only. Called by every thread; ends with a barrier.
template <bool FULL>
__device__ __forceinline__ void write_kept(
    FilterShared& sh, const double* __restrict__ positions, const int32_t* __restrict__ sorted_index, const PairOutput& out,
    unsigned long long capacity, VerletState* state, int n_write
) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const unsigned long long per_hit = FULL ? 2 : 1;
    if (threadIdx.x == 0) {
        // one claim per 256 kept pairs: the cursor is a single word that every CTA adds to
        const unsigned long long wanted = static_cast<unsigned long long>(n_write) * per_hit;
        const unsigned long long first = atomicAdd(&state->pair_cursor, wanted);
        sh.claim = (first + wanted <= capacity) ? first : ~0ull; // past the capacity: the host grows the arrays and filters again
    }
    __syncthreads();
    const unsigned long long claim = sh.claim;
    const int n_valid = min(32, n_write - 32 * warp);
    if (claim != ~0ull && n_valid > 0) {
        uint32_t i = 0, j = 0, packed = (SHIFT_BIAS) | (SHIFT_BIAS << 10) | (SHIFT_BIAS << 20);
        if (lane < n_valid) {
            i = sh.kept[32 * warp + lane][0];
            j = sh.kept[32 * warp + lane][1];
            packed = sh.kept[32 * warp + lane][2];
        }
        const int s0 = static_cast<int>(packed & 1023u) - SHIFT_BIAS;
        const int s1 = static_cast<int>((packed >> 10) & 1023u) - SHIFT_BIAS;
        const int s2 = static_cast<int>((packed >> 20) & 1023u) - SHIFT_BIAS;
        double vx = 0.0, vy = 0.0, vz = 0.0, d = 0.0;
        if (lane < n_valid) {
            long long index_i, index_j; // the caller's indices travel with the positions
            d = __dsqrt_rn(record_pair(positions, sh.H, i, j, s0, s1, s2, vx, vy, vz, index_i, index_j));
            i = static_cast<uint32_t>(index_i);
            j = static_cast<uint32_t>(index_j);
        }
        const unsigned long long first = claim + 32ull * warp * per_hit;
        if (FULL) {
            if (out.interleave_ok) {
                store_both(sh.transpose[warp], out, lane, first, n_valid, i, j, s0, s1, s2, d, vx, vy, vz);
            } else {
                store_pairs(sh.transpose[warp], out, lane, first, n_valid, i, j, s0, s1, s2, d, vx, vy, vz);
                store_pairs(sh.transpose[warp], out, lane, first + n_valid, n_valid, j, i, -s0, -s1, -s2, d, -vx, -vy, -vz);
            }
        } else {
            store_pairs(sh.transpose[warp], out, lane, first, n_valid, i, j, s0, s1, s2, d, vx, vy, vz);
        }
    }
    __syncthreads();
}

template <bool FULL>
__global__ void __launch_bounds__(VERLET_THREADS) verlet_filter_kernel(
    const uint32_t* __restrict__ records, size_t n, const double* __restrict__ positions, const int32_t* __restrict__ sorted_index,
    const RealView box, double cutoff2, PairOutput out, unsigned long long capacity, VerletState* state
) {
    __shared__ FilterShared sh;
    if (*reinterpret_cast<volatile int*>(&state->stale)) {
        return; // the candidates do not fit these inputs any more: the host rebuilds them
    }
    if (threadIdx.x < 9) {
        sh.H[threadIdx.x] = load_value(box, threadIdx.x);
    }
    if (threadIdx.x == 0) {
        sh.n_kept = 0;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;

    // a CTA takes 256 consecutive records per round; the kept ones gather in a list of the CTA
    const size_t n_rounds = (n + VERLET_THREADS - 1) / VERLET_THREADS;
    for (size_t round = blockIdx.x; round < n_rounds; round += gridDim.x) {
        const size_t r = round * VERLET_THREADS + threadIdx.x;
        bool hit = false;
        uint32_t i = 0, j = 0, packed = 0;
        if (r < n) {
            i = records[3 * r + 0];
            j = records[3 * r + 1];
            packed = records[3 * r + 2];
            const int s0 = static_cast<int>(packed & 1023u) - SHIFT_BIAS;
            const int s1 = static_cast<int>((packed >> 10) & 1023u) - SHIFT_BIAS;
            const int s2 = static_cast<int>((packed >> 20) & 1023u) - SHIFT_BIAS;
            double vx, vy, vz;
            long long index_i, index_j;
            hit = record_pair(positions, sh.H, i, j, s0, s1, s2, vx, vy, vz, index_i, index_j) < cutoff2;
        }
        const unsigned ballot = __ballot_sync(FULL_MASK, hit);
        if (ballot != 0) {
            int base = 0;
            if (lane == 0) {
                base = atomicAdd(&sh.n_kept, __popc(ballot));
            }
            base = __shfl_sync(FULL_MASK, base, 0);
            if (hit) {
                const int slot = base + __popc(ballot & ((1u << lane) - 1u));
                sh.kept[slot][0] = i;
                sh.kept[slot][1] = j;
                sh.kept[slot][2] = packed;
            }
        }
        __syncthreads();
        const int n_kept = sh.n_kept; // fewer than 2 * FILTER_CHUNK: below FILTER_CHUNK before this round
        if (n_kept >= FILTER_CHUNK) {
            write_kept<FULL>(sh, positions, sorted_index, out, capacity, state, FILTER_CHUNK);
            // what is left moves to the front of the list
            uint32_t moved[3] = {0, 0, 0};
            const int left = n_kept - FILTER_CHUNK;
            if (static_cast<int>(threadIdx.x) < left) {
                moved[0] = sh.kept[FILTER_CHUNK + threadIdx.x][0];
                moved[1] = sh.kept[FILTER_CHUNK + threadIdx.x][1];
                moved[2] = sh.kept[FILTER_CHUNK + threadIdx.x][2];
            }
            __syncthreads();
            if (static_cast<int>(threadIdx.x) < left) {
                sh.kept[threadIdx.x][0] = moved[0];
                sh.kept[threadIdx.x][1] = moved[1];
                sh.kept[threadIdx.x][2] = moved[2];
            }
            if (threadIdx.x == 0) {
                sh.n_kept = left;
            }
            __syncthreads();
        }
    }
    const int n_kept = sh.n_kept;
    if (n_kept > 0) {
        write_kept<FULL>(sh, positions, sorted_index, out, capacity, state, n_kept);
    }
}

} // namespace

void launch_verlet_pack(
    const unsigned long long* pairs, const int32_t* shifts, size_t n, const int32_t* sorted_index, size_t n_points, uint32_t* rank_of,
    uint32_t* records, VerletState* state, cudaStream_t stream
) {
    if (n_points != 0) {
        const size_t blocks = (n_points + VERLET_THREADS - 1) / VERLET_THREADS;
        verlet_rank_kernel<<<static_cast<unsigned>(blocks), VERLET_THREADS, 0, stream>>>(sorted_index, n_points, rank_of);
    }
    if (n == 0) {
        return;
    }
    const size_t blocks = std::min<size_t>((n + VERLET_THREADS - 1) / VERLET_THREADS, 148 * 16);
    verlet_pack_kernel<<<static_cast<unsigned>(blocks), VERLET_THREADS, 0, stream>>>(pairs, shifts, n, rank_of, records, state);
}

void launch_verlet_positions(
    RealView points, const int32_t* sorted_index, size_t n_points, double* positions, const VerletState* state, cudaStream_t stream
) {
    if (n_points == 0) {
        return;
    }
    const size_t blocks = (4 * n_points + VERLET_THREADS - 1) / VERLET_THREADS;
    verlet_positions_kernel<<<static_cast<unsigned>(blocks), VERLET_THREADS, 0, stream>>>(points, sorted_index, n_points, positions, state);
}

void launch_verlet_check(
    RealView points, RealView reference_points, size_t n, RealView box, const bool* periodic, const double* reference_box,
    const unsigned char* reference_periodic, double skin, VerletState* state, cudaStream_t stream
) {
    const size_t blocks = std::max<size_t>(1, std::min<size_t>((n + VERLET_THREADS - 1) / VERLET_THREADS, 148 * 8));
    verlet_check_kernel<<<static_cast<unsigned>(blocks), VERLET_THREADS, 0, stream>>>(
        points, reference_points, n, box, periodic, reference_box, reference_periodic, skin, state
    );
}

void launch_verlet_filter(
    const uint32_t* records, size_t n, const double* positions, const int32_t* sorted_index, RealView box, double cutoff2, bool full,
    PairOutput out, unsigned long long capacity, VerletState* state, cudaStream_t stream
) {
    if (n == 0) {
        return;
    }
    const auto aligned = [](const void* pointer, uintptr_t bytes) { return reinterpret_cast<uintptr_t>(pointer) % bytes == 0; };
    const uintptr_t value_bytes = out.values_float ? 8 : 16;
    out.interleave_ok = aligned(out.pairs, 32) && aligned(out.shifts, 8) && aligned(out.distances, value_bytes) && aligned(out.vectors, value_bytes);
    // a CTA takes 256 records per round; enough CTAs to fill the GPU, few enough that the
    // partly filled chunks at the end of every CTA's walk stay rare
    const size_t rounds = (n + VERLET_THREADS - 1) / VERLET_THREADS;
    const size_t blocks = std::max<size_t>(1, std::min<size_t>(rounds, 148 * 8));
    if (full) {
        verlet_filter_kernel<true><<<static_cast<unsigned>(blocks), VERLET_THREADS, 0, stream>>>(
            records, n, positions, sorted_index, box, cutoff2, out, capacity, state
        );
    } else {
        verlet_filter_kernel<false><<<static_cast<unsigned>(blocks), VERLET_THREADS, 0, stream>>>(
            records, n, positions, sorted_index, box, cutoff2, out, capacity, state
        );
    }
}

} // namespace vb200
