// Batches of independent small systems. Two passes (count, emit) so that every
// system owns one contiguous, exactly sized block of the output. Two kernels:
//   * molecules (no periodic direction, at most 96 points): a WARP per system,
//     eight systems per CTA; lanes take the pairs i < j of the flattened upper
//     triangle, decide them with an fp32 screen (coordinates relative to the
//     first point) and the exact fp64 predicate inside the error band, gather
//     the hits in a per-warp list and write them 32 at a time through the
//     coalesced stores of the large-system kernels;
//   * everything else (periodic systems, up to 2048 points): a CTA per system,
//     all pairs times the periodic images that can reach the cutoff, exact fp64
//     predicate for every candidate.
//
// Replaces, for this use, the per-system loop of the callers
// (python/vesin/vesin/metatomic/_neighbors.py:197-199) and the brute-force
// kernels of the reference (vesin/src/cuda/bruteforce.cu:241-573), which keep
// one image per pair and therefore need cutoff <= half the smallest face
// distance; here the number of images per direction follows from the box.
#include "kernels.cuh"

#include "emit.cuh"
#include "plan.hpp"

#include <cfloat>

namespace vb200 {

namespace {

constexpr int SMALL_THREADS = 128;
constexpr int SMALL_WARPS = SMALL_THREADS / 32;
constexpr unsigned FULL_MASK = 0xffffffffu;

struct SystemFrame {
    double H[3][3];    // box, rows of non-periodic directions replaced by unit vectors
    double Hinv[3][3];
    int periodic[3];
    int reach[3];      // images to try on each side of the nearest one
    int singular;
};

__device__ __forceinline__ void cross3(const double a[3], const double b[3], double out[3]) {
    out[0] = a[1] * b[2] - a[2] * b[1];
    out[1] = a[2] * b[0] - a[0] * b[2];
    out[2] = a[0] * b[1] - a[1] * b[0];
}

__device__ __forceinline__ void unit3(double v[3]) {
    double inv = 1.0 / sqrt(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]);
    v[0] *= inv;
    v[1] *= inv;
    v[2] *= inv;
}

/// Same normalisation of the box as the host plan (and as the reference CPU
/// path, vesin/src/types.hpp:41-97): rows of non-periodic directions become
/// unit vectors orthogonal to the periodic ones.
__device__ void make_frame(SystemFrame& frame, const BatchInput& in, unsigned system, const bool* periodic, double cutoff) {
    int n_periodic = 0, first = -1, second = -1;
    for (int i = 0; i < 3; i++) {
        for (int j = 0; j < 3; j++) {
            const size_t k = 9 * static_cast<size_t>(system) + 3 * i + j;
            frame.H[i][j] = (in.boxes == nullptr) ? 0.0 : (in.is_float ? static_cast<double>(static_cast<const float*>(in.boxes)[k]) : static_cast<const double*>(in.boxes)[k]);
        }
        frame.periodic[i] = (periodic != nullptr && periodic[i]) ? 1 : 0;
        if (frame.periodic[i]) {
            n_periodic++;
            if (first < 0) {
                first = i;
            } else if (second < 0) {
                second = i;
            }
        }
    }
    if (n_periodic == 0) {
        for (int i = 0; i < 3; i++) {
            for (int j = 0; j < 3; j++) {
                frame.H[i][j] = (i == j) ? 1.0 : 0.0;
            }
        }
    } else if (n_periodic == 1) {
        double a[3] = {frame.H[first][0], frame.H[first][1], frame.H[first][2]};
        double an[3] = {a[0], a[1], a[2]};
        unit3(an);
        double helper[3] = {0, 1, 0};
        if (fabs(an[1]) > 0.9) {
            helper[1] = 0;
            helper[2] = 1;
        }
        double c[3], b[3];
        cross3(a, helper, c);
        unit3(c);
        cross3(c, a, b);
        unit3(b);
        for (int k = 0; k < 3; k++) {
            frame.H[(first + 1) % 3][k] = b[k];
            frame.H[(first + 2) % 3][k] = c[k];
        }
    } else if (n_periodic == 2) {
        double c[3];
        cross3(frame.H[first], frame.H[second], c);
        unit3(c);
        for (int k = 0; k < 3; k++) {
            frame.H[3 - first - second][k] = c[k];
        }
    }
    const double (*m)[3] = frame.H;
    double det = m[0][0] * (m[1][1] * m[2][2] - m[2][1] * m[1][2]) - m[0][1] * (m[1][0] * m[2][2] - m[1][2] * m[2][0]) +
                 m[0][2] * (m[1][0] * m[2][1] - m[1][1] * m[2][0]);
    frame.singular = !(fabs(det) >= 1e-30);
    if (frame.singular) {
        return;
    }
    double (*inv)[3] = frame.Hinv;
    inv[0][0] = (m[1][1] * m[2][2] - m[2][1] * m[1][2]) / det;
    inv[0][1] = (m[0][2] * m[2][1] - m[0][1] * m[2][2]) / det;
    inv[0][2] = (m[0][1] * m[1][2] - m[0][2] * m[1][1]) / det;
    inv[1][0] = (m[1][2] * m[2][0] - m[1][0] * m[2][2]) / det;
    inv[1][1] = (m[0][0] * m[2][2] - m[0][2] * m[2][0]) / det;
    inv[1][2] = (m[1][0] * m[0][2] - m[0][0] * m[1][2]) / det;
    inv[2][0] = (m[1][0] * m[2][1] - m[2][0] * m[1][1]) / det;
    inv[2][1] = (m[2][0] * m[0][1] - m[0][0] * m[2][1]) / det;
    inv[2][2] = (m[0][0] * m[1][1] - m[1][0] * m[0][1]) / det;
    for (int k = 0; k < 3; k++) {
        frame.reach[k] = 0;
        if (frame.periodic[k]) {
            // |fractional distance + image| * face distance <= |v| < cutoff, and the
            // nearest image leaves at most half a cell: images within cutoff / d + 1/2
            double inv_face = sqrt(inv[0][k] * inv[0][k] + inv[1][k] * inv[1][k] + inv[2][k] * inv[2][k]);
            double reach = floor(cutoff * inv_face * (1.0 + 1e-9) + 0.5 + 1e-9);
            frame.reach[k] = static_cast<int>(fmin(reach, 1.0e6));
        }
    }
    // images per pair: beyond the limit the system is refused (2: "cutoff too large for the box")
    const double images = (2.0 * frame.reach[0] + 1.0) * (2.0 * frame.reach[1] + 1.0) * (2.0 * frame.reach[2] + 1.0);
    if (images > static_cast<double>(MAX_STENCIL_CELLS)) {
        frame.singular = 2;
    }
}

__device__ __forceinline__ bool half_rule_small(int s0, int s1, int s2) {
    // vesin/src/cpu_cell_list.cpp:107-132
    int sum = s0 + s1 + s2;
    if (sum < 0) {
        return false;
    }
    if (sum == 0 && (s2 < 0 || (s2 == 0 && s1 < 0))) {
        return false;
    }
    return true;
}

constexpr int MOLECULE_MAX_POINTS = 96;  // largest system the warp-per-system kernel takes
constexpr int MOLECULE_WARPS = 8;

__device__ __forceinline__ double batch_coordinate(const BatchInput& in, size_t k) {
    // float -> double is exact: fp32 inputs are decided with the same fp64 arithmetic
    return in.is_float ? static_cast<double>(static_cast<const float*>(in.points)[k]) : static_cast<const double*>(in.points)[k];
}

/// Systems without a periodic direction and with few points go to the
/// warp-per-system kernel.
__device__ __forceinline__ bool taken_by_warp_kernel(const BatchInput& in, unsigned system, int n) {
    if (n > MOLECULE_MAX_POINTS) {
        return false;
    }
    if (in.periodic == nullptr) {
        return true;
    }
    const bool* periodic = in.periodic + 3 * static_cast<size_t>(system);
    return !(periodic[0] || periodic[1] || periodic[2]);
}

struct MoleculeShared {
    double x[MOLECULE_WARPS][MOLECULE_MAX_POINTS]; // original positions
    double y[MOLECULE_WARPS][MOLECULE_MAX_POINTS];
    double z[MOLECULE_WARPS][MOLECULE_MAX_POINTS];
    float fx[MOLECULE_WARPS][MOLECULE_MAX_POINTS]; // relative to the first point of the system
    float fy[MOLECULE_WARPS][MOLECULE_MAX_POINTS];
    float fz[MOLECULE_WARPS][MOLECULE_MAX_POINTS];
    alignas(16) double transpose[MOLECULE_WARPS][TRANSPOSE_DOUBLES];
    unsigned short list[MOLECULE_WARPS][64]; // hits waiting to be written: (i << 8) | j
};

/// Row i of the strict upper triangle of an n x n matrix starts at this
/// position of the flattened triangle.
__device__ __forceinline__ int triangle_row_start(int i, int n) {
    return (i * (2 * n - i - 1)) >> 1;
}

/// Writes `n_valid` hits of the warp's list (lane l takes entry l) at element
/// `first` of the output: both orientations side by side for full lists.
__device__ __forceinline__ void write_molecule_hits(
    MoleculeShared& sh, const BatchInput& in, const PairOutput& out, int warp, int lane, unsigned long long first, int n_valid,
    unsigned long long index_offset
) {
    int i = 0, j = 0;
    if (lane < n_valid) {
        const unsigned entry = sh.list[warp][lane];
        i = entry >> 8;
        j = entry & 255;
    }
    // the reference's arithmetic for S = 0 (vesin/src/cpu_cell_list.cpp:135-138): the shift term is an exact zero
    const double vx = __dadd_rn(__dsub_rn(sh.x[warp][j], sh.x[warp][i]), 0.0);
    const double vy = __dadd_rn(__dsub_rn(sh.y[warp][j], sh.y[warp][i]), 0.0);
    const double vz = __dadd_rn(__dsub_rn(sh.z[warp][j], sh.z[warp][i]), 0.0);
    const double d = __dsqrt_rn(__dadd_rn(__dadd_rn(__dmul_rn(vx, vx), __dmul_rn(vy, vy)), __dmul_rn(vz, vz)));
    const unsigned long long gi = index_offset + i;
    const unsigned long long gj = index_offset + j;
    if (in.full) {
        if (out.interleave_ok) {
            store_both(sh.transpose[warp], out, lane, first, n_valid, gi, gj, 0, 0, 0, d, vx, vy, vz);
        } else {
            store_pairs(sh.transpose[warp], out, lane, first, n_valid, gi, gj, 0, 0, 0, d, vx, vy, vz);
            store_pairs(sh.transpose[warp], out, lane, first + n_valid, n_valid, gj, gi, 0, 0, 0, d, -vx, -vy, -vz);
        }
    } else {
        store_pairs(sh.transpose[warp], out, lane, first, n_valid, gi, gj, 0, 0, 0, d, vx, vy, vz);
    }
}

template <bool EMIT>
__global__ void __launch_bounds__(MOLECULE_WARPS * 32) molecules_kernel(
    const BatchInput in, unsigned long long* __restrict__ system_count, const unsigned long long* __restrict__ system_start, PairOutput out,
    DeviceHeader* header, const unsigned long long capacity
) {
    __shared__ MoleculeShared sh;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const unsigned warps_in_grid = gridDim.x * MOLECULE_WARPS;

    for (unsigned system = blockIdx.x * MOLECULE_WARPS + warp; system < in.n_systems; system += warps_in_grid) {
        const unsigned long long begin = in.offsets[system];
        const int n = static_cast<int>(in.offsets[system + 1] - begin);
        if (!taken_by_warp_kernel(in, system, n)) {
            continue;
        }
        if (EMIT && system_start[system + 1] > capacity) {
            continue; // written before the host knew the total: the arrays are too short, the host will grow them
        }
        __syncwarp();
        // ---- the system's points: originals for the exact arithmetic, fp32 copies relative to the
        //      first point for the screen; M bounds the relative coordinates ----
        const double ox = (n > 0) ? batch_coordinate(in, 3 * begin + 0) : 0.0;
        const double oy = (n > 0) ? batch_coordinate(in, 3 * begin + 1) : 0.0;
        const double oz = (n > 0) ? batch_coordinate(in, 3 * begin + 2) : 0.0;
        float reach = 0.0f;
        for (int k = lane; k < n; k += 32) {
            const double x = batch_coordinate(in, 3 * (begin + k) + 0);
            const double y = batch_coordinate(in, 3 * (begin + k) + 1);
            const double z = batch_coordinate(in, 3 * (begin + k) + 2);
            sh.x[warp][k] = x;
            sh.y[warp][k] = y;
            sh.z[warp][k] = z;
            const float fx = static_cast<float>(x - ox);
            const float fy = static_cast<float>(y - oy);
            const float fz = static_cast<float>(z - oz);
            sh.fx[warp][k] = fx;
            sh.fy[warp][k] = fy;
            sh.fz[warp][k] = fz;
            reach = fmaxf(reach, fmaxf(fabsf(fx), fmaxf(fabsf(fy), fabsf(fz))));
            if (!EMIT && !(isfinite(x) && isfinite(y) && isfinite(z))) {
                atomicOr(&header->status, STATUS_BAD_POINT);
                atomicMin(&header->first_bad, begin + k);
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            reach = fmaxf(reach, __shfl_xor_sync(FULL_MASK, reach, offset));
        }
        __syncwarp();
        // fp32 screen: candidates whose squared distance is outside [lo, hi] are decided, the
        // others go to the exact predicate. The band covers the rounding of the coordinates
        // (relative error 2^-24 of values up to M), of the differences and of the sum.
        const float m = reach * 1.7320508f * 1.0001f + 1.0e-30f; // bound on the length of a relative position
        const float c = static_cast<float>(in.cutoff) * 1.01f;
        const float eps = 5.9604644775390625e-08f;
        float band = 4.0f * eps * (2.0f * 1.7320508f * c * (2.0f * m + c) + 3.0f * c * c) + 40.0f * eps * m * m + 4.0f * eps * c * c;
        band *= 1.01f; // this expression is itself evaluated in fp32
        const float cutoff2 = static_cast<float>(in.cutoff2);
        const float lo = cutoff2 - band;
        const float hi = cutoff2 + band;

        const unsigned long long base = EMIT ? system_start[system] : 0ull;
        const unsigned long long index_offset = in.global_indices ? begin : 0ull;
        const unsigned per_hit = in.full ? 2u : 1u;
        unsigned long long written = 0; // output elements of the system written so far
        int listed = 0;                 // hits waiting in the list (the same value in every lane)
        unsigned hits_total = 0;

        const int n_candidates = (n * (n - 1)) >> 1;
        for (int c0 = 0; c0 < n_candidates; c0 += 32) {
            const int candidate = c0 + lane;
            bool hit = false;
            int i = 0, j = 0;
            if (candidate < n_candidates) {
                // (i, j) from the position in the flattened strict upper triangle
                const float b = static_cast<float>(2 * n - 1);
                i = static_cast<int>(0.5f * (b - sqrtf(b * b - 8.0f * static_cast<float>(candidate))));
                i = min(max(i, 0), n - 2);
                while (triangle_row_start(i + 1, n) <= candidate) {
                    i++;
                }
                while (triangle_row_start(i, n) > candidate) {
                    i--;
                }
                j = i + 1 + (candidate - triangle_row_start(i, n));
                const float dx = sh.fx[warp][j] - sh.fx[warp][i];
                const float dy = sh.fy[warp][j] - sh.fy[warp][i];
                const float dz = sh.fz[warp][j] - sh.fz[warp][i];
                const float d2 = dx * dx + dy * dy + dz * dz;
                if (d2 < lo) {
                    hit = true;
                } else if (d2 <= hi || !(d2 == d2)) {
                    // the reference's arithmetic, operation for operation (vesin/src/cpu_cell_list.cpp:135-138)
                    const double vx = __dadd_rn(__dsub_rn(sh.x[warp][j], sh.x[warp][i]), 0.0);
                    const double vy = __dadd_rn(__dsub_rn(sh.y[warp][j], sh.y[warp][i]), 0.0);
                    const double vz = __dadd_rn(__dsub_rn(sh.z[warp][j], sh.z[warp][i]), 0.0);
                    hit = __dadd_rn(__dadd_rn(__dmul_rn(vx, vx), __dmul_rn(vy, vy)), __dmul_rn(vz, vz)) < in.cutoff2;
                }
            }
            const unsigned ballot = __ballot_sync(FULL_MASK, hit);
            if (ballot == 0) {
                continue;
            }
            const int hits = __popc(ballot);
            hits_total += hits;
            if (!EMIT) {
                continue;
            }
            if (hit) {
                sh.list[warp][listed + __popc(ballot & ((1u << lane) - 1u))] = static_cast<unsigned short>((i << 8) | j);
            }
            listed += hits;
            __syncwarp();
            if (listed >= 32) {
                write_molecule_hits(sh, in, out, warp, lane, base + written, 32, index_offset);
                written += 32ull * per_hit;
                listed -= 32;
                // what is left moves to the front of the list
                unsigned short moved = 0;
                if (lane < listed) {
                    moved = sh.list[warp][32 + lane];
                }
                __syncwarp();
                if (lane < listed) {
                    sh.list[warp][lane] = moved;
                }
                __syncwarp();
            }
        }
        if (EMIT) {
            if (listed > 0) {
                write_molecule_hits(sh, in, out, warp, lane, base + written, listed, index_offset);
            }
        } else if (lane == 0) {
            system_count[system] = static_cast<unsigned long long>(hits_total) * per_hit;
        }
    }
}

struct SmallShared {
    SystemFrame frame;
    unsigned long long counter; // pairs counted (pass 1) / written so far (pass 2)
    unsigned long long warp_sum[SMALL_WARPS];
};

template <bool EMIT>
__global__ void __launch_bounds__(SMALL_THREADS) small_systems_kernel(
    const BatchInput in, unsigned long long* __restrict__ system_count, const unsigned long long* __restrict__ system_start, PairOutput out,
    DeviceHeader* header, const unsigned long long capacity
) {
    extern __shared__ __align__(16) unsigned char small_smem[];
    SmallShared& sh = *reinterpret_cast<SmallShared*>(small_smem);
    double* px = reinterpret_cast<double*>(small_smem + sizeof(SmallShared));

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    for (unsigned system = blockIdx.x; system < in.n_systems; system += gridDim.x) {
        const unsigned long long begin = in.offsets[system];
        const int n = static_cast<int>(in.offsets[system + 1] - begin);
        if (taken_by_warp_kernel(in, system, n)) {
            continue;
        }
        if (EMIT && system_start[system + 1] > capacity) {
            continue; // as in the warp kernel
        }
        double* py = px + n;
        double* pz = py + n;
        __syncthreads(); // previous system done with shared memory
        if (threadIdx.x == 0) {
            make_frame(sh.frame, in, system, in.periodic ? in.periodic + 3 * static_cast<size_t>(system) : nullptr, in.cutoff);
            sh.counter = 0;
            if (sh.frame.singular && !EMIT) {
                atomicOr(&header->status, sh.frame.singular == 2 ? STATUS_STENCIL_TOO_LARGE : STATUS_SINGULAR_BOX);
                atomicMin(&header->mask_cursor, static_cast<unsigned long long>(system)); // first offending system
            }
        }
        for (int k = threadIdx.x; k < n; k += SMALL_THREADS) {
            const double x = batch_coordinate(in, 3 * (begin + k) + 0);
            const double y = batch_coordinate(in, 3 * (begin + k) + 1);
            const double z = batch_coordinate(in, 3 * (begin + k) + 2);
            px[k] = x;
            py[k] = y;
            pz[k] = z;
            if (!EMIT && !(isfinite(x) && isfinite(y) && isfinite(z))) {
                atomicOr(&header->status, STATUS_BAD_POINT);
                atomicMin(&header->first_bad, begin + k);
            }
        }
        __syncthreads();
        const SystemFrame& frame = sh.frame;
        if (frame.singular) {
            if (!EMIT && threadIdx.x == 0) {
                system_count[system] = 0;
            }
            continue;
        }
        const int w0 = 2 * frame.reach[0] + 1;
        const int w1 = 2 * frame.reach[1] + 1;
        const int w2 = 2 * frame.reach[2] + 1;
        const int n_images = w0 * w1 * w2;
        const unsigned long long base = EMIT ? system_start[system] : 0ull;
        const unsigned long long index_offset = in.global_indices ? begin : 0ull;
        unsigned long long my_count = 0;

        // a warp takes point i; its lanes take (j >= i, image) candidates
        for (int i = warp; i < n; i += SMALL_WARPS) {
            const double rix = px[i], riy = py[i], riz = pz[i];
            const long long n_candidates = static_cast<long long>(n - i) * n_images;
            for (long long c0 = 0; c0 < n_candidates; c0 += 32) {
                const long long c = c0 + lane;
                bool hit = false;
                int s0 = 0, s1 = 0, s2 = 0, j = i;
                double vx = 0, vy = 0, vz = 0, d2 = 0;
                if (c < n_candidates) {
                    j = i + static_cast<int>(c / n_images);
                    const int image = static_cast<int>(c % n_images);
                    const double rjx = px[j], rjy = py[j], rjz = pz[j];
                    const double dx = rjx - rix, dy = rjy - riy, dz = rjz - riz;
                    int nearest[3];
#pragma unroll
                    for (int k = 0; k < 3; k++) {
                        const double fractional = dx * frame.Hinv[0][k] + dy * frame.Hinv[1][k] + dz * frame.Hinv[2][k];
                        nearest[k] = frame.periodic[k] ? -static_cast<int>(rint(fmin(fmax(fractional, -1.0e9), 1.0e9))) : 0;
                    }
                    const int e0 = image % w0 - frame.reach[0];
                    const int e1 = (image / w0) % w1 - frame.reach[1];
                    const int e2 = image / (w0 * w1) - frame.reach[2];
                    s0 = nearest[0] + e0;
                    s1 = nearest[1] + e1;
                    s2 = nearest[2] + e2;
                    // a point with itself: only images, and only one of S / -S
                    // (the other one is written as the reversed pair)
                    bool keep = (j != i) || (((s0 | s1 | s2) != 0) && half_rule_small(s0, s1, s2));
                    if (keep) {
                        const double f0 = static_cast<double>(s0), f1 = static_cast<double>(s1), f2 = static_cast<double>(s2);
                        // the reference's arithmetic, operation for operation
                        // (vesin/src/cpu_cell_list.cpp:135-138, types.hpp:232-243)
                        const double shx = __dadd_rn(__dadd_rn(__dmul_rn(f0, frame.H[0][0]), __dmul_rn(f1, frame.H[1][0])), __dmul_rn(f2, frame.H[2][0]));
                        const double shy = __dadd_rn(__dadd_rn(__dmul_rn(f0, frame.H[0][1]), __dmul_rn(f1, frame.H[1][1])), __dmul_rn(f2, frame.H[2][1]));
                        const double shz = __dadd_rn(__dadd_rn(__dmul_rn(f0, frame.H[0][2]), __dmul_rn(f1, frame.H[1][2])), __dmul_rn(f2, frame.H[2][2]));
                        vx = __dadd_rn(__dsub_rn(rjx, rix), shx);
                        vy = __dadd_rn(__dsub_rn(rjy, riy), shy);
                        vz = __dadd_rn(__dsub_rn(rjz, riz), shz);
                        d2 = __dadd_rn(__dadd_rn(__dmul_rn(vx, vx), __dmul_rn(vy, vy)), __dmul_rn(vz, vz));
                        hit = d2 < in.cutoff2;
                    }
                }
                const unsigned ballot = __ballot_sync(FULL_MASK, hit);
                if (ballot == 0) {
                    continue;
                }
                const unsigned per_hit = in.full ? 2u : 1u;
                if (!EMIT) {
                    if (lane == 0) {
                        my_count += static_cast<unsigned long long>(__popc(ballot)) * per_hit;
                    }
                    continue;
                }
                unsigned long long first = 0;
                if (lane == 0) {
                    first = atomicAdd(&sh.counter, static_cast<unsigned long long>(__popc(ballot)) * per_hit);
                }
                first = __shfl_sync(FULL_MASK, first, 0);
                if (hit) {
                    const unsigned long long rank = __popc(ballot & ((1u << lane) - 1u));
                    unsigned long long dest = base + first + rank * per_hit;
                    const unsigned long long gi = index_offset + i, gj = index_offset + j;
                    const double d = __dsqrt_rn(d2);
                    // half lists keep i <= j (i < j, or the image the rule keeps): the forward pair
                    reinterpret_cast<ulonglong2*>(out.pairs)[dest] = make_ulonglong2(gi, gj);
                    if (out.shifts) {
                        out.shifts[3 * dest + 0] = s0;
                        out.shifts[3 * dest + 1] = s1;
                        out.shifts[3 * dest + 2] = s2;
                    }
                    if (out.distances) {
                        if (out.values_float) {
                            reinterpret_cast<float*>(out.distances)[dest] = static_cast<float>(d);
                        } else {
                            out.distances[dest] = d;
                        }
                    }
                    if (out.vectors) {
                        if (out.values_float) {
                            float* vectors = reinterpret_cast<float*>(out.vectors);
                            vectors[3 * dest + 0] = static_cast<float>(vx);
                            vectors[3 * dest + 1] = static_cast<float>(vy);
                            vectors[3 * dest + 2] = static_cast<float>(vz);
                        } else {
                            out.vectors[3 * dest + 0] = vx;
                            out.vectors[3 * dest + 1] = vy;
                            out.vectors[3 * dest + 2] = vz;
                        }
                    }
                    if (in.full) {
                        dest += 1;
                        reinterpret_cast<ulonglong2*>(out.pairs)[dest] = make_ulonglong2(gj, gi);
                        if (out.shifts) {
                            out.shifts[3 * dest + 0] = -s0;
                            out.shifts[3 * dest + 1] = -s1;
                            out.shifts[3 * dest + 2] = -s2;
                        }
                        if (out.distances) {
                            if (out.values_float) {
                                reinterpret_cast<float*>(out.distances)[dest] = static_cast<float>(d);
                            } else {
                                out.distances[dest] = d;
                            }
                        }
                        if (out.vectors) {
                            if (out.values_float) {
                                float* vectors = reinterpret_cast<float*>(out.vectors);
                                vectors[3 * dest + 0] = -static_cast<float>(vx);
                                vectors[3 * dest + 1] = -static_cast<float>(vy);
                                vectors[3 * dest + 2] = -static_cast<float>(vz);
                            } else {
                                out.vectors[3 * dest + 0] = -vx;
                                out.vectors[3 * dest + 1] = -vy;
                                out.vectors[3 * dest + 2] = -vz;
                            }
                        }
                    }
                }
            }
        }
        if (!EMIT) {
            if (lane == 0) {
                sh.warp_sum[warp] = my_count;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                unsigned long long total = 0;
                for (int w = 0; w < SMALL_WARPS; w++) {
                    total += sh.warp_sum[w];
                }
                system_count[system] = total;
            }
        }
    }
}

} // namespace

size_t small_systems_max_points() {
    return 2048;
}

static size_t small_shared_bytes(size_t max_points) {
    return sizeof(SmallShared) + 3 * max_points * sizeof(double);
}

void configure_small_systems() {
    int bytes = static_cast<int>(small_shared_bytes(small_systems_max_points()));
    cudaFuncSetAttribute(small_systems_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    cudaFuncSetAttribute(small_systems_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

static unsigned small_grid(unsigned n_systems) {
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    }
    unsigned cap = static_cast<unsigned>(sms) * 8;
    return n_systems < cap ? (n_systems ? n_systems : 1) : cap;
}

static unsigned molecules_grid(unsigned n_systems) {
    int device = 0, sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    }
    const unsigned wanted = (n_systems + MOLECULE_WARPS - 1) / MOLECULE_WARPS;
    const unsigned cap = static_cast<unsigned>(sms) * 8;
    return wanted < cap ? (wanted ? wanted : 1) : cap;
}

void launch_small_count(
    const BatchInput& in, size_t max_points, bool any_for_cta_kernel, unsigned long long* system_count, DeviceHeader* header, cudaStream_t stream
) {
    const PairOutput nothing{nullptr, nullptr, nullptr, nullptr, 0, 0};
    molecules_kernel<false><<<molecules_grid(in.n_systems), MOLECULE_WARPS * 32, 0, stream>>>(in, system_count, nullptr, nothing, header, 0ull);
    if (any_for_cta_kernel) {
        small_systems_kernel<false><<<small_grid(in.n_systems), SMALL_THREADS, small_shared_bytes(max_points), stream>>>(
            in, system_count, nullptr, nothing, header, 0ull
        );
    }
}

void launch_small_emit(
    const BatchInput& in, size_t max_points, bool any_for_cta_kernel, const unsigned long long* system_start, PairOutput out,
    DeviceHeader* header, cudaStream_t stream, unsigned long long capacity
) {
    // paired stores of full lists need aligned arrays (every system of a full list starts on an even element)
    const auto aligned = [](const void* pointer, uintptr_t bytes) { return reinterpret_cast<uintptr_t>(pointer) % bytes == 0; };
    const uintptr_t value_bytes = out.values_float ? 8 : 16;
    out.interleave_ok = aligned(out.pairs, 32) && aligned(out.shifts, 8) && aligned(out.distances, value_bytes) && aligned(out.vectors, value_bytes);
    molecules_kernel<true><<<molecules_grid(in.n_systems), MOLECULE_WARPS * 32, 0, stream>>>(in, nullptr, system_start, out, header, capacity);
    if (any_for_cta_kernel) {
        small_systems_kernel<true><<<small_grid(in.n_systems), SMALL_THREADS, small_shared_bytes(max_points), stream>>>(
            in, nullptr, system_start, out, header, capacity
        );
    }
}

size_t molecules_max_points() {
    return MOLECULE_MAX_POINTS;
}

} // namespace vb200
