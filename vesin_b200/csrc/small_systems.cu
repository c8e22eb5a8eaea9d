// Batches of independent small systems: one CTA per system, all pairs times
// the periodic images that can reach the cutoff, exact fp64 predicate for
// every candidate. Two passes (count, emit) so that every system owns one
// contiguous, exactly sized block of the output.
//
// Replaces, for this use, the per-system loop of the callers
// (python/vesin/vesin/metatomic/_neighbors.py:197-199) and the brute-force
// kernels of the reference (vesin/src/cuda/bruteforce.cu:241-573), which keep
// one image per pair and therefore need cutoff <= half the smallest face
// distance; here the number of images per direction follows from the box.
#include "kernels.cuh"

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
__device__ void make_frame(SystemFrame& frame, const double* box, const bool* periodic, double cutoff) {
    int n_periodic = 0, first = -1, second = -1;
    for (int i = 0; i < 3; i++) {
        for (int j = 0; j < 3; j++) {
            frame.H[i][j] = (box != nullptr) ? box[3 * i + j] : 0.0;
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

struct SmallShared {
    SystemFrame frame;
    unsigned long long counter; // pairs counted (pass 1) / written so far (pass 2)
    unsigned long long warp_sum[SMALL_WARPS];
};

template <bool EMIT>
__global__ void __launch_bounds__(SMALL_THREADS) small_systems_kernel(
    const BatchInput in, unsigned long long* __restrict__ system_count, const unsigned long long* __restrict__ system_start, PairOutput out,
    DeviceHeader* header
) {
    extern __shared__ __align__(16) unsigned char small_smem[];
    SmallShared& sh = *reinterpret_cast<SmallShared*>(small_smem);
    double* px = reinterpret_cast<double*>(small_smem + sizeof(SmallShared));

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    for (unsigned system = blockIdx.x; system < in.n_systems; system += gridDim.x) {
        const unsigned long long begin = in.offsets[system];
        const int n = static_cast<int>(in.offsets[system + 1] - begin);
        double* py = px + n;
        double* pz = py + n;
        __syncthreads(); // previous system done with shared memory
        if (threadIdx.x == 0) {
            make_frame(
                sh.frame, in.boxes ? in.boxes + 9 * static_cast<size_t>(system) : nullptr,
                in.periodic ? in.periodic + 3 * static_cast<size_t>(system) : nullptr, in.cutoff
            );
            sh.counter = 0;
            if (sh.frame.singular && !EMIT) {
                atomicOr(&header->status, STATUS_SINGULAR_BOX);
                atomicMin(&header->mask_cursor, static_cast<unsigned long long>(system)); // first offending system
            }
        }
        for (int k = threadIdx.x; k < n; k += SMALL_THREADS) {
            const double x = in.points[3 * (begin + k) + 0];
            const double y = in.points[3 * (begin + k) + 1];
            const double z = in.points[3 * (begin + k) + 2];
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
                        out.distances[dest] = d;
                    }
                    if (out.vectors) {
                        out.vectors[3 * dest + 0] = vx;
                        out.vectors[3 * dest + 1] = vy;
                        out.vectors[3 * dest + 2] = vz;
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
                            out.distances[dest] = d;
                        }
                        if (out.vectors) {
                            out.vectors[3 * dest + 0] = -vx;
                            out.vectors[3 * dest + 1] = -vy;
                            out.vectors[3 * dest + 2] = -vz;
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

void launch_small_count(const BatchInput& in, size_t max_points, unsigned long long* system_count, DeviceHeader* header, cudaStream_t stream) {
    small_systems_kernel<false><<<small_grid(in.n_systems), SMALL_THREADS, small_shared_bytes(max_points), stream>>>(
        in, system_count, nullptr, PairOutput{nullptr, nullptr, nullptr, nullptr}, header
    );
}

void launch_small_emit(
    const BatchInput& in, size_t max_points, const unsigned long long* system_start, PairOutput out, DeviceHeader* header,
    cudaStream_t stream
) {
    small_systems_kernel<true><<<small_grid(in.n_systems), SMALL_THREADS, small_shared_bytes(max_points), stream>>>(
        in, nullptr, system_start, out, header
    );
}

} // namespace vb200
