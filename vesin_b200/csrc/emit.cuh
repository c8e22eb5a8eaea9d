// Coalesced stores of a warp's pairs (shared by the pair kernels of large
// systems and of batches of small ones): lane l holds pair l; indices and
// distances leave as whole vectors per lane, the 12- and 24-byte elements of
// shifts and vectors pass through a per-warp shared-memory buffer so that every
// store instruction covers one contiguous span. The list is written once and
// not read again by the build: the stores carry the streaming hint (.cs), which
// keeps the cell-sorted records, read 14 times each, in L2 (1-2 % on the pair kernel).
#ifndef VESIN_B200_EMIT_CUH
#define VESIN_B200_EMIT_CUH

#include "kernels.cuh"

namespace vb200 {

/// Doubles of shared memory a warp needs for the transposes below.
constexpr int TRANSPOSE_DOUBLES = 192;

/// Write `n_valid` consecutive pairs starting at output element `first`:
/// lane l holds pair l. 12- and 24-byte elements are transposed through
/// shared memory so that every store instruction covers one contiguous span.
__device__ __forceinline__ void store_pairs(
    double* transpose, const PairOutput& out, int lane, unsigned long long first, int n_valid, unsigned long long a,
    unsigned long long b, int s0, int s1, int s2, double d, double vx, double vy, double vz
) {
    if (lane < n_valid) {
        __stcs(reinterpret_cast<ulonglong2*>(out.pairs) + first + lane, make_ulonglong2(a, b));
        if (out.distances != nullptr) {
            if (out.values_float) {
                __stcs(reinterpret_cast<float*>(out.distances) + first + lane, static_cast<float>(d));
            } else {
                __stcs(out.distances + first + lane, d);
            }
        }
    }
    if (out.shifts != nullptr) {
        int* buffer = reinterpret_cast<int*>(transpose);
        buffer[3 * lane + 0] = s0;
        buffer[3 * lane + 1] = s1;
        buffer[3 * lane + 2] = s2;
        __syncwarp();
        int32_t* dst = out.shifts + 3 * first;
#pragma unroll
        for (int k = 0; k < 3; k++) {
            const int w = k * 32 + lane;
            if (w < 3 * n_valid) {
                __stcs(&dst[w], buffer[w]);
            }
        }
        __syncwarp();
    }
    if (out.vectors != nullptr && out.values_float) {
        // fp32 output: rounded once from the fp64 result
        float* buffer = reinterpret_cast<float*>(transpose);
        buffer[3 * lane + 0] = static_cast<float>(vx);
        buffer[3 * lane + 1] = static_cast<float>(vy);
        buffer[3 * lane + 2] = static_cast<float>(vz);
        __syncwarp();
        float* dst = reinterpret_cast<float*>(out.vectors) + 3 * first;
#pragma unroll
        for (int k = 0; k < 3; k++) {
            const int w = k * 32 + lane;
            if (w < 3 * n_valid) {
                __stcs(&dst[w], buffer[w]);
            }
        }
    } else if (out.vectors != nullptr) {
        double* buffer = transpose;
        buffer[3 * lane + 0] = vx;
        buffer[3 * lane + 1] = vy;
        buffer[3 * lane + 2] = vz;
        __syncwarp();
        double* dst = out.vectors + 3 * first;
#pragma unroll
        for (int k = 0; k < 3; k++) {
            const int w = k * 32 + lane;
            if (w < 3 * n_valid) {
                __stcs(&dst[w], buffer[w]);
            }
        }
    }
    __syncwarp();
}

/// Full lists: lane l holds hit l and writes both orientations as the two
/// consecutive elements first + 2 l (i, j, S, d, v) and first + 2 l + 1
/// (j, i, -S, d, -v). `first` is even and the arrays are aligned (checked by
/// the launch wrapper), so a lane stores its 32 bytes of indices and 16 bytes
/// of distances at once, and the 24 + 48 bytes of shifts and vectors leave as
/// 8- and 16-byte pieces of one contiguous span after a pass through shared
/// memory.
///
/// A claim that starts on an odd element (slab-decomposed lists, where some
/// blocks hold one orientation only) is written one element further on, which
/// is even again; the reversed pair of its LAST hit then does not fit behind
/// the block and goes to the block's first element instead. `tail_lane` is the
/// lane that holds that hit in this chunk (-1: none), `tail_to` the element.
__device__ __forceinline__ void store_both(
    double* transpose, const PairOutput& out, int lane, unsigned long long first, int n_valid, unsigned long long a,
    unsigned long long b, int s0, int s1, int s2, double d, double vx, double vy, double vz, int tail_lane = -1,
    unsigned long long tail_to = 0
) {
    const unsigned long long mine = first + 2 * lane;
    const bool is_tail = lane == tail_lane;
    if (lane < n_valid && !is_tail) {
        unsigned long long* dst = out.pairs + 2 * mine;
        asm volatile("st.global.cs.v4.b64 [%0], {%1, %2, %3, %4};" ::"l"(dst), "l"(a), "l"(b), "l"(b), "l"(a) : "memory");
        if (out.distances != nullptr) {
            if (out.values_float) {
                const float df = static_cast<float>(d);
                __stcs(reinterpret_cast<float2*>(reinterpret_cast<float*>(out.distances) + mine), make_float2(df, df));
            } else {
                __stcs(reinterpret_cast<double2*>(out.distances + mine), make_double2(d, d));
            }
        }
    }
    if (is_tail) {
        // forward pair in place, reversed pair at the head of the block, element by element
        reinterpret_cast<ulonglong2*>(out.pairs)[mine] = make_ulonglong2(a, b);
        reinterpret_cast<ulonglong2*>(out.pairs)[tail_to] = make_ulonglong2(b, a);
        if (out.distances != nullptr) {
            if (out.values_float) {
                reinterpret_cast<float*>(out.distances)[mine] = static_cast<float>(d);
                reinterpret_cast<float*>(out.distances)[tail_to] = static_cast<float>(d);
            } else {
                out.distances[mine] = d;
                out.distances[tail_to] = d;
            }
        }
        if (out.shifts != nullptr) {
            out.shifts[3 * tail_to + 0] = -s0;
            out.shifts[3 * tail_to + 1] = -s1;
            out.shifts[3 * tail_to + 2] = -s2;
        }
        if (out.vectors != nullptr) {
            if (out.values_float) {
                float* vectors = reinterpret_cast<float*>(out.vectors);
                vectors[3 * tail_to + 0] = -static_cast<float>(vx);
                vectors[3 * tail_to + 1] = -static_cast<float>(vy);
                vectors[3 * tail_to + 2] = -static_cast<float>(vz);
            } else {
                out.vectors[3 * tail_to + 0] = -vx;
                out.vectors[3 * tail_to + 1] = -vy;
                out.vectors[3 * tail_to + 2] = -vz;
            }
        }
    }
    const bool whole = n_valid == 32 && tail_lane < 0; // the usual case: no bounds to check on the way out
    // pieces of the transposed buffers: 3 per lane; of the tail lane's, the second is half
    // forward pair (its first word is written alone) and the third is not written at all
    const int tail_half = (tail_lane >= 0) ? 3 * tail_lane + 1 : -1;
    if (out.shifts != nullptr) {
        int2* buffer = reinterpret_cast<int2*>(transpose);
        buffer[3 * lane + 0] = make_int2(s0, s1);
        buffer[3 * lane + 1] = make_int2(s2, -s0);
        buffer[3 * lane + 2] = make_int2(-s1, -s2);
        __syncwarp();
        int2* dst = reinterpret_cast<int2*>(out.shifts + 3 * first) + lane;
        if (whole) {
            __stcs(&dst[0], buffer[lane]);
            __stcs(&dst[32], buffer[lane + 32]);
            __stcs(&dst[64], buffer[lane + 64]);
        } else {
#pragma unroll
            for (int k = 0; k < 3; k++) {
                const int piece = k * 32 + lane;
                if (piece < 3 * n_valid && (tail_half < 0 || piece < tail_half)) {
                    __stcs(&dst[k * 32], buffer[piece]);
                } else if (piece == tail_half) {
                    reinterpret_cast<int*>(dst + k * 32)[0] = buffer[piece].x;
                }
            }
        }
        __syncwarp();
    }
    if (out.vectors != nullptr && out.values_float) {
        const float fx = static_cast<float>(vx);
        const float fy = static_cast<float>(vy);
        const float fz = static_cast<float>(vz);
        float2* buffer = reinterpret_cast<float2*>(transpose);
        buffer[3 * lane + 0] = make_float2(fx, fy);
        buffer[3 * lane + 1] = make_float2(fz, -fx);
        buffer[3 * lane + 2] = make_float2(-fy, -fz);
        __syncwarp();
        float2* dst = reinterpret_cast<float2*>(reinterpret_cast<float*>(out.vectors) + 3 * first) + lane;
        if (whole) {
            __stcs(&dst[0], buffer[lane]);
            __stcs(&dst[32], buffer[lane + 32]);
            __stcs(&dst[64], buffer[lane + 64]);
        } else {
#pragma unroll
            for (int k = 0; k < 3; k++) {
                const int piece = k * 32 + lane;
                if (piece < 3 * n_valid && (tail_half < 0 || piece < tail_half)) {
                    __stcs(&dst[k * 32], buffer[piece]);
                } else if (piece == tail_half) {
                    reinterpret_cast<float*>(dst + k * 32)[0] = buffer[piece].x;
                }
            }
        }
        __syncwarp();
    } else if (out.vectors != nullptr) {
        double2* buffer = reinterpret_cast<double2*>(transpose);
        buffer[3 * lane + 0] = make_double2(vx, vy);
        buffer[3 * lane + 1] = make_double2(vz, -vx);
        buffer[3 * lane + 2] = make_double2(-vy, -vz);
        __syncwarp();
        double2* dst = reinterpret_cast<double2*>(out.vectors + 3 * first) + lane;
        if (whole) {
            __stcs(&dst[0], buffer[lane]);
            __stcs(&dst[32], buffer[lane + 32]);
            __stcs(&dst[64], buffer[lane + 64]);
        } else {
#pragma unroll
            for (int k = 0; k < 3; k++) {
                const int piece = k * 32 + lane;
                if (piece < 3 * n_valid && (tail_half < 0 || piece < tail_half)) {
                    __stcs(&dst[k * 32], buffer[piece]);
                } else if (piece == tail_half) {
                    reinterpret_cast<double*>(dst + k * 32)[0] = buffer[piece].x;
                }
            }
        }
        __syncwarp();
    }
}

} // namespace vb200

#endif
