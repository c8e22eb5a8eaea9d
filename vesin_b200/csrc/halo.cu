// Selection of the points a rank has to send to its two slab neighbours.
//
// A rank owns the points whose wrapped fractional coordinate g along the cut
// direction lies in [lower, upper). The points with g - lower <= reach go to
// the lower neighbour, those with upper - g <= reach to the upper neighbour
// (reach = cutoff / face distance). One pass over the owned points, slots
// handed out by warp-aggregated atomics; the two messages are ready to be
// sent as they are: row 0 carries the number of records, every other row is
// (x, y, z, global index as raw bits). No counterpart in the reference, which
// has no multi-GPU notion.
#include <cstdint>
#include <stdexcept>
#include <string>

#include <cuda_runtime.h>

#include "vesin_b200.h"

namespace {

constexpr unsigned FULL_MASK = 0xffffffffu;

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned mask;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(mask));
    return mask;
}

/// Append one record per set lane to `message`; returns nothing, overflowing
/// records are counted but not stored.
__device__ __forceinline__ void append(
    bool take, double x, double y, double z, long long index, double* message, unsigned long long* counter, unsigned long long capacity
) {
    const unsigned takers = __ballot_sync(FULL_MASK, take);
    if (takers == 0) {
        return;
    }
    const int lane = threadIdx.x & 31;
    const int leader = __ffs(takers) - 1;
    unsigned long long base = 0;
    if (lane == leader) {
        base = atomicAdd(counter, static_cast<unsigned long long>(__popc(takers)));
    }
    base = __shfl_sync(FULL_MASK, base, leader);
    if (take) {
        const unsigned long long slot = base + __popc(takers & lanemask_lt());
        if (slot < capacity) {
            double* row = message + 4 * (slot + 1);
            row[0] = x;
            row[1] = y;
            row[2] = z;
            row[3] = __longlong_as_double(index);
        }
    }
}

__global__ void __launch_bounds__(256) pack_halo_kernel(
    const double* __restrict__ points, const long long* __restrict__ global_index, size_t n, double h0, double h1, double h2, double lower,
    double upper, double reach, double* to_lower, double* to_upper, unsigned long long capacity, unsigned long long* counts
) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    // whole warps stay in the loop together: the appends vote
    const size_t n_rounded = (n + 31) / 32 * 32;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_rounded; i += stride) {
        bool down = false, up = false;
        double x = 0, y = 0, z = 0;
        long long index = 0;
        if (i < n) {
            x = points[3 * i + 0];
            y = points[3 * i + 1];
            z = points[3 * i + 2];
            index = global_index[i];
            const double f = x * h0 + y * h1 + z * h2;
            double g = f - floor(f);
            if (g >= 1.0) {
                g = 0.0;
            }
            down = (g - lower) <= reach;
            up = (upper - g) <= reach;
        }
        append(down, x, y, z, index, to_lower, counts + 0, capacity);
        append(up, x, y, z, index, to_upper, counts + 1, capacity);
    }
}

/// Row 0 of each message: the number of records (as a double; exact below 2^53).
__global__ void finish_halo_kernel(double* to_lower, double* to_upper, const unsigned long long* counts) {
    if (threadIdx.x == 0) {
        to_lower[0] = static_cast<double>(counts[0]);
        to_upper[0] = static_cast<double>(counts[1]);
    }
}

thread_local std::string HALO_ERROR;

} // namespace

extern "C" int vesin_b200_pack_halo(
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
) {
    if (error_message == nullptr) {
        return 1;
    }
    if (inverse_column == nullptr || to_lower == nullptr || to_upper == nullptr || counts == nullptr ||
        (n_points > 0 && (points == nullptr || global_index == nullptr))) {
        *error_message = "vesin_b200_pack_halo: NULL pointer argument";
        return 1;
    }
    // the legacy default stream: ordered with the caller's default-stream work
    cudaStream_t stream = cudaStreamLegacy;
    cudaError_t status = cudaMemsetAsync(counts, 0, 2 * sizeof(uint64_t), stream);
    if (status == cudaSuccess && n_points > 0) {
        size_t blocks = (n_points + 255) / 256;
        if (blocks > 148 * 8) {
            blocks = 148 * 8;
        }
        pack_halo_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            reinterpret_cast<const double*>(points), reinterpret_cast<const long long*>(global_index), n_points, inverse_column[0],
            inverse_column[1], inverse_column[2], lower, upper, reach, to_lower, to_upper, capacity,
            reinterpret_cast<unsigned long long*>(counts)
        );
    }
    if (status == cudaSuccess) {
        finish_halo_kernel<<<1, 32, 0, stream>>>(to_lower, to_upper, reinterpret_cast<const unsigned long long*>(counts));
        status = cudaGetLastError();
    }
    if (status != cudaSuccess) {
        HALO_ERROR = std::string("CUDA error in vesin_b200_pack_halo: ") + cudaGetErrorString(status);
        *error_message = HALO_ERROR.c_str();
        return 1;
    }
    return 0;
}
