// Selection of the points a rank has to send to its two slab neighbours.
//
// A rank owns the points whose wrapped fractional coordinate g along the cut
// direction lies in [lower, upper). The points with g - lower <= reach go to
// the lower neighbour, those with upper - g <= reach to the upper neighbour
// (reach = cutoff / face distance). One pass over the owned points, slots
// handed out by warp-aggregated atomics; the two messages are ready to be
// sent as they are: row 0 carries the number of records, every other row is
// (x, y, z, global index as raw bits). The block that finishes last writes the
// two counts into the messages and clears the counters for the next call, so a
// packing is ONE launch. No counterpart in the reference, which has no
// multi-GPU notion.
#include <cstdint>
#include <stdexcept>
#include <string>

#include <cuda_runtime.h>

#include "vesin_b200.h"

#include "halo.cuh"

namespace vb200 {

namespace {

constexpr unsigned FULL_MASK = 0xffffffffu;

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned mask;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(mask));
    return mask;
}

/// Append one record per set lane to `message`; overflowing records are
/// counted but not stored.
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
            // one 32-byte record: two 16-byte stores
            double2* row = reinterpret_cast<double2*>(message + 4 * (slot + 1));
            row[0] = make_double2(x, y);
            row[1] = make_double2(z, __longlong_as_double(index));
        }
    }
}

__global__ void __launch_bounds__(256) pack_halo_kernel(
    const RealView points, const long long* __restrict__ global_index, size_t n, double h0, double h1, double h2, double lower,
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
            if (points.is_float) {
                const float* p = static_cast<const float*>(points.data) + 3 * i;
                x = p[0];
                y = p[1];
                z = p[2];
            } else {
                const double* p = static_cast<const double*>(points.data) + 3 * i;
                x = p[0];
                y = p[1];
                z = p[2];
            }
            index = (global_index != nullptr) ? global_index[i] : static_cast<long long>(i);
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

    // the block that arrives last knows that every record is counted: it fills row 0 of
    // both messages (the count as a double; exact below 2^53) and clears the counters
    __shared__ bool is_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned long long ticket = atomicAdd(counts + 2, 1ull);
        is_last = ticket + 1 == gridDim.x;
    }
    __syncthreads();
    if (is_last && threadIdx.x == 0) {
        __threadfence();
        const unsigned long long n_lower = atomicExch(counts + 0, 0ull);
        const unsigned long long n_upper = atomicExch(counts + 1, 0ull);
        to_lower[0] = static_cast<double>(n_lower);
        to_upper[0] = static_cast<double>(n_upper);
        counts[2] = 0ull;
    }
}

thread_local std::string HALO_ERROR;

} // namespace

void launch_pack_halo(
    RealView points, const long long* global_index, size_t n_points, const double inverse_column[3], double lower, double upper,
    double reach, double* to_lower, double* to_upper, size_t capacity, unsigned long long* counts, cudaStream_t stream
) {
    size_t blocks = (n_points + 255) / 256;
    if (blocks > 148 * 8) {
        blocks = 148 * 8;
    }
    if (blocks == 0) {
        blocks = 1;
    }
    pack_halo_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        points, global_index, n_points, inverse_column[0], inverse_column[1], inverse_column[2], lower, upper, reach, to_lower, to_upper,
        capacity, counts
    );
}

} // namespace vb200

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
    using vb200::HALO_ERROR;
    if (error_message == nullptr) {
        return 1;
    }
    if (inverse_column == nullptr || to_lower == nullptr || to_upper == nullptr || counts == nullptr ||
        (n_points > 0 && (points == nullptr || global_index == nullptr))) {
        *error_message = "vesin_b200_pack_halo: NULL pointer argument";
        return 1;
    }
    // every array must be device memory of ONE device: the kernel runs there, whatever device is current
    int device = -1;
    const void* arrays[5] = {to_lower, to_upper, counts, n_points > 0 ? static_cast<const void*>(points) : nullptr, n_points > 0 ? global_index : nullptr};
    for (const void* pointer : arrays) {
        if (pointer == nullptr) {
            continue;
        }
        cudaPointerAttributes attributes;
        if (cudaPointerGetAttributes(&attributes, pointer) != cudaSuccess || attributes.type != cudaMemoryTypeDevice) {
            cudaGetLastError();
            *error_message = "vesin_b200_pack_halo: every array must be device memory";
            return 1;
        }
        if (device >= 0 && attributes.device != device) {
            *error_message = "vesin_b200_pack_halo: the arrays do not live on the same device";
            return 1;
        }
        device = attributes.device;
    }
    int previous = -1;
    cudaError_t status = cudaGetDevice(&previous);
    if (status == cudaSuccess && previous != device) {
        status = cudaSetDevice(device);
    }
    if (status == cudaSuccess) {
        // the legacy default stream: ordered with the caller's default-stream work
        cudaStream_t stream = cudaStreamLegacy;
        status = cudaMemsetAsync(counts, 0, 3 * sizeof(uint64_t), stream);
        if (status == cudaSuccess) {
            vb200::launch_pack_halo(
                vb200::RealView{points, 0}, reinterpret_cast<const long long*>(global_index), n_points, inverse_column, lower, upper, reach,
                to_lower, to_upper, capacity, reinterpret_cast<unsigned long long*>(counts), stream
            );
            status = cudaGetLastError();
        }
    }
    if (previous >= 0 && previous != device) {
        cudaSetDevice(previous);
    }
    if (status != cudaSuccess) {
        HALO_ERROR = std::string("CUDA error in vesin_b200_pack_halo: ") + cudaGetErrorString(status);
        *error_message = HALO_ERROR.c_str();
        return 1;
    }
    return 0;
}
