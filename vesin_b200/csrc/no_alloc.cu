// An entry point that builds a neighbor list without allocating anything.
//
// Who needs it: code that may not call cudaMalloc at the moment it needs a
// list. A host application that handed all device memory to its own pool at
// start-up has none left for the driver to give out; a simulation loop with a
// hard bound on the latency of a step cannot afford a call that may block on
// the whole device; a plugin running inside a framework that forbids
// allocations outside its allocator is simply not allowed to. vesin_neighbors
// grows its workspace and its output arrays with cudaMalloc whenever a system
// is larger than the last one; this entry point never does: the caller brings
// the output arrays, and the scratch the kernels need (cell histogram, cell
// offsets, the cell-sorted copy of the points, the read-back header) lives in
// one file-scope device array of fixed size that every GPU holds from the
// moment the library is loaded until the process exits.
//
// How it runs: every kernel is launched on the legacy default stream, and the
// host reads a small header back twice with a blocking cudaMemcpy (after the
// pass over the points that finds their extent, and at the end for the number
// of pairs). The call therefore behaves like any synchronous default-stream
// work of the caller.
//
// Consequences of the fixed array, all documented in include/vesin_b200.h:
//   * systems larger than VESIN_B200_NO_ALLOC_MAX_POINTS are refused;
//   * every call re-uses the same memory, which still holds the previous
//     call's data: what has to start at zero is cleared at the start of a call;
//   * two calls that overlap on one GPU would corrupt each other. Calls made
//     through this entry point are serialised by a per-device host lock and
//     run on the legacy default stream, so that can only happen across
//     processes that share nothing anyway (each process has its own array).
//   * the first call on a device looks up the device address of the array
//     (cudaGetSymbolAddress) and opts the kernels into large shared memory;
//     make that first call before any stream capture begins.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>

#include <cuda_runtime.h>

#include "vesin.h"
#include "vesin_b200.h"

#include "kernels.cuh"
#include "plan.hpp"

namespace {

using namespace vb200;

constexpr size_t MAX_POINTS = VESIN_B200_NO_ALLOC_MAX_POINTS;
constexpr size_t MAX_CELLS = VESIN_B200_NO_ALLOC_MAX_POINTS;

constexpr size_t align_up(size_t value) {
    return (value + 255) / 256 * 256;
}

// carve-up of the scratch array (byte offsets, each 256-byte aligned)
constexpr size_t OFF_HEADER = 0;
constexpr size_t OFF_CELL_OF = OFF_HEADER + align_up(sizeof(DeviceHeader));
constexpr size_t OFF_RANK = OFF_CELL_OF + align_up(MAX_POINTS * sizeof(int32_t));
constexpr size_t OFF_SHIFT = OFF_RANK + align_up(MAX_POINTS * sizeof(int32_t));
constexpr size_t OFF_CELL_COUNT = OFF_SHIFT + align_up(MAX_POINTS * 3 * sizeof(int32_t));
constexpr size_t OFF_CELL_START = OFF_CELL_COUNT + align_up(MAX_CELLS * sizeof(int32_t));
constexpr size_t OFF_SORTED_POS = OFF_CELL_START + align_up((MAX_CELLS + 1) * sizeof(int32_t));
constexpr size_t OFF_SORTED_INDEX = OFF_SORTED_POS + align_up(MAX_POINTS * 3 * sizeof(double));
constexpr size_t OFF_SORTED_SHIFT = OFF_SORTED_INDEX + align_up(MAX_POINTS * sizeof(int32_t));
constexpr size_t OFF_SCAN_TMP = OFF_SORTED_SHIFT + align_up(MAX_POINTS * 3 * sizeof(int32_t));
constexpr size_t SCAN_TMP_BYTES = 4096;
constexpr size_t SCRATCH_BYTES = OFF_SCAN_TMP + SCAN_TMP_BYTES;

// The scratch itself: about 2.3 MB per GPU. In host code this name is only a
// handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char NO_ALLOC_SCRATCH[SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
struct DeviceState {
    std::mutex lock;
    unsigned char* scratch = nullptr; // device address of NO_ALLOC_SCRATCH on this device
};
DeviceState DEVICES[MAX_DEVICES];

thread_local std::string NO_ALLOC_ERROR;

void check(cudaError_t status, const char* what) {
    if (status != cudaSuccess) {
        throw std::runtime_error(std::string("CUDA error in ") + what + ": " + cudaGetErrorString(status));
    }
}

double key_to_double(unsigned long long key) {
    unsigned long long bits = (key >> 63) ? (key & 0x7fffffffffffffffull) : ~key;
    double value;
    std::memcpy(&value, &bits, sizeof(value));
    return value;
}

bool on_device(const void* ptr, int device) {
    cudaPointerAttributes attributes;
    if (ptr == nullptr || cudaPointerGetAttributes(&attributes, ptr) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return attributes.type == cudaMemoryTypeDevice && attributes.device == device;
}

size_t build(
    const double* points, size_t n_points, const double* box, const bool* periodic, int device, double cutoff, bool full,
    size_t capacity, PairOutput out
) {
    if (device < 0 || device >= MAX_DEVICES) {
        throw std::runtime_error("device_id is out of range");
    }
    if (n_points > MAX_POINTS) {
        throw std::runtime_error(
            "vesin_b200_neighbors_no_alloc handles at most " + std::to_string(MAX_POINTS) + " points (got " +
            std::to_string(n_points) + "): its scratch memory has a fixed size; use vesin_neighbors for larger systems"
        );
    }
    if (!on_device(points, device) || !on_device(box, device) || !on_device(periodic, device)) {
        throw std::runtime_error("`points`, `box` and `periodic` must be device memory on device_id");
    }
    if (capacity > 0 && !on_device(out.pairs, device)) {
        throw std::runtime_error("`pairs` must be device memory on device_id");
    }

    int previous = -1;
    check(cudaGetDevice(&previous), "cudaGetDevice");
    if (previous != device) {
        check(cudaSetDevice(device), "cudaSetDevice");
    }
    struct Restore {
        int device;
        ~Restore() {
            if (device >= 0) {
                cudaSetDevice(device);
            }
        }
    } restore{previous != device ? previous : -1};

    DeviceState& state = DEVICES[device];
    std::lock_guard<std::mutex> guard(state.lock);
    if (state.scratch == nullptr) {
        // once per device, with that device current
        void* address = nullptr;
        check(cudaGetSymbolAddress(&address, NO_ALLOC_SCRATCH), "cudaGetSymbolAddress(NO_ALLOC_SCRATCH)");
        configure_kernels();
        state.scratch = static_cast<unsigned char*>(address);
    }
    unsigned char* base = state.scratch;
    auto* d_header = reinterpret_cast<DeviceHeader*>(base + OFF_HEADER);
    auto* cell_of = reinterpret_cast<int32_t*>(base + OFF_CELL_OF);
    auto* rank = reinterpret_cast<int32_t*>(base + OFF_RANK);
    auto* shift = reinterpret_cast<int32_t*>(base + OFF_SHIFT);
    auto* cell_count = reinterpret_cast<int32_t*>(base + OFF_CELL_COUNT);
    auto* cell_start = reinterpret_cast<int32_t*>(base + OFF_CELL_START);
    SortedPoints sorted{
        reinterpret_cast<double*>(base + OFF_SORTED_POS),
        reinterpret_cast<int32_t*>(base + OFF_SORTED_INDEX),
        reinterpret_cast<int32_t*>(base + OFF_SORTED_SHIFT),
    };
    void* scan_tmp = base + OFF_SCAN_TMP;
    cudaStream_t stream = nullptr; // legacy default stream

    // the header (cursor, status, bounds) is re-initialised by a kernel
    launch_header_init(d_header, RealView{box, 0}, periodic, stream);
    launch_bounds(flat_source(RealView{points, 0}, n_points), d_header, stream);
    check(cudaGetLastError(), "launch");
    DeviceHeader header;
    check(cudaMemcpy(&header, d_header, sizeof(header), cudaMemcpyDeviceToHost), "cudaMemcpy(header)");

    if (header.first_bad != NO_BAD_POINT) {
        throw std::runtime_error("point " + std::to_string(header.first_bad) + " has a non-finite coordinate");
    }
    bool host_periodic[3] = {header.periodic[0] != 0, header.periodic[1] != 0, header.periodic[2] != 0};
    PointBounds bounds{};
    for (int c = 0; c < 3; c++) {
        bounds.min[c] = n_points ? key_to_double(header.min_key[c]) : 0.0;
        bounds.max[c] = n_points ? key_to_double(header.max_key[c]) : 0.0;
    }
    GridPlan plan = make_plan(header.box, host_periodic, bounds, n_points, cutoff, full, /*sorted=*/false, MAX_CELLS);
    if (n_points == 0) {
        return 0;
    }
    if (scan_tmp_bytes(static_cast<size_t>(plan.n_cells_total)) > SCAN_TMP_BYTES) {
        throw std::runtime_error("internal error: scan scratch too small");
    }

    // the histogram is the one array that has to start at zero
    check(cudaMemsetAsync(cell_count, 0, static_cast<size_t>(plan.n_cells_total) * sizeof(int32_t), stream), "cudaMemsetAsync");
    launch_bin(flat_source(RealView{points, 0}, n_points), 0, n_points, plan, cell_of, rank, shift, cell_count, d_header, false, true, stream);
    launch_scan_cells(cell_count, cell_start, static_cast<size_t>(plan.n_cells_total), scan_tmp, stream);
    launch_scatter(
        flat_source(RealView{points, 0}, n_points), cell_of, rank, shift, cell_start, static_cast<size_t>(plan.n_cells_total), sorted, nullptr,
        d_header, stream
    );
    launch_pairs(plan, cell_start, sorted, out, capacity, d_header, stream);
    check(cudaGetLastError(), "launch");
    check(cudaMemcpy(&header, d_header, sizeof(header), cudaMemcpyDeviceToHost), "cudaMemcpy(header)");
    return static_cast<size_t>(header.pair_cursor);
}

} // namespace

extern "C" int vesin_b200_neighbors_no_alloc(
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
) {
    if (error_message == nullptr) {
        return 1;
    }
    if (points == nullptr || box == nullptr || periodic == nullptr || length == nullptr) {
        *error_message = "`points`, `box`, `periodic` and `length` can not be NULL pointers";
        return 1;
    }
    if (!std::isfinite(cutoff) || cutoff <= 1e-6) {
        *error_message = "cutoff must be a finite number larger than 1e-6";
        return 1;
    }
    if (capacity > 0 && pairs == nullptr) {
        *error_message = "`pairs` can not be a NULL pointer when capacity is not zero";
        return 1;
    }
    // a pair of indices is written with one 16-byte store; the other arrays need the alignment of their elements
    if (reinterpret_cast<uintptr_t>(pairs) % 16 != 0 || reinterpret_cast<uintptr_t>(shifts) % 4 != 0 ||
        reinterpret_cast<uintptr_t>(distances) % 8 != 0 || reinterpret_cast<uintptr_t>(vectors) % 8 != 0) {
        *error_message = "`pairs` must be aligned to 16 bytes, `shifts` to 4, `distances` and `vectors` to 8";
        return 1;
    }
    try {
        vb200::PairOutput out{
            reinterpret_cast<unsigned long long*>(pairs),
            reinterpret_cast<int32_t*>(shifts),
            distances,
            reinterpret_cast<double*>(vectors),
        };
        size_t total = build(
            reinterpret_cast<const double*>(points), n_points, reinterpret_cast<const double*>(box), periodic, device_id, cutoff,
            full, capacity, out
        );
        *length = total;
        if (total > capacity) {
            NO_ALLOC_ERROR = "the list has " + std::to_string(total) + " pairs but the output arrays hold " +
                             std::to_string(capacity) + ": call again with larger arrays (nothing usable was written)";
            *error_message = NO_ALLOC_ERROR.c_str();
            return 1;
        }
    } catch (const std::exception& e) {
        NO_ALLOC_ERROR = e.what();
        *error_message = NO_ALLOC_ERROR.c_str();
        return 1;
    }
    return 0;
}
