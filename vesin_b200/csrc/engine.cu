// Host orchestration: workspace (grow-only device scratch + output arrays),
// the launch sequence of one build, and the host decisions between launches.
#include "engine.hpp"

#include <atomic>
#include <chrono>
#include <cerrno>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <utility>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "vesin_b200.h"

#include "kernels.cuh"
#include "plan.hpp"

namespace vb200 {

namespace {

std::atomic<bool> PROFILING{false};

void check(cudaError_t status, const char* what) {
    if (status == cudaSuccess) {
        return;
    }
    if (status == cudaErrorMemoryAllocation) {
        cudaGetLastError(); // clear the sticky-less error
        throw std::bad_alloc();
    }
    throw std::runtime_error(std::string("CUDA error in ") + what + ": " + cudaGetErrorString(status));
}

#define VB200_CUDA(call) ::vb200::check((call), #call)

/// Makes `device` current for the lifetime of the guard.
struct DeviceGuard {
    int previous = -1;
    explicit DeviceGuard(int device) {
        VB200_CUDA(cudaGetDevice(&previous));
        if (previous != device) {
            VB200_CUDA(cudaSetDevice(device));
        } else {
            previous = -1;
        }
    }
    ~DeviceGuard() {
        if (previous >= 0) {
            cudaSetDevice(previous);
        }
    }
};

/// Grow-only device allocation; contents are scratch and are not preserved.
struct DeviceBuffer {
    void* ptr = nullptr;
    size_t bytes = 0;

    void reserve(size_t wanted) {
        if (wanted <= bytes) {
            return;
        }
        release();
        VB200_CUDA(cudaMalloc(&ptr, wanted));
        bytes = wanted;
    }

    void release() {
        if (ptr != nullptr) {
            cudaFree(ptr);
        }
        ptr = nullptr;
        bytes = 0;
    }

    template <typename T>
    T* as() const {
        return static_cast<T*>(ptr);
    }
};

constexpr int N_STAGES = VesinB200StageCount_;

/// Everything a VesinNeighborList owns besides the four output pointers;
/// lives behind VesinNeighborList.opaque. Replaces CudaNeighborListExtras +
/// CellListBuffers (vesin/src/cuda_buffers.cpp:95-136,196-257).
struct Workspace {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::vector<size_t> batch_offsets_host; // what `batch_offsets` holds on the device
    // slab builds: the halo is sorted in, and the units next to it are paired, on a stream of
    // their own while the units that need no halo are paired on `stream`
    cudaStream_t side_stream = nullptr;
    cudaEvent_t owned_sorted = nullptr;
    cudaEvent_t side_done = nullptr;
    DeviceHeader* d_header = nullptr;
    DeviceHeader* h_header = nullptr; // pinned

    DeviceBuffer cell_of, rank, shift, cell_count, cell_start;
    DeviceBuffer sorted_pos, sorted_index, sorted_shift;
    DeviceBuffer masks, unit_mask_base, unit_words, unit_count, unit_start;
    DeviceBuffer row_count, row_start, row_fill, scan_tmp;
    DeviceBuffer batch_offsets; // batches: where each system starts in the points array
    DeviceBuffer sorted_global; // slabs: index of every cell-sorted record in the whole system
    DeviceBuffer checksum;      // 4 words of vesin_b200_list_checksum
    bool values_float = false;  // element type of `distances` / `vectors` of the last build

    // Slab builds: extent of the local points along non-periodic directions as the last build
    // that looked found it (the binning kernel checks every point against it), and the number
    // of local points of the last build (sizes the pencils of the next one).
    struct SlabCache {
        bool bounds_valid = false;
        PointBounds bounds{};
        size_t n_local = 0;
    } slab;

    // output arrays (capacity in pairs); kept allocated when not requested
    DeviceBuffer out_pairs, out_shifts, out_distances, out_vectors;
    // second set of output arrays: where a canonical list is sorted into (the sets swap roles)
    DeviceBuffer alt_pairs, alt_shifts, alt_distances, alt_vectors;

    // What the last build on this list saw, and the plan made from it: the
    // next build starts from this plan without waiting for a read-back.
    struct PlanCache {
        bool valid = false;
        double box[9] = {};
        bool periodic[3] = {};
        size_t n_points = 0;
        double cutoff = 0.0;
        bool full = false;
        bool sorted = false;
        GridPlan plan{};
    } cache;

    // Verlet-skin cache (options.skin > 0): candidates found at cutoff + skin, kept as records,
    // and what they were built for. `candidates` is a list of its own, built like any other.
    struct VerletCache {
        bool valid = false;
        // every call rebuilds: shifts of this system do not fit the records, or filtering the
        // candidates of this system turned out slower than building a list (dense systems)
        bool disabled = false;
        double build_seconds = 0.0; // host time of the last build of candidates
        // Does re-filtering beat a plain build for this list? Settled once by the clock:
        // 0 = time the next filter pass, 1 = a plain build to warm its workspace up,
        // 2 = a plain build that is timed and compared, 3 = settled.
        int trial = 0;
        double filter_seconds = 0.0;
        double cutoff = 0.0;
        double skin = 0.0;
        bool full = false;
        bool float_io = false;
        size_t n_points = 0;
        size_t n_records = 0;
        VesinNeighborList candidates{};
        DeviceBuffer records, reference_points, reference_box, state, rank_of, positions;
        VerletState* h_state = nullptr; // pinned
    } verlet;

    cudaEvent_t events[2 * N_STAGES] = {};
    bool events_created = false;
    bool timed = false;
    double stage_ms[N_STAGES] = {};

    ~Workspace() {
        for (DeviceBuffer* buffer :
             {&cell_of, &rank, &shift, &cell_count, &cell_start, &sorted_pos, &sorted_index, &sorted_shift, &masks, &unit_mask_base,
              &unit_words, &unit_count, &unit_start, &row_count, &row_start, &row_fill, &scan_tmp, &batch_offsets, &sorted_global, &checksum, &out_pairs,
              &out_shifts, &out_distances, &out_vectors, &alt_pairs, &alt_shifts, &alt_distances, &alt_vectors}) {
            buffer->release();
        }
        for (DeviceBuffer* buffer : {&verlet.records, &verlet.reference_points, &verlet.reference_box, &verlet.state, &verlet.rank_of, &verlet.positions}) {
            buffer->release();
        }
        if (verlet.h_state != nullptr) {
            cudaFreeHost(verlet.h_state);
        }
        if (verlet.candidates.opaque != nullptr) {
            free_neighbors(verlet.candidates);
        }
        if (d_header != nullptr) {
            cudaFree(d_header);
        }
        if (h_header != nullptr) {
            cudaFreeHost(h_header);
        }
        if (events_created) {
            for (auto& event : events) {
                cudaEventDestroy(event);
            }
        }
        if (owned_sorted != nullptr) {
            cudaEventDestroy(owned_sorted);
        }
        if (side_done != nullptr) {
            cudaEventDestroy(side_done);
        }
        if (side_stream != nullptr) {
            cudaStreamDestroy(side_stream);
        }
        if (stream != nullptr) {
            cudaStreamDestroy(stream);
        }
    }
};

Workspace& workspace_of(VesinNeighborList& list) {
    if (list.opaque == nullptr) {
        auto* ws = new Workspace();
        list.opaque = ws;
        ws->device = list.device.device_id;
        // A blocking stream: ordered after work the caller queued on the
        // legacy default stream, like the reference (which runs on it).
        VB200_CUDA(cudaStreamCreate(&ws->stream));
        VB200_CUDA(cudaMalloc(reinterpret_cast<void**>(&ws->d_header), sizeof(DeviceHeader)));
        VB200_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&ws->h_header), sizeof(DeviceHeader), cudaHostAllocDefault));
        configure_kernels();
        configure_small_systems();
    }
    return *static_cast<Workspace*>(list.opaque);
}

double key_to_double(unsigned long long key) {
    unsigned long long bits = (key >> 63) ? (key & 0x7fffffffffffffffull) : ~key;
    double value;
    std::memcpy(&value, &bits, sizeof(value));
    return value;
}

struct PointerInfo {
    bool resolved = false;
    bool on_device = false;
    int device = -1;
};

PointerInfo inspect(const void* ptr) {
    PointerInfo info;
    if (ptr == nullptr) {
        return info;
    }
    cudaPointerAttributes attributes;
    if (cudaPointerGetAttributes(&attributes, ptr) != cudaSuccess) {
        cudaGetLastError();
        return info;
    }
    info.resolved = true;
    info.on_device = attributes.type == cudaMemoryTypeDevice;
    info.device = info.on_device ? attributes.device : -1;
    return info;
}

/// Same checks, order and messages as vesin/src/vesin_cuda.cpp:831-854.
void validate_pointers(const void* points, const void* box, const void* periodic, const VesinNeighborList& list) {
    struct Named {
        const void* ptr;
        const char* name;
    };
    PointerInfo infos[3];
    const Named named[3] = {{points, "points"}, {box, "box"}, {periodic, "periodic"}};
    for (int k = 0; k < 3; k++) {
        infos[k] = inspect(named[k].ptr);
        if (!infos[k].resolved) {
            throw std::runtime_error(std::string("failed to resolve attributes for pointer: ") + named[k].name);
        }
        if (!infos[k].on_device) {
            throw std::runtime_error(std::string("`") + named[k].name + "` pointer is not allocated on a CUDA device");
        }
    }
    if (infos[0].device != infos[1].device) {
        throw std::runtime_error("`points` and `box` do not exist on the same device");
    }
    if (infos[0].device != infos[2].device) {
        throw std::runtime_error("`points` and `periodic` do not exist on the same device");
    }
    if (infos[0].device != list.device.device_id) {
        throw std::runtime_error("`points`, `box` and `periodic` device differs from input neighbors device_id");
    }
}

/// The reference sizes its output for max(128, ceil(cutoff^3)) pairs per
/// point (or VESIN_CUDA_MAX_PAIRS_PER_POINT) and fails beyond that
/// (vesin/src/vesin_cuda.cpp:866-886,901-919). This engine sizes the output
/// exactly, but keeps the same limit and message as a check on the total.
size_t max_pairs_per_point(double cutoff) {
    size_t result = std::max<size_t>(128, static_cast<size_t>(std::ceil(std::pow(cutoff, 3))));
    const char* env = std::getenv("VESIN_CUDA_MAX_PAIRS_PER_POINT");
    if (env != nullptr) {
        size_t length = std::strlen(env);
        char* end = nullptr;
        errno = 0;
        long long parsed = std::strtoll(env, &end, 10);
        if (errno != 0 || end != env + length || parsed <= 0) {
            throw std::runtime_error("Invalid value for VESIN_CUDA_MAX_PAIRS_PER_POINT: '" + std::string(env) + "'");
        }
        result = static_cast<size_t>(parsed);
    }
    return result;
}

struct StageTimer {
    Workspace& ws;
    bool enabled;
    StageTimer(Workspace& workspace, bool on): ws(workspace), enabled(on) {
        if (enabled && !ws.events_created) {
            for (auto& event : ws.events) {
                VB200_CUDA(cudaEventCreate(&event));
            }
            ws.events_created = true;
        }
        for (auto& ms : ws.stage_ms) {
            ms = 0.0;
        }
        ws.timed = false;
    }
    void begin(int stage) {
        if (enabled) {
            VB200_CUDA(cudaEventRecord(ws.events[2 * stage], ws.stream));
        }
    }
    void end(int stage) {
        if (enabled) {
            VB200_CUDA(cudaEventRecord(ws.events[2 * stage + 1], ws.stream));
        }
    }
    /// call after a stream synchronisation that covers `stage`
    void collect(int stage) {
        if (enabled) {
            float ms = 0.0f;
            VB200_CUDA(cudaEventElapsedTime(&ms, ws.events[2 * stage], ws.events[2 * stage + 1]));
            ws.stage_ms[stage] += ms;
        }
    }
};

void read_header(Workspace& ws) {
    VB200_CUDA(cudaMemcpyAsync(ws.h_header, ws.d_header, sizeof(DeviceHeader), cudaMemcpyDeviceToHost, ws.stream));
    VB200_CUDA(cudaStreamSynchronize(ws.stream));
}

/// Pairs that fit every output array this call needs, as allocated now.
size_t common_capacity(const Workspace& ws, const VesinOptions& options) {
    size_t capacity = ws.out_pairs.bytes / (2 * sizeof(size_t));
    if (options.return_shifts) {
        capacity = std::min(capacity, ws.out_shifts.bytes / (3 * sizeof(int32_t)));
    }
    if (options.return_distances) {
        capacity = std::min(capacity, ws.out_distances.bytes / sizeof(double));
    }
    if (options.return_vectors) {
        capacity = std::min(capacity, ws.out_vectors.bytes / (3 * sizeof(double)));
    }
    return capacity;
}

void set_outputs(VesinNeighborList& list, Workspace& ws, const VesinOptions& options, size_t capacity) {
    ws.out_pairs.reserve(capacity * 2 * sizeof(size_t));
    list.pairs = reinterpret_cast<size_t(*)[2]>(ws.out_pairs.ptr);
    list.shifts = nullptr;
    list.distances = nullptr;
    list.vectors = nullptr;
    if (options.return_shifts) {
        ws.out_shifts.reserve(capacity * 3 * sizeof(int32_t));
        list.shifts = reinterpret_cast<int32_t(*)[3]>(ws.out_shifts.ptr);
    }
    if (options.return_distances) {
        ws.out_distances.reserve(capacity * sizeof(double));
        list.distances = ws.out_distances.as<double>();
    }
    if (options.return_vectors) {
        ws.out_vectors.reserve(capacity * 3 * sizeof(double));
        list.vectors = reinterpret_cast<double(*)[3]>(ws.out_vectors.ptr);
    }
}

} // namespace

void set_profiling(bool enabled) {
    PROFILING.store(enabled);
}

bool profiling_enabled() {
    return PROFILING.load();
}

bool stage_times(const VesinNeighborList& list, double* stage_ms) {
    if (list.opaque == nullptr || list.device.type != VesinCUDA) {
        return false;
    }
    const auto& ws = *static_cast<const Workspace*>(list.opaque);
    if (!ws.timed) {
        return false;
    }
    for (int k = 0; k < N_STAGES; k++) {
        stage_ms[k] = ws.stage_ms[k];
    }
    return true;
}

namespace {

/// `skin > 0`: the list from cached candidates when they still fit the inputs,
/// else candidates are rebuilt at cutoff + skin first. Either way the result is
/// the exact list at the cutoff (vesin/src/verlet_cuda.cpp:307-322).
void neighbors_with_skin(
    const void* points, size_t n_points, const void* box, const bool periodic[3], VesinOptions options, VesinNeighborList& list,
    bool float_io
) {
    DeviceGuard guard(list.device.device_id);
    Workspace& ws = workspace_of(list);
    auto& cache = ws.verlet;
    ws.values_float = float_io;
    ws.cache.valid = false; // the plain build's plan is not kept up to date by these calls
    cudaStream_t stream = ws.stream;
    StageTimer timer(ws, PROFILING.load());
    const RealView flat_points{points, float_io ? 1 : 0};
    const RealView flat_box{box, float_io ? 1 : 0};
    const size_t pair_limit_per_point = max_pairs_per_point(options.cutoff);
    const size_t value_bytes = float_io ? sizeof(float) : sizeof(double);

    if (cache.h_state == nullptr) {
        VB200_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&cache.h_state), sizeof(VerletState), cudaHostAllocDefault));
        cache.state.reserve(sizeof(VerletState));
        cache.reference_box.reserve(9 * sizeof(double) + 8);
    }
    auto* d_state = cache.state.as<VerletState>();
    const auto read_state = [&]() {
        VB200_CUDA(cudaMemcpyAsync(cache.h_state, d_state, sizeof(VerletState), cudaMemcpyDeviceToHost, stream));
        VB200_CUDA(cudaStreamSynchronize(stream));
    };

    if (cache.disabled) {
        options.skin = 0.0;
        neighbors(points, n_points, box, periodic, options, list, float_io, false);
        return;
    }
    bool usable = cache.valid && cache.cutoff == options.cutoff && cache.skin == options.skin && cache.full == options.full &&
                  cache.float_io == float_io && cache.n_points == n_points;
    if (usable && (cache.trial == 1 || cache.trial == 2)) {
        // the same list by a plain build (the candidates stay as they are)
        const auto plain_started = std::chrono::steady_clock::now();
        VesinOptions plain = options;
        plain.skin = 0.0;
        neighbors(points, n_points, box, periodic, plain, list, float_io, false);
        const double plain_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - plain_started).count();
        if (cache.trial == 2 && plain_seconds < cache.filter_seconds) {
            cache.disabled = true;
            cache.valid = false;
        }
        cache.trial++;
        return;
    }
    std::chrono::steady_clock::time_point filter_started{};
    for (int round = 0;; round++) {
        if (!usable) {
            // ---- candidates: the half list at cutoff + skin, built like any list ----
            cache.valid = false;
            cache.candidates.device = list.device;
            VesinOptions wide = options;
            wide.cutoff = options.cutoff + options.skin;
            wide.skin = 0.0;
            wide.full = false;
            wide.sorted = false;
            wide.return_shifts = true;
            wide.return_distances = false;
            wide.return_vectors = false;
            const auto build_started = std::chrono::steady_clock::now();
            neighbors(points, n_points, box, periodic, wide, cache.candidates, float_io, false);
            cache.build_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - build_started).count();
            cache.n_records = cache.candidates.length;
            cache.records.reserve(std::max<size_t>(cache.n_records, 1) * 3 * sizeof(uint32_t));
            cache.reference_points.reserve(std::max<size_t>(n_points, 1) * 3 * value_bytes);
            VB200_CUDA(cudaMemsetAsync(d_state, 0, sizeof(VerletState), stream));
            // records name the points by their position in the cell-sorted order of this very build
            const auto* built = static_cast<const Workspace*>(cache.candidates.opaque);
            cache.rank_of.reserve(std::max<size_t>(n_points, 1) * sizeof(uint32_t));
            cache.positions.reserve(std::max<size_t>(n_points, 1) * 4 * sizeof(double));
            launch_verlet_pack(
                reinterpret_cast<const unsigned long long*>(cache.candidates.pairs), reinterpret_cast<const int32_t*>(cache.candidates.shifts),
                cache.n_records, built->sorted_index.as<int32_t>(), n_points, cache.rank_of.as<uint32_t>(), cache.records.as<uint32_t>(), d_state,
                stream
            );
            if (timer.enabled && built->timed) {
                for (int k = 0; k < N_STAGES; k++) {
                    ws.stage_ms[k] += built->stage_ms[k]; // the build of the candidates belongs to this call
                }
            }
            VB200_CUDA(cudaMemcpyAsync(cache.reference_points.ptr, points, n_points * 3 * value_bytes, cudaMemcpyDeviceToDevice, stream));
            // box as doubles and the periodicity flags behind it
            if (float_io) {
                float box32[9];
                VB200_CUDA(cudaMemcpy(box32, box, sizeof(box32), cudaMemcpyDeviceToHost));
                double box64[9];
                for (int k = 0; k < 9; k++) {
                    box64[k] = box32[k];
                }
                VB200_CUDA(cudaMemcpyAsync(cache.reference_box.ptr, box64, sizeof(box64), cudaMemcpyHostToDevice, stream));
                VB200_CUDA(cudaStreamSynchronize(stream)); // box64 leaves scope
            } else {
                VB200_CUDA(cudaMemcpyAsync(cache.reference_box.ptr, box, 9 * sizeof(double), cudaMemcpyDeviceToDevice, stream));
            }
            VB200_CUDA(cudaMemcpyAsync(cache.reference_box.as<double>() + 9, periodic, 3, cudaMemcpyDeviceToDevice, stream));
            cache.cutoff = options.cutoff;
            cache.skin = options.skin;
            cache.full = options.full;
            cache.float_io = float_io;
            cache.n_points = n_points;
            cache.valid = true;
        } else {
            filter_started = std::chrono::steady_clock::now();
            timer.begin(VesinB200StageBounds);
            VB200_CUDA(cudaMemsetAsync(d_state, 0, sizeof(VerletState), stream));
            launch_verlet_check(
                flat_points, RealView{cache.reference_points.ptr, float_io ? 1 : 0}, n_points, flat_box, periodic, cache.reference_box.as<double>(),
                reinterpret_cast<const unsigned char*>(cache.reference_box.as<double>() + 9), options.skin, d_state, stream
            );
            timer.end(VesinB200StageBounds);
        }

        // ---- filter: into the arrays of the previous call first; when the pairs do not fit they
        // have still been counted: grow to the exact total and filter again ----
        set_outputs(list, ws, options, std::max<size_t>(common_capacity(ws, options), 256));
        size_t capacity = common_capacity(ws, options);
        bool stale = false;
        for (int attempt = 0;; attempt++) {
            PairOutput out{
                reinterpret_cast<unsigned long long*>(list.pairs),
                reinterpret_cast<int32_t*>(list.shifts),
                list.distances,
                reinterpret_cast<double*>(list.vectors),
                float_io ? 1 : 0,
            };
            const auto* built = static_cast<const Workspace*>(cache.candidates.opaque);
            timer.begin(VesinB200StageEmit);
            if (attempt == 0) {
                launch_verlet_positions(flat_points, built->sorted_index.as<int32_t>(), n_points, cache.positions.as<double>(), d_state, stream);
            }
            launch_verlet_filter(
                cache.records.as<uint32_t>(), cache.n_records, cache.positions.as<double>(), built->sorted_index.as<int32_t>(), flat_box,
                options.cutoff * options.cutoff, options.full, out, capacity, d_state, stream
            );
            timer.end(VesinB200StageEmit);
            VB200_CUDA(cudaGetLastError());
            read_state();
            if (attempt == 0 && usable) {
                timer.collect(VesinB200StageBounds);
            }
            timer.collect(VesinB200StageEmit);
            if (cache.h_state->unpackable) {
                // shifts beyond the records' range (points very far outside the box): no cache for this list
                cache.disabled = true;
                cache.valid = false;
                options.skin = 0.0;
                neighbors(points, n_points, box, periodic, options, list, float_io, false);
                return;
            }
            if (cache.h_state->stale) {
                stale = true;
                break;
            }
            const size_t total = static_cast<size_t>(cache.h_state->pair_cursor);
            if (total > n_points * pair_limit_per_point) {
                throw std::runtime_error(
                    "The number of neighbor pairs exceeds the maximum capacity of " + std::to_string(n_points * pair_limit_per_point) +
                    " (max_pairs_per_point=" + std::to_string(pair_limit_per_point) + "; n_points=" + std::to_string(n_points) + "). " +
                    "Consider reducing the cutoff distance, or explicitly setting " +
                    "VESIN_CUDA_MAX_PAIRS_PER_POINT as an environment variable."
                );
            }
            if (total <= capacity) {
                list.length = total;
                ws.timed = timer.enabled;
                if (usable && attempt == 0) {
                    // Re-filtering pays when few candidates lie between cutoff and cutoff + skin per kept
                    // pair and the build has many candidates to screen per pair; otherwise a build is
                    // cheaper than a pass over the candidates. Decided by the clock: this pass is timed,
                    // the next two calls are served by plain builds (the second one timed), and the
                    // faster way serves the list from then on.
                    // (small systems are bound by launch latency either way: they keep their candidates)
                    if (cache.trial == 0) {
                        cache.filter_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - filter_started).count();
                        cache.trial = (cache.filter_seconds > 2.0e-4) ? 1 : 3;
                    }
                }
                return;
            }
            if (attempt >= 2) {
                throw std::runtime_error("internal error: the pair total kept changing between passes");
            }
            set_outputs(list, ws, options, total + total / 16 + 256);
            capacity = common_capacity(ws, options);
            VB200_CUDA(cudaMemsetAsync(&d_state->pair_cursor, 0, sizeof(unsigned long long), stream));
        }
        if (!stale || round >= 1) {
            throw std::runtime_error("internal error: candidates built for these very inputs were refused");
        }
        usable = false; // some point moved too far, or the box did: new candidates
    }
}

} // namespace

void neighbors(
    const void* points,
    size_t n_points,
    const void* box,
    const bool periodic[3],
    VesinOptions options,
    VesinNeighborList& list,
    bool float_io,
    bool canonical
) {
    if (canonical) {
        options.sorted = true; // rows in index order first, then every row is sorted
    }
    int device_count = 0;
    if (cudaGetDeviceCount(&device_count) != cudaSuccess || device_count == 0) {
        cudaGetLastError();
        throw std::runtime_error("no CUDA device is available to this process");
    }
    validate_pointers(points, box, periodic, list);
    if (n_points >= (1ull << 31) - 1) {
        throw std::runtime_error("this engine indexes points with 31 bits: too many points");
    }

    if (options.skin > 0.0 && std::isfinite(options.skin) && !options.sorted && n_points > 0 && options.algorithm != VesinBruteForce) {
        // cached candidates at cutoff + skin, re-filtered (the result is the list at the cutoff all the same)
        neighbors_with_skin(points, n_points, box, periodic, options, list, float_io);
        return;
    }

    DeviceGuard guard(list.device.device_id);
    Workspace& ws = workspace_of(list);
    const size_t pair_limit_per_point = max_pairs_per_point(options.cutoff);
    StageTimer timer(ws, PROFILING.load());
    cudaStream_t stream = ws.stream;
    const RealView flat_points{points, float_io ? 1 : 0};
    const RealView flat_box{box, float_io ? 1 : 0};
    const PointSource source = flat_source(flat_points, n_points);
    ws.values_float = float_io;

    const DeviceHeader& header = *ws.h_header;
    const size_t max_cells = size_t(1) << 27;

    const auto bad_point_error = [&]() {
        // same text as the CPU path (vesin/src/types.hpp:163-169)
        double bad[3];
        if (float_io) {
            float bad32[3];
            VB200_CUDA(cudaMemcpy(bad32, static_cast<const float*>(points) + 3 * header.first_bad, sizeof(bad32), cudaMemcpyDeviceToHost));
            bad[0] = bad32[0];
            bad[1] = bad32[1];
            bad[2] = bad32[2];
        } else {
            VB200_CUDA(cudaMemcpy(bad, static_cast<const double*>(points) + 3 * header.first_bad, sizeof(bad), cudaMemcpyDeviceToHost));
        }
        for (int axis = 0; axis < 3; axis++) {
            if (!std::isfinite(bad[axis])) {
                return std::runtime_error(
                    "point " + std::to_string(header.first_bad) + " has non-finite coordinate along axis " + std::to_string(axis) +
                    ": " + std::to_string(bad[axis])
                );
            }
        }
        return std::runtime_error("point " + std::to_string(header.first_bad) + " has a non-finite coordinate");
    };
    const auto pair_limit_error = [&]() {
        return std::runtime_error(
            "The number of neighbor pairs exceeds the maximum capacity of " + std::to_string(n_points * pair_limit_per_point) +
            " (max_pairs_per_point=" + std::to_string(pair_limit_per_point) + "; n_points=" + std::to_string(n_points) + "). " +
            "Consider reducing the cutoff distance, or explicitly setting " +
            "VESIN_CUDA_MAX_PAIRS_PER_POINT as an environment variable."
        );
    };
    // Plan from the header the host has just read. Errors in the reference's
    // order: box first (vesin/src/types.hpp:75-78), then the points.
    const auto plan_from_header = [&]() {
        auto& cache = ws.cache;
        cache.valid = false;
        PointBounds bounds{};
        for (int c = 0; c < 3; c++) {
            bool have = n_points != 0 && header.min_key[c] != ~0ull;
            bounds.min[c] = have ? key_to_double(header.min_key[c]) : 0.0;
            bounds.max[c] = have ? key_to_double(header.max_key[c]) : 0.0;
            cache.periodic[c] = header.periodic[c] != 0;
        }
        std::memcpy(cache.box, header.box, sizeof(cache.box));
        cache.plan = make_plan(header.box, cache.periodic, bounds, n_points, options.cutoff, options.full, options.sorted, max_cells);
        if (header.first_bad != NO_BAD_POINT) {
            throw bad_point_error();
        }
        cache.n_points = n_points;
        cache.cutoff = options.cutoff;
        cache.full = options.full;
        cache.sorted = options.sorted;
        cache.valid = true;
    };

    // ---- speculation: reuse the plan of the previous build when the request
    // is the same; a kernel checks that box, periodicity and extent still are ----
    bool speculative = ws.cache.valid && ws.cache.n_points == n_points && ws.cache.cutoff == options.cutoff &&
                       ws.cache.full == options.full && ws.cache.sorted == options.sorted &&
                       options.algorithm != VesinBruteForce; // its legality check wants the box of THIS call
    bool header_is_fresh = false;

    for (int round = 0;; round++) {
        timer.begin(VesinB200StageBounds);
        bool histogram_zeroed = false;
        // small systems: one CTA resets the header, checks the plan, bins, scans and scatters
        const bool fused_front = speculative && small_front_fits(n_points, ws.cache.plan);
        if (fused_front) {
            // launched below, once the scratch arrays are there
        } else if (speculative) {
            // the plan is known already: no pass over the points for their bounds. The first
            // kernel zeroes the cell histogram and checks box and periodicity, the binning
            // kernel checks every point against the plan
            const size_t cached_cells = static_cast<size_t>(ws.cache.plan.n_cells_total);
            ws.cell_count.reserve(cached_cells * sizeof(int32_t));
            launch_header_init_speculative(
                ws.d_header, flat_box, periodic, ws.cell_count.as<int32_t>(), cached_cells, ws.cache.box, ws.cache.periodic, stream
            );
            histogram_zeroed = true;
        } else {
            launch_header_init(ws.d_header, flat_box, periodic, stream);
            launch_bounds(source, ws.d_header, stream);
        }
        timer.end(VesinB200StageBounds);
        if (!speculative) {
            if (!header_is_fresh) {
                VB200_CUDA(cudaGetLastError());
                read_header(ws);
            }
            plan_from_header();
        }
        const GridPlan& plan = ws.cache.plan;

        if (options.algorithm == VesinBruteForce && 2.0 * options.cutoff > min_periodic_face_distance(plan)) {
            // vesin/src/vesin_cuda.cpp:404-409
            throw std::runtime_error("Invalid cutoff: too large for box dimensions");
        }

        if (n_points == 0) {
            VB200_CUDA(cudaGetLastError());
            read_header(ws);
            if (header.status & STATUS_PLAN_STALE) {
                speculative = false;
                header_is_fresh = true;
                continue;
            }
            set_outputs(list, ws, options, 256);
            list.length = 0;
            ws.timed = timer.enabled;
            return;
        }

        // ---- scratch ----
        const size_t n_cells = static_cast<size_t>(plan.n_cells_total);
        const size_t n_units = static_cast<size_t>(plan.n_units);
        ws.cell_of.reserve(n_points * sizeof(int32_t));
        ws.rank.reserve(n_points * sizeof(int32_t));
        ws.shift.reserve(n_points * 3 * sizeof(int32_t));
        ws.cell_count.reserve(n_cells * sizeof(int32_t));
        ws.cell_start.reserve((n_cells + 1) * sizeof(int32_t));
        ws.sorted_pos.reserve(n_points * 3 * sizeof(double));
        ws.sorted_index.reserve(n_points * sizeof(int32_t));
        ws.sorted_shift.reserve(n_points * 3 * sizeof(int32_t));
        ws.scan_tmp.reserve(scan_tmp_bytes(std::max(n_points, n_cells)));
        SortedPoints sorted{ws.sorted_pos.as<double>(), ws.sorted_index.as<int32_t>(), ws.sorted_shift.as<int32_t>()};

        // ---- cell list ----
        if (fused_front || (!speculative && small_front_fits(n_points, plan))) {
            timer.begin(VesinB200StageBin);
            launch_small_front(
                flat_points, n_points, plan, ws.cell_of.as<int32_t>(), ws.rank.as<int32_t>(), ws.shift.as<int32_t>(),
                ws.cell_start.as<int32_t>(), sorted, ws.d_header, flat_box, periodic, speculative, ws.cache.box, ws.cache.periodic, stream
            );
            timer.end(VesinB200StageBin);
            timer.begin(VesinB200StageScanCells);
            timer.end(VesinB200StageScanCells);
            timer.begin(VesinB200StageScatter);
            timer.end(VesinB200StageScatter);
        } else {
            timer.begin(VesinB200StageBin);
            if (!histogram_zeroed) {
                VB200_CUDA(cudaMemsetAsync(ws.cell_count.ptr, 0, n_cells * sizeof(int32_t), stream));
            }
            launch_bin(
                source, 0, n_points, plan, ws.cell_of.as<int32_t>(), ws.rank.as<int32_t>(), ws.shift.as<int32_t>(),
                ws.cell_count.as<int32_t>(), ws.d_header, speculative, true, stream
            );
            timer.end(VesinB200StageBin);
            timer.begin(VesinB200StageScanCells);
            launch_scan_cells(ws.cell_count.as<int32_t>(), ws.cell_start.as<int32_t>(), n_cells, ws.scan_tmp.ptr, stream);
            timer.end(VesinB200StageScanCells);
            timer.begin(VesinB200StageScatter);
            launch_scatter(
                source, ws.cell_of.as<int32_t>(), ws.rank.as<int32_t>(), ws.shift.as<int32_t>(), ws.cell_start.as<int32_t>(), n_cells,
                sorted, nullptr, ws.d_header, stream
            );
            timer.end(VesinB200StageScatter);
        }
        const auto collect_front_stages = [&]() {
            timer.collect(VesinB200StageBounds);
            timer.collect(VesinB200StageBin);
            timer.collect(VesinB200StageScanCells);
            timer.collect(VesinB200StageScatter);
        };
        // after a read-back: did the kernels accept the plan?
        const auto plan_was_refused = [&]() {
            if ((header.status & STATUS_ABORT_MASK) == 0) {
                return false;
            }
            if (!speculative) {
                // a plan made from this very header can only be refused for a bad point
                throw bad_point_error();
            }
            speculative = false;
            header_is_fresh = false; // the speculative round did not compute the bounds of the points
            return true;
        };

        if (!plan.by_index) {
            // ---- unsorted list: one fused pass, one read-back. The arrays of
            // the previous call are tried first; when the pairs do not fit,
            // the pass has still counted them: grow to the exact total and run
            // it again (first build on a list, or a system that grew). ----
            set_outputs(list, ws, options, std::max<size_t>(common_capacity(ws, options), 256));
            size_t capacity = common_capacity(ws, options);
            size_t total = 0;
            bool refused = false;
            // arrays of the minimum size (a list that was never filled) cannot hold the pairs
            // of a large system: the first pass then only counts (capacity 0)
            bool count_only = capacity <= 256 && n_points >= 4096;
            for (int attempt = 0;; attempt++) {
                PairOutput out{
                    reinterpret_cast<unsigned long long*>(list.pairs),
                    reinterpret_cast<int32_t*>(list.shifts),
                    list.distances,
                    reinterpret_cast<double*>(list.vectors),
                    float_io ? 1 : 0,
                };
                const size_t pass_capacity = count_only ? 0 : capacity;
                timer.begin(VesinB200StageEmit);
                launch_pairs(plan, ws.cell_start.as<int32_t>(), sorted, out, pass_capacity, ws.d_header, stream, n_points);
                timer.end(VesinB200StageEmit);
                VB200_CUDA(cudaGetLastError());
                read_header(ws);
                if (attempt == 0) {
                    collect_front_stages();
                    if (plan_was_refused()) {
                        refused = true;
                        break;
                    }
                }
                timer.collect(VesinB200StageEmit);
                total = static_cast<size_t>(header.pair_cursor);
                if (total > n_points * pair_limit_per_point) {
                    throw pair_limit_error();
                }
                if (total <= pass_capacity) {
                    break;
                }
                if (attempt >= 2) {
                    throw std::runtime_error("internal error: the pair total kept changing between passes");
                }
                count_only = false;
                if (total > capacity) {
                    set_outputs(list, ws, options, total + total / 16 + 256);
                    capacity = common_capacity(ws, options);
                }
                VB200_CUDA(cudaMemsetAsync(&ws.d_header->pair_cursor, 0, 2 * sizeof(unsigned long long), stream)); // and run_cursor
            }
            if (refused) {
                continue;
            }
            list.length = total;
            ws.timed = timer.enabled;
            return;
        }

        // ---- sorted list: rows in index order need a scan between two passes ----
        ws.unit_mask_base.reserve(n_units * sizeof(unsigned long long));
        ws.unit_words.reserve(n_units * sizeof(uint32_t));
        ws.row_count.reserve(n_points * sizeof(uint32_t));
        ws.row_start.reserve((n_points + 1) * sizeof(unsigned long long));
        ws.row_fill.reserve(n_points * sizeof(uint32_t));
        if (ws.masks.bytes == 0) {
            // first guess for the hit-mask storage: uniform density. Every unit
            // stores (tiles of 32 lanes) x (words per home point).
            double per_cell = static_cast<double>(n_points) / static_cast<double>(n_cells);
            double stencil_cells = (plan.pencil + 2.0 * plan.n_search[0]) * (2.0 * plan.n_search[1] + 1.0) * (2.0 * plan.n_search[2] + 1.0);
            double words = per_cell * stencil_cells / 32.0 + 1.5;
            double lanes = static_cast<double>(n_units) * 32.0 * std::ceil(per_cell * plan.pencil / 32.0 + 0.35);
            double guess = std::min(1.2 * words * lanes * sizeof(uint32_t), 2.0e9);
            ws.masks.reserve(static_cast<size_t>(guess) + 1024);
        }

        bool refused = false;
        for (int attempt = 0;; attempt++) {
            timer.begin(VesinB200StageCount);
            VB200_CUDA(cudaMemsetAsync(ws.row_count.ptr, 0, n_points * sizeof(uint32_t), stream));
            launch_count(
                plan, ws.cell_start.as<int32_t>(), sorted, ws.masks.as<uint32_t>(), ws.masks.bytes / sizeof(uint32_t),
                ws.unit_mask_base.as<unsigned long long>(), ws.unit_words.as<uint32_t>(), ws.row_count.as<uint32_t>(), ws.d_header, stream
            );
            timer.end(VesinB200StageCount);
            timer.begin(VesinB200StageScanRows);
            launch_scan_rows(
                ws.row_count.as<uint32_t>(), ws.row_start.as<unsigned long long>(), n_points, ws.scan_tmp.ptr,
                &ws.d_header->total_pairs, stream
            );
            timer.end(VesinB200StageScanRows);
            VB200_CUDA(cudaGetLastError());
            read_header(ws);
            if (attempt == 0) {
                collect_front_stages();
                if (plan_was_refused()) {
                    refused = true;
                    break;
                }
            }
            timer.collect(VesinB200StageCount);
            timer.collect(VesinB200StageScanRows);
            if ((header.status & STATUS_MASK_OVERFLOW) == 0) {
                break;
            }
            if (attempt >= 2) {
                throw std::runtime_error("internal error: hit-mask storage kept overflowing");
            }
            // the cursor holds the exact requirement: grow and decide again
            size_t wanted = static_cast<size_t>(header.mask_cursor) * sizeof(uint32_t);
            ws.masks.reserve(wanted + wanted / 16 + 1024);
            size_t offset = offsetof(DeviceHeader, total_pairs);
            VB200_CUDA(cudaMemsetAsync(reinterpret_cast<char*>(ws.d_header) + offset, 0, offsetof(DeviceHeader, box) - offset, stream));
        }
        if (refused) {
            continue;
        }

        const size_t total = static_cast<size_t>(header.total_pairs);
        if (total > n_points * pair_limit_per_point) {
            throw pair_limit_error();
        }
        size_t capacity = std::max<size_t>(total, 256);
        if (capacity > common_capacity(ws, options) && ws.out_pairs.bytes != 0) {
            capacity += capacity / 16; // a list that keeps growing gets some headroom
        }
        set_outputs(list, ws, options, capacity);
        if (total > 0) {
            PairOutput out{
                reinterpret_cast<unsigned long long*>(list.pairs),
                reinterpret_cast<int32_t*>(list.shifts),
                list.distances,
                reinterpret_cast<double*>(list.vectors),
                float_io ? 1 : 0,
            };
            timer.begin(VesinB200StageEmit);
            VB200_CUDA(cudaMemsetAsync(ws.row_fill.ptr, 0, n_points * sizeof(uint32_t), stream));
            launch_emit(
                plan, ws.cell_start.as<int32_t>(), sorted, ws.masks.as<uint32_t>(), ws.unit_mask_base.as<unsigned long long>(),
                ws.unit_words.as<uint32_t>(), ws.row_start.as<unsigned long long>(), ws.row_fill.as<uint32_t>(), out, stream
            );
            if (canonical) {
                // every row sorted by (second index, shift) into a second set of arrays, which then become the list's
                ws.alt_pairs.reserve(ws.out_pairs.bytes);
                PairOutput sorted_out{ws.alt_pairs.as<unsigned long long>(), nullptr, nullptr, nullptr, float_io ? 1 : 0};
                if (options.return_shifts) {
                    ws.alt_shifts.reserve(ws.out_shifts.bytes);
                    sorted_out.shifts = ws.alt_shifts.as<int32_t>();
                }
                if (options.return_distances) {
                    ws.alt_distances.reserve(ws.out_distances.bytes);
                    sorted_out.distances = ws.alt_distances.as<double>();
                }
                if (options.return_vectors) {
                    ws.alt_vectors.reserve(ws.out_vectors.bytes);
                    sorted_out.vectors = ws.alt_vectors.as<double>();
                }
                // a second index can come twice in a row only with two images of the same point
                // within the cutoff of the first: a lattice vector shorter than twice the cutoff
                bool duplicates_possible = false;
                for (int k = 0; k < 3; k++) {
                    duplicates_possible = duplicates_possible || (plan.periodic[k] && plan.face_dist[k] < 2.0 * options.cutoff * (1.0 + 1e-9));
                }
                launch_sort_rows(ws.row_start.as<unsigned long long>(), n_points, out, sorted_out, duplicates_possible, stream);
                std::swap(ws.out_pairs, ws.alt_pairs);
                list.pairs = reinterpret_cast<size_t(*)[2]>(ws.out_pairs.ptr);
                if (options.return_shifts) {
                    std::swap(ws.out_shifts, ws.alt_shifts);
                    list.shifts = reinterpret_cast<int32_t(*)[3]>(ws.out_shifts.ptr);
                }
                if (options.return_distances) {
                    std::swap(ws.out_distances, ws.alt_distances);
                    list.distances = ws.out_distances.as<double>();
                }
                if (options.return_vectors) {
                    std::swap(ws.out_vectors, ws.alt_vectors);
                    list.vectors = reinterpret_cast<double(*)[3]>(ws.out_vectors.ptr);
                }
            }
            timer.end(VesinB200StageEmit);
            VB200_CUDA(cudaGetLastError());
            VB200_CUDA(cudaStreamSynchronize(stream));
            timer.collect(VesinB200StageEmit);
        }
        list.length = total;
        ws.timed = timer.enabled;
        return;
    }
}

void neighbors_batch(
    const void* points,
    bool float_io,
    const size_t* system_offsets,
    size_t n_systems,
    const void* boxes,
    const bool (*periodic)[3],
    VesinOptions options,
    bool global_indices,
    VesinNeighborList& list,
    const size_t** pair_offsets
) {
    if (n_systems >= (1ull << 31)) {
        throw std::runtime_error("too many systems in the batch");
    }
    for (size_t k = 0; k < n_systems; k++) {
        if (system_offsets[k + 1] < system_offsets[k]) {
            throw std::runtime_error("`system_offsets` must not decrease");
        }
    }
    const size_t n_points = n_systems ? system_offsets[n_systems] - system_offsets[0] : 0;
    size_t largest = 0;
    for (size_t k = 0; k < n_systems; k++) {
        largest = std::max(largest, system_offsets[k + 1] - system_offsets[k]);
    }
    if (largest > small_systems_max_points()) {
        throw std::runtime_error(
            "a system of the batch has " + std::to_string(largest) + " points; the batch entry point handles at most " +
            std::to_string(small_systems_max_points()) + " points per system, use vesin_neighbors for larger systems"
        );
    }
    const auto on_device = [&](const void* ptr) {
        PointerInfo info = inspect(ptr);
        return info.resolved && info.on_device && info.device == list.device.device_id;
    };
    if (n_points > 0 && !on_device(points)) {
        throw std::runtime_error("`points` pointer is not allocated on the CUDA device of `neighbors`");
    }
    if ((boxes != nullptr && !on_device(boxes)) || (periodic != nullptr && !on_device(periodic))) {
        throw std::runtime_error("`boxes` and `periodic` must be NULL or device memory on the CUDA device of `neighbors`");
    }
    if ((boxes == nullptr) != (periodic == nullptr)) {
        throw std::runtime_error("`boxes` and `periodic` must be given together");
    }

    DeviceGuard guard(list.device.device_id);
    Workspace& ws = workspace_of(list);
    ws.cache.valid = false; // the list was used for something else than a single system
    ws.values_float = float_io;
    const size_t pair_limit_per_point = max_pairs_per_point(options.cutoff);
    cudaStream_t stream = ws.stream;
    const DeviceHeader& header = *ws.h_header;

    {
        const void* before = ws.batch_offsets.ptr;
        ws.batch_offsets.reserve((n_systems + 1) * sizeof(unsigned long long));
        if (ws.batch_offsets.ptr != before) {
            ws.batch_offsets_host.clear(); // a new buffer holds nothing yet
        }
    }
    ws.unit_count.reserve(std::max<size_t>(n_systems, 1) * sizeof(unsigned long long));
    ws.unit_start.reserve((n_systems + 1) * sizeof(unsigned long long));
    ws.scan_tmp.reserve(scan_tmp_bytes(std::max<size_t>(n_systems, 1)));
    static_assert(sizeof(size_t) == sizeof(unsigned long long), "offsets are copied as they are");
    // (a batch with the same layout as the last one, the usual case in a loop over steps, keeps
    //  the copy of its offsets on the device: an upload from pageable memory costs 20-30 us)
    if (ws.batch_offsets_host.size() != n_systems + 1 ||
        std::memcmp(ws.batch_offsets_host.data(), system_offsets, (n_systems + 1) * sizeof(size_t)) != 0) {
        ws.batch_offsets_host.assign(system_offsets, system_offsets + n_systems + 1);
        VB200_CUDA(cudaMemcpyAsync(
            ws.batch_offsets.ptr, ws.batch_offsets_host.data(), (n_systems + 1) * sizeof(size_t), cudaMemcpyHostToDevice, stream
        ));
    }
    VB200_CUDA(cudaMemsetAsync(ws.d_header, 0, sizeof(DeviceHeader), stream));
    VB200_CUDA(cudaMemsetAsync(&ws.d_header->first_bad, 0xff, sizeof(unsigned long long), stream));
    VB200_CUDA(cudaMemsetAsync(&ws.d_header->mask_cursor, 0xff, sizeof(unsigned long long), stream)); // first singular system

    BatchInput in{};
    in.points = points;
    in.is_float = float_io ? 1 : 0;
    in.offsets = ws.batch_offsets.as<unsigned long long>();
    in.boxes = boxes;
    in.periodic = reinterpret_cast<const bool*>(periodic);
    in.n_systems = static_cast<unsigned>(n_systems);
    in.cutoff = options.cutoff;
    in.cutoff2 = options.cutoff * options.cutoff;
    in.full = options.full ? 1 : 0;
    in.global_indices = global_indices ? 1 : 0;

    // systems with a periodic direction or many points take the CTA-per-system kernel
    const bool any_for_cta_kernel = periodic != nullptr || largest > molecules_max_points();
    const auto outputs = [&]() {
        return PairOutput{
            reinterpret_cast<unsigned long long*>(list.pairs),
            reinterpret_cast<int32_t*>(list.shifts),
            list.distances,
            reinterpret_cast<double*>(list.vectors),
            float_io ? 1 : 0,
        };
    };
    // A list that was filled before writes into the arrays it has, right behind the counting pass
    // and the scan, without waiting for the host to see the total: one read-back per call. A
    // system whose block does not fit writes nothing; the host then grows the arrays and runs the
    // writing pass again.
    const size_t existing = common_capacity(ws, options);
    const bool speculative = n_systems > 0 && existing >= 256;
    size_t total = 0;
    if (n_systems > 0) {
        launch_small_count(in, largest, any_for_cta_kernel, ws.unit_count.as<unsigned long long>(), ws.d_header, stream);
        launch_scan_units(
            ws.unit_count.as<unsigned long long>(), ws.unit_start.as<unsigned long long>(), n_systems, ws.scan_tmp.ptr,
            &ws.d_header->total_pairs, stream
        );
        if (speculative) {
            set_outputs(list, ws, options, existing);
            launch_small_emit(in, largest, any_for_cta_kernel, ws.unit_start.as<unsigned long long>(), outputs(), ws.d_header, stream, existing);
        }
        VB200_CUDA(cudaGetLastError());
        read_header(ws);
        if (header.status & STATUS_STENCIL_TOO_LARGE) {
            throw std::runtime_error("the cutoff is too large for the box of system " + std::to_string(header.mask_cursor) + " of the batch");
        }
        if (header.status & STATUS_SINGULAR_BOX) {
            throw std::runtime_error("the box matrix is not invertible (system " + std::to_string(header.mask_cursor) + " of the batch)");
        }
        if (header.status & STATUS_BAD_POINT) {
            throw std::runtime_error("point " + std::to_string(header.first_bad) + " of the batch has a non-finite coordinate");
        }
        total = static_cast<size_t>(header.total_pairs);
        if (total > n_points * pair_limit_per_point) {
            throw std::runtime_error(
                "The number of neighbor pairs exceeds the maximum capacity of " + std::to_string(n_points * pair_limit_per_point) +
                " (max_pairs_per_point=" + std::to_string(pair_limit_per_point) + "; n_points=" + std::to_string(n_points) + "). " +
                "Consider reducing the cutoff distance, or explicitly setting " +
                "VESIN_CUDA_MAX_PAIRS_PER_POINT as an environment variable."
            );
        }
    } else {
        VB200_CUDA(cudaMemsetAsync(ws.unit_start.ptr, 0, sizeof(unsigned long long), stream));
    }

    if (!(speculative && total <= existing)) {
        size_t capacity = std::max<size_t>(total, 256);
        if (capacity > common_capacity(ws, options) && ws.out_pairs.bytes != 0) {
            capacity += capacity / 16;
        }
        set_outputs(list, ws, options, capacity);
        if (total > 0) {
            launch_small_emit(in, largest, any_for_cta_kernel, ws.unit_start.as<unsigned long long>(), outputs(), ws.d_header, stream);
            VB200_CUDA(cudaGetLastError());
        }
    }
    VB200_CUDA(cudaStreamSynchronize(stream));
    list.length = total;
    if (pair_offsets != nullptr) {
        *pair_offsets = reinterpret_cast<const size_t*>(ws.unit_start.ptr);
    }
}

cudaStream_t list_stream(VesinNeighborList& list) {
    DeviceGuard guard(list.device.device_id);
    return workspace_of(list).stream;
}

void neighbors_slab_core(
    const void* points,
    bool float_io,
    size_t n_array,
    size_t n_owned,
    const int64_t* global_index,
    const HaloMessages* halo,
    const double box[9],
    const bool periodic[3],
    int axis,
    double lower,
    double upper,
    VesinOptions options,
    VesinNeighborList& list
) {
    if (n_owned > n_array) {
        throw std::runtime_error("`n_owned` can not be larger than `n_points`");
    }
    if (options.sorted) {
        throw std::runtime_error("sorted lists are not available for slab-decomposed systems");
    }
    const bool with_messages = halo != nullptr && halo->capacity > 0;
    PointSource source = flat_source(RealView{points, float_io ? 1 : 0}, n_array);
    source.global_index = reinterpret_cast<const long long*>(global_index);
    if (with_messages) {
        source.message[0] = halo->from_upper;
        source.message[1] = halo->from_lower;
        source.capacity = halo->capacity;
    }
    const size_t n_index = source.n_index();
    if (n_index >= (1ull << 31) - 1) {
        throw std::runtime_error("this engine indexes points with 31 bits: too many points");
    }

    DeviceGuard guard(list.device.device_id);
    Workspace& ws = workspace_of(list);
    ws.cache.valid = false; // this list is not used for plain single-system builds
    ws.values_float = float_io;
    const size_t pair_limit_per_point = max_pairs_per_point(options.cutoff);
    StageTimer timer(ws, PROFILING.load());
    cudaStream_t stream = ws.stream;
    const DeviceHeader& header = *ws.h_header;
    const size_t max_cells = size_t(1) << 27;

    // the halo messages arrive on another stream: this stream waits for them once,
    // as late as the work allows
    // (the caller may leave it to the build to say when the exchange is to be queued: behind
    //  the launches of the sort of the owned points, whose host time then hides it)
    bool exchange_started = !(with_messages && halo->start_exchange);
    const auto start_exchange_once = [&]() {
        if (!exchange_started) {
            exchange_started = true;
            halo->start_exchange();
        }
    };
    bool messages_awaited = !(with_messages && halo->received != nullptr);
    const auto await_messages = [&]() {
        start_exchange_once();
        if (!messages_awaited) {
            VB200_CUDA(cudaStreamWaitEvent(stream, halo->received, 0));
            messages_awaited = true;
        }
    };

    const bool any_open = !(periodic[0] && periodic[1] && periodic[2]);
    size_t n_estimate = ws.slab.n_local != 0 ? ws.slab.n_local : n_array + (with_messages ? halo->expected_records : 0);

    for (int round = 0;; round++) {
        // ---- extent of the points along non-periodic directions: taken from the last
        // build that computed it (the binning kernel checks every point against it) ----
        const bool bounds_cached = ws.slab.bounds_valid;
        if (any_open && !bounds_cached) {
            await_messages();
            timer.begin(VesinB200StageBounds);
            launch_header_reset(ws.d_header, nullptr, 0, stream);
            launch_bounds(source, ws.d_header, stream);
            timer.end(VesinB200StageBounds);
            VB200_CUDA(cudaGetLastError());
            read_header(ws);
            timer.collect(VesinB200StageBounds);
            if (header.first_bad != NO_BAD_POINT) {
                throw std::runtime_error("local point " + std::to_string(header.first_bad) + " has a non-finite coordinate");
            }
            for (int c = 0; c < 3; c++) {
                const bool have = header.min_key[c] != ~0ull;
                ws.slab.bounds.min[c] = have ? key_to_double(header.min_key[c]) : 0.0;
                ws.slab.bounds.max[c] = have ? key_to_double(header.max_key[c]) : 0.0;
            }
            ws.slab.bounds_valid = true;
        }
        const PointBounds bounds = any_open ? ws.slab.bounds : PointBounds{};
        GridPlan plan = make_plan(box, periodic, bounds, std::max<size_t>(n_estimate, 1), options.cutoff, options.full, false, max_cells);
        make_slab_window(plan, axis, lower, upper, std::max<size_t>(n_estimate, 1), n_owned, options.cutoff);

        const size_t n_cells = static_cast<size_t>(plan.n_cells_total);
        const size_t n_slots = std::max<size_t>(n_index, 1);
        ws.cell_of.reserve(n_slots * sizeof(int32_t));
        ws.rank.reserve(n_slots * sizeof(int32_t));
        ws.shift.reserve(n_slots * 3 * sizeof(int32_t));
        ws.cell_count.reserve(n_cells * sizeof(int32_t));
        ws.cell_start.reserve((n_cells + 1) * sizeof(int32_t));
        ws.sorted_pos.reserve(n_slots * 3 * sizeof(double));
        ws.sorted_index.reserve(n_slots * sizeof(int32_t));
        ws.sorted_shift.reserve(n_slots * 3 * sizeof(int32_t));
        ws.sorted_global.reserve(n_slots * sizeof(int32_t));
        ws.scan_tmp.reserve(scan_tmp_bytes(std::max(n_slots, n_cells)));
        SortedPoints sorted{ws.sorted_pos.as<double>(), ws.sorted_index.as<int32_t>(), ws.sorted_shift.as<int32_t>()};
        // the pair pass writes global indices: it reads them where a plain build keeps local ones
        SortedPoints sorted_for_pairs{sorted.pos, ws.sorted_global.as<int32_t>(), sorted.shift};

        // Cut along the last direction: the cells of the owned layers come first in the cell
        // order (see window_storage_layer), so the owned points are sorted on their own, while
        // the messages are on their way; the halo is sorted behind them. Other directions:
        // everything is sorted together once the messages are there.
        const bool owned_first = with_messages && axis == 2 && n_owned == n_array;
        const size_t owned_cells = owned_first ? n_cells / static_cast<size_t>(plan.n_cells[2]) * static_cast<size_t>(plan.n_cells[2] - 2) : n_cells;
        set_outputs(list, ws, options, std::max<size_t>(common_capacity(ws, options), 256));
        size_t capacity = common_capacity(ws, options);
        bool count_only = capacity <= 256 && n_owned >= 4096;
        const auto outputs = [&]() {
            return PairOutput{
                reinterpret_cast<unsigned long long*>(list.pairs),
                reinterpret_cast<int32_t*>(list.shifts),
                list.distances,
                reinterpret_cast<double*>(list.vectors),
                float_io ? 1 : 0,
            };
        };
        // The units that need nothing from the halo are paired while the halo is received and
        // sorted in on a second stream, which also pairs the units next to the halo; the two
        // streams join before the header is read. (Stage times are taken on one stream: a
        // profiled build runs everything in order.)
        const bool overlapped = owned_first && !timer.enabled && pairs_have_interior(plan);
        bool pairs_launched = false;

        timer.begin(VesinB200StageBin);
        launch_header_reset(ws.d_header, ws.cell_count.as<int32_t>(), n_cells, stream);
        // points of the caller's array first: their binning runs while the messages are on their way
        launch_bin(
            source, 0, n_array, plan, ws.cell_of.as<int32_t>(), ws.rank.as<int32_t>(), ws.shift.as<int32_t>(), ws.cell_count.as<int32_t>(),
            ws.d_header, true, true, stream
        );
        timer.end(VesinB200StageBin);
        if (owned_first) {
            timer.begin(VesinB200StageScanCells);
            launch_scan_cells(ws.cell_count.as<int32_t>(), ws.cell_start.as<int32_t>(), owned_cells, ws.scan_tmp.ptr, stream);
            timer.end(VesinB200StageScanCells);
            timer.begin(VesinB200StageScatter);
            launch_scatter(
                source, ws.cell_of.as<int32_t>(), ws.rank.as<int32_t>(), ws.shift.as<int32_t>(), ws.cell_start.as<int32_t>(), n_cells, sorted,
                ws.sorted_global.as<int32_t>(), ws.d_header, stream, 0, n_array
            );
            timer.end(VesinB200StageScatter);
            cudaStream_t halo_stream = stream;
            const size_t pass_capacity = count_only ? 0 : capacity;
            if (overlapped) {
                if (ws.side_stream == nullptr) {
                    VB200_CUDA(cudaStreamCreateWithFlags(&ws.side_stream, cudaStreamNonBlocking));
                    VB200_CUDA(cudaEventCreateWithFlags(&ws.owned_sorted, cudaEventDisableTiming));
                    VB200_CUDA(cudaEventCreateWithFlags(&ws.side_done, cudaEventDisableTiming));
                }
                halo_stream = ws.side_stream;
                start_exchange_once(); // before the interior kernel takes every SM
                VB200_CUDA(cudaEventRecord(ws.owned_sorted, stream));
                launch_pairs(
                    plan, ws.cell_start.as<int32_t>(), sorted_for_pairs, outputs(), pass_capacity, ws.d_header, stream, 0, PAIR_PART_INTERIOR
                );
                VB200_CUDA(cudaStreamWaitEvent(halo_stream, ws.owned_sorted, 0));
                if (halo->received != nullptr) {
                    VB200_CUDA(cudaStreamWaitEvent(halo_stream, halo->received, 0));
                }
            } else {
                timer.begin(VesinB200StageHalo);
                await_messages();
            }
            // the halo: binned, scanned behind the owned cells, scattered behind the owned records
            launch_bin(
                source, n_array, n_index, plan, ws.cell_of.as<int32_t>(), ws.rank.as<int32_t>(), ws.shift.as<int32_t>(),
                ws.cell_count.as<int32_t>(), ws.d_header, true, false, halo_stream
            );
            launch_scan_cells(
                ws.cell_count.as<int32_t>() + owned_cells, ws.cell_start.as<int32_t>() + owned_cells, n_cells - owned_cells, ws.scan_tmp.ptr,
                halo_stream, ws.cell_start.as<int32_t>() + owned_cells
            );
            launch_scatter(
                source, ws.cell_of.as<int32_t>(), ws.rank.as<int32_t>(), ws.shift.as<int32_t>(), ws.cell_start.as<int32_t>(), n_cells, sorted,
                ws.sorted_global.as<int32_t>(), ws.d_header, halo_stream, n_array, n_index
            );
            if (overlapped) {
                launch_pairs(
                    plan, ws.cell_start.as<int32_t>(), sorted_for_pairs, outputs(), pass_capacity, ws.d_header, halo_stream, 0, PAIR_PART_BOUNDARY
                );
                // everything queued on `stream` from here on comes after both parts
                VB200_CUDA(cudaEventRecord(ws.side_done, halo_stream));
                VB200_CUDA(cudaStreamWaitEvent(stream, ws.side_done, 0));
                messages_awaited = true;
                pairs_launched = true;
            } else {
                timer.end(VesinB200StageHalo);
            }
        } else {
            if (with_messages) {
                timer.begin(VesinB200StageHalo);
                await_messages();
                launch_bin(
                    source, n_array, n_index, plan, ws.cell_of.as<int32_t>(), ws.rank.as<int32_t>(), ws.shift.as<int32_t>(),
                    ws.cell_count.as<int32_t>(), ws.d_header, true, false, stream
                );
                timer.end(VesinB200StageHalo);
            }
            timer.begin(VesinB200StageScanCells);
            launch_scan_cells(ws.cell_count.as<int32_t>(), ws.cell_start.as<int32_t>(), n_cells, ws.scan_tmp.ptr, stream);
            timer.end(VesinB200StageScanCells);
            timer.begin(VesinB200StageScatter);
            launch_scatter(
                source, ws.cell_of.as<int32_t>(), ws.rank.as<int32_t>(), ws.shift.as<int32_t>(), ws.cell_start.as<int32_t>(), n_cells, sorted,
                ws.sorted_global.as<int32_t>(), ws.d_header, stream
            );
            timer.end(VesinB200StageScatter);
        }

        size_t total = 0;
        bool refused = false;
        for (int attempt = 0;; attempt++) {
            const size_t pass_capacity = count_only ? 0 : capacity;
            if (!(attempt == 0 && pairs_launched)) {
                timer.begin(VesinB200StageEmit);
                launch_pairs(plan, ws.cell_start.as<int32_t>(), sorted_for_pairs, outputs(), pass_capacity, ws.d_header, stream);
                timer.end(VesinB200StageEmit);
            }
            VB200_CUDA(cudaGetLastError());
            read_header(ws);
            if (attempt == 0) {
                timer.collect(VesinB200StageBin);
                timer.collect(VesinB200StageScanCells);
                timer.collect(VesinB200StageScatter);
                if (with_messages) {
                    timer.collect(VesinB200StageHalo);
                }
                if (header.status & STATUS_BAD_POINT) {
                    throw std::runtime_error("local point " + std::to_string(header.first_bad) + " has a non-finite coordinate");
                }
                if (header.status & STATUS_HALO_OVERFLOW) {
                    throw std::runtime_error(
                        "a halo message brought " + std::to_string(std::max(header.halo_count[0], header.halo_count[1])) +
                        " records but holds " + std::to_string(source.capacity) + ": raise the halo capacity (the same value on every rank)"
                    );
                }
                if (header.status & STATUS_INDEX_RANGE) {
                    throw std::runtime_error("a global index is negative or does not fit 31 bits");
                }
                if (header.status & STATUS_PLAN_STALE) {
                    if (!bounds_cached || round >= 2) {
                        throw std::runtime_error("internal error: a plan made from the bounds of these very points was refused");
                    }
                    ws.slab.bounds_valid = false; // the points left the extent of an earlier build: look again
                    refused = true;
                    break;
                }
            }
            timer.collect(VesinB200StageEmit);
            total = static_cast<size_t>(header.pair_cursor);
            if (total > std::max<size_t>(n_owned, 1) * 2 * pair_limit_per_point) {
                throw std::runtime_error(
                    "The number of neighbor pairs exceeds the maximum capacity of " + std::to_string(n_owned * pair_limit_per_point) +
                    " (max_pairs_per_point=" + std::to_string(pair_limit_per_point) + "; n_points=" + std::to_string(n_owned) + "). " +
                    "Consider reducing the cutoff distance, or explicitly setting " +
                    "VESIN_CUDA_MAX_PAIRS_PER_POINT as an environment variable."
                );
            }
            if (total <= pass_capacity) {
                break;
            }
            if (attempt >= 2) {
                throw std::runtime_error("internal error: the pair total kept changing between passes");
            }
            count_only = false;
            if (total > capacity) {
                set_outputs(list, ws, options, total + total / 16 + 256);
                capacity = common_capacity(ws, options);
            }
            // mask_cursor (the second run counter of a slab build), pair_cursor and run_cursor
            VB200_CUDA(cudaMemsetAsync(&ws.d_header->mask_cursor, 0, 3 * sizeof(unsigned long long), stream));
        }
        if (refused) {
            continue;
        }
        ws.slab.n_local = n_array + static_cast<size_t>(std::min<unsigned long long>(header.halo_count[0], source.capacity)) +
                          static_cast<size_t>(std::min<unsigned long long>(header.halo_count[1], source.capacity));
        list.length = total;
        ws.timed = timer.enabled;
        return;
    }
}

void neighbors_slab(
    const void* points,
    bool float_io,
    size_t n_points,
    size_t n_owned,
    const int64_t* global_index,
    const void* box,
    const bool periodic[3],
    int axis,
    double lower,
    double upper,
    VesinOptions options,
    VesinNeighborList& list
) {
    validate_pointers(points, box, periodic, list);
    {
        PointerInfo info = inspect(global_index);
        if (n_points > 0 && !(info.resolved && info.on_device && info.device == list.device.device_id)) {
            throw std::runtime_error("`global_index` pointer is not allocated on the CUDA device of `neighbors`");
        }
    }
    // box and periodicity live in device memory (the convention of vesin_neighbors): bring them over
    double host_box[9];
    bool host_periodic[3];
    {
        DeviceGuard guard(list.device.device_id);
        if (float_io) {
            float box32[9];
            VB200_CUDA(cudaMemcpy(box32, box, sizeof(box32), cudaMemcpyDeviceToHost));
            for (int k = 0; k < 9; k++) {
                host_box[k] = box32[k];
            }
        } else {
            VB200_CUDA(cudaMemcpy(host_box, box, sizeof(host_box), cudaMemcpyDeviceToHost));
        }
        VB200_CUDA(cudaMemcpy(host_periodic, periodic, sizeof(host_periodic), cudaMemcpyDeviceToHost));
    }
    neighbors_slab_core(
        points, float_io, n_points, n_owned, global_index, nullptr, host_box, host_periodic, axis, lower, upper, options, list
    );
}

int list_value_bytes(const VesinNeighborList& list) {
    if (list.opaque == nullptr || list.device.type != VesinCUDA) {
        return 0;
    }
    return static_cast<const Workspace*>(list.opaque)->values_float ? 4 : 8;
}

void list_checksum(const VesinNeighborList& list, unsigned long long result[4]) {
    if (list.opaque == nullptr || list.device.type != VesinCUDA) {
        throw std::runtime_error("the list holds nothing: build it first");
    }
    DeviceGuard guard(list.device.device_id);
    Workspace& ws = *static_cast<Workspace*>(list.opaque);
    ws.checksum.reserve(4 * sizeof(unsigned long long));
    launch_checksum(
        reinterpret_cast<const unsigned long long*>(list.pairs), reinterpret_cast<const int32_t*>(list.shifts), list.distances,
        ws.values_float ? 1 : 0, list.length, ws.checksum.as<unsigned long long>(), ws.stream
    );
    VB200_CUDA(cudaGetLastError());
    VB200_CUDA(cudaMemcpyAsync(result, ws.checksum.ptr, 4 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, ws.stream));
    VB200_CUDA(cudaStreamSynchronize(ws.stream));
    result[3] = list.length;
}

void free_neighbors(VesinNeighborList& list) {
    if (list.opaque != nullptr) {
        auto* ws = static_cast<Workspace*>(list.opaque);
        int previous = -1;
        cudaGetDevice(&previous);
        cudaSetDevice(ws->device);
        delete ws;
        if (previous >= 0) {
            cudaSetDevice(previous);
        }
        list.opaque = nullptr;
    }
    list.pairs = nullptr;
    list.shifts = nullptr;
    list.distances = nullptr;
    list.vectors = nullptr;
}

} // namespace vb200
