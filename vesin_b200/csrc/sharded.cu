// One periodic system spread over several GPUs, one slab per rank.
//
// A build on a rank: one kernel selects the owned points within the cutoff of
// the two faces of the slab and packs them into two messages; the messages go
// to the two neighbouring ranks with ncclSend / ncclRecv inside one group (NCCL
// over NVLink; what arrives lands in this GPU's own memory before any kernel
// reads it: no peer loads); the local build then bins owned points and received
// records together and writes the pairs of the owned points. Packing and
// exchange run on a stream of their own, so the binning of the owned points
// overlaps with them; the build's stream waits for the messages right before
// it bins them.
//
// The reference has no multi-GPU notion (one system, one device per call,
// vesin/include/vesin.h:103-108): everything here is additive.
//
// NCCL is looked up at run time (dlopen): programs that never build a sharded
// list do not need it, and a program that already loaded NCCL (PyTorch does)
// shares its copy.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <new>
#include <stdexcept>
#include <string>

#include <cuda_runtime.h>
#include <dlfcn.h>

#include "vesin.h"
#include "vesin_b200.h"

#include "engine.hpp"
#include "halo.cuh"
#include "plan.hpp"

namespace {

// ---- the few NCCL declarations this file needs (public NCCL 2.x API) ----
struct NcclUniqueId {
    char internal[128];
};
static_assert(sizeof(NcclUniqueId) == VESIN_B200_UNIQUE_ID_BYTES, "size of ncclUniqueId");
using NcclComm = void*;
constexpr int NCCL_SUCCESS = 0;
constexpr int NCCL_UINT64 = 5;
constexpr int NCCL_FLOAT64 = 8;
constexpr int NCCL_MAX = 2;

struct Nccl {
    void* library = nullptr;
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*Send)(const void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    std::string problem;
};

Nccl load_nccl() {
    Nccl nccl;
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
        nccl.library = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (nccl.library != nullptr) {
            break;
        }
    }
    if (nccl.library == nullptr) {
        nccl.problem = "NCCL (libnccl.so.2) could not be loaded: sharded lists need it";
        return nccl;
    }
    const auto find = [&](const char* symbol) {
        void* address = dlsym(nccl.library, symbol);
        if (address == nullptr && nccl.problem.empty()) {
            nccl.problem = std::string("the NCCL library has no symbol ") + symbol;
        }
        return address;
    };
    nccl.GetUniqueId = reinterpret_cast<decltype(nccl.GetUniqueId)>(find("ncclGetUniqueId"));
    nccl.CommInitRank = reinterpret_cast<decltype(nccl.CommInitRank)>(find("ncclCommInitRank"));
    nccl.CommDestroy = reinterpret_cast<decltype(nccl.CommDestroy)>(find("ncclCommDestroy"));
    nccl.GroupStart = reinterpret_cast<decltype(nccl.GroupStart)>(find("ncclGroupStart"));
    nccl.GroupEnd = reinterpret_cast<decltype(nccl.GroupEnd)>(find("ncclGroupEnd"));
    nccl.Send = reinterpret_cast<decltype(nccl.Send)>(find("ncclSend"));
    nccl.Recv = reinterpret_cast<decltype(nccl.Recv)>(find("ncclRecv"));
    nccl.AllReduce = reinterpret_cast<decltype(nccl.AllReduce)>(find("ncclAllReduce"));
    nccl.GetErrorString = reinterpret_cast<decltype(nccl.GetErrorString)>(find("ncclGetErrorString"));
    return nccl;
}

const Nccl& nccl() {
    static const Nccl instance = load_nccl();
    if (!instance.problem.empty()) {
        throw std::runtime_error(instance.problem);
    }
    return instance;
}

void check_nccl(int status, const char* what) {
    if (status != NCCL_SUCCESS) {
        throw std::runtime_error(std::string("NCCL error in ") + what + ": " + nccl().GetErrorString(status));
    }
}

void check_cuda(cudaError_t status, const char* what) {
    if (status == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        throw std::bad_alloc();
    }
    if (status != cudaSuccess) {
        throw std::runtime_error(std::string("CUDA error in ") + what + ": " + cudaGetErrorString(status));
    }
}

#define SHARDED_CUDA(call) check_cuda((call), #call)

struct CurrentDevice {
    int previous = -1;
    explicit CurrentDevice(int device) {
        SHARDED_CUDA(cudaGetDevice(&previous));
        if (previous != device) {
            SHARDED_CUDA(cudaSetDevice(device));
        } else {
            previous = -1;
        }
    }
    ~CurrentDevice() {
        if (previous >= 0) {
            cudaSetDevice(previous);
        }
    }
};

thread_local std::string SHARDED_ERROR;

/// What the decomposition needs to know about the box.
struct SlabGeometry {
    int axis;
    double inverse_column[3]; // f = x c[0] + y c[1] + z c[2]: fractional coordinate along the cut direction
    double reach;             // fractional thickness of the layer a rank sends to a neighbour
};

SlabGeometry slab_geometry(const double box[9], const bool periodic[3], double cutoff) {
    // the plan of a one-point system: normalised box, inverse and face distances
    const vb200::GridPlan plan = vb200::make_plan(box, periodic, vb200::PointBounds{}, 1, cutoff, true, false, 1);
    int axis = -1;
    // the periodic direction with the largest face distance; on ties the later direction wins
    // (pencils of cells run along the first one)
    for (int k = 2; k >= 0; k--) {
        if (periodic[k] && (axis < 0 || plan.face_dist[k] > plan.face_dist[axis])) {
            axis = k;
        }
    }
    if (axis < 0) {
        throw std::runtime_error("slab decomposition needs at least one periodic direction");
    }
    SlabGeometry geometry;
    geometry.axis = axis;
    for (int c = 0; c < 3; c++) {
        geometry.inverse_column[c] = plan.Hinv[c][axis];
    }
    geometry.reach = cutoff * (1.0 + 1e-9) / plan.face_dist[axis];
    return geometry;
}

} // namespace

struct VesinB200Sharded {
    int rank = 0;
    int world = 1;
    int device = 0;
    NcclComm comm = nullptr;
    cudaStream_t stream = nullptr; // packing and exchange
    cudaEvent_t received = nullptr;
    cudaEvent_t timing[3] = {nullptr, nullptr, nullptr}; // before the packing, between packing and exchange, after the exchange
    double* messages[4] = {nullptr, nullptr, nullptr, nullptr}; // to lower, to upper, from upper, from lower
    size_t capacity = 0;                                        // records per message
    unsigned long long* counts = nullptr;                       // 4 words: scratch of the packing kernel, capacity agreement
    double pack_ms = 0.0;
    double exchange_ms = 0.0;
    bool timed = false;

    ~VesinB200Sharded() {
        int previous = -1;
        cudaGetDevice(&previous);
        cudaSetDevice(device);
        if (stream != nullptr) {
            cudaStreamSynchronize(stream);
        }
        if (comm != nullptr) {
            nccl().CommDestroy(comm);
        }
        for (double* message : messages) {
            if (message != nullptr) {
                cudaFree(message);
            }
        }
        if (counts != nullptr) {
            cudaFree(counts);
        }
        if (received != nullptr) {
            cudaEventDestroy(received);
        }
        for (cudaEvent_t event : timing) {
            if (event != nullptr) {
                cudaEventDestroy(event);
            }
        }
        if (stream != nullptr) {
            cudaStreamDestroy(stream);
        }
        if (previous >= 0) {
            cudaSetDevice(previous);
        }
    }
};

namespace {

void allocate_messages(VesinB200Sharded& sharded, size_t capacity) {
    for (double*& message : sharded.messages) {
        if (message != nullptr) {
            cudaFree(message);
            message = nullptr;
        }
    }
    sharded.capacity = 0;
    for (double*& message : sharded.messages) {
        SHARDED_CUDA(cudaMalloc(reinterpret_cast<void**>(&message), (capacity + 1) * 4 * sizeof(double)));
        // row 0 = "no records" until a message has been packed or received
        SHARDED_CUDA(cudaMemset(message, 0, 4 * sizeof(double)));
    }
    sharded.capacity = capacity;
}

/// The same capacity on every rank: the largest of the ranks' wishes.
void agree_on_capacity(VesinB200Sharded& sharded, size_t wanted) {
    unsigned long long agreed = wanted;
    if (sharded.comm != nullptr) {
        unsigned long long* word = sharded.counts + 3;
        SHARDED_CUDA(cudaMemcpyAsync(word, &agreed, sizeof(agreed), cudaMemcpyHostToDevice, sharded.stream));
        check_nccl(nccl().AllReduce(word, word, 1, NCCL_UINT64, NCCL_MAX, sharded.comm, sharded.stream), "ncclAllReduce");
        SHARDED_CUDA(cudaMemcpyAsync(&agreed, word, sizeof(agreed), cudaMemcpyDeviceToHost, sharded.stream));
        SHARDED_CUDA(cudaStreamSynchronize(sharded.stream));
    }
    allocate_messages(sharded, static_cast<size_t>(agreed));
}

struct Inputs {
    const void* points;
    bool float_io;
    const int64_t* global_index;
    size_t n_owned;
    double box[9];
    bool periodic[3];
};

Inputs gather_inputs(const void* points, bool float_io, const int64_t* global_index, size_t n_owned, const void* box, const bool periodic[3]) {
    if (box == nullptr || periodic == nullptr) {
        throw std::runtime_error("`box` and `periodic` can not be NULL pointers");
    }
    if (n_owned > 0 && (points == nullptr || global_index == nullptr)) {
        throw std::runtime_error("`points` and `global_index` can not be NULL pointers");
    }
    Inputs inputs;
    inputs.points = points;
    inputs.float_io = float_io;
    inputs.global_index = global_index;
    inputs.n_owned = n_owned;
    for (int k = 0; k < 9; k++) {
        inputs.box[k] = float_io ? static_cast<double>(static_cast<const float*>(box)[k]) : static_cast<const double*>(box)[k];
    }
    for (int k = 0; k < 3; k++) {
        inputs.periodic[k] = periodic[k];
    }
    return inputs;
}

void check_on_device(const VesinB200Sharded& sharded, const Inputs& inputs) {
    if (inputs.n_owned == 0) {
        return;
    }
    for (const void* pointer : {inputs.points, static_cast<const void*>(inputs.global_index)}) {
        cudaPointerAttributes attributes;
        if (cudaPointerGetAttributes(&attributes, pointer) != cudaSuccess || attributes.type != cudaMemoryTypeDevice ||
            attributes.device != sharded.device) {
            cudaGetLastError();
            throw std::runtime_error("`points` and `global_index` must be device memory on the device of the sharded list");
        }
    }
}

/// Packs the two outgoing messages on the handle's stream (one launch).
void pack(VesinB200Sharded& sharded, const Inputs& inputs, const SlabGeometry& geometry) {
    const double lower = static_cast<double>(sharded.rank) / sharded.world;
    const double upper = static_cast<double>(sharded.rank + 1) / sharded.world;
    if (sharded.capacity == 0) {
        const double share = geometry.reach * sharded.world; // of the slab's points, if they are spread evenly
        const double wanted = 1.5 * static_cast<double>(inputs.n_owned) * std::min(1.0, share) + 4096.0;
        agree_on_capacity(sharded, static_cast<size_t>(wanted));
    }
    vb200::launch_pack_halo(
        vb200::RealView{inputs.points, inputs.float_io ? 1 : 0}, reinterpret_cast<const long long*>(inputs.global_index), inputs.n_owned,
        geometry.inverse_column, lower, upper, geometry.reach, sharded.messages[0], sharded.messages[1], sharded.capacity, sharded.counts,
        sharded.stream
    );
    SHARDED_CUDA(cudaGetLastError());
}

/// Both messages to the neighbours, theirs into this GPU's memory: one NCCL group.
void exchange(VesinB200Sharded& sharded) {
    const Nccl& api = nccl();
    const int lower_rank = (sharded.rank + sharded.world - 1) % sharded.world;
    const int upper_rank = (sharded.rank + 1) % sharded.world;
    const size_t count = (sharded.capacity + 1) * 4;
    // With two ranks both neighbours are the same peer: operations between two ranks pair up in
    // the order they are issued, so the sends (to lower, to upper) meet the peer's receives
    // (from upper, from lower).
    check_nccl(api.GroupStart(), "ncclGroupStart");
    check_nccl(api.Send(sharded.messages[0], count, NCCL_FLOAT64, lower_rank, sharded.comm, sharded.stream), "ncclSend");
    check_nccl(api.Send(sharded.messages[1], count, NCCL_FLOAT64, upper_rank, sharded.comm, sharded.stream), "ncclSend");
    check_nccl(api.Recv(sharded.messages[2], count, NCCL_FLOAT64, upper_rank, sharded.comm, sharded.stream), "ncclRecv");
    check_nccl(api.Recv(sharded.messages[3], count, NCCL_FLOAT64, lower_rank, sharded.comm, sharded.stream), "ncclRecv");
    check_nccl(api.GroupEnd(), "ncclGroupEnd");
}

void build(
    VesinB200Sharded& sharded, const Inputs& inputs, const SlabGeometry& geometry, bool wait_for_event, VesinOptions options,
    VesinNeighborList& list, std::function<void()> start_exchange = nullptr
) {
    vb200::HaloMessages halo{};
    halo.from_upper = sharded.messages[2];
    halo.from_lower = sharded.messages[3];
    halo.capacity = sharded.capacity;
    halo.received = wait_for_event ? sharded.received : nullptr;
    halo.start_exchange = std::move(start_exchange);
    halo.expected_records = static_cast<size_t>(2.0 * static_cast<double>(inputs.n_owned) * std::min(1.0, geometry.reach * sharded.world));
    const double lower = static_cast<double>(sharded.rank) / sharded.world;
    const double upper = static_cast<double>(sharded.rank + 1) / sharded.world;
    vb200::neighbors_slab_core(
        inputs.points, inputs.float_io, inputs.n_owned, inputs.n_owned, inputs.global_index, &halo, inputs.box, inputs.periodic,
        geometry.axis, lower, upper, options, list
    );
}

void check_options(const VesinOptions& options) {
    if (!std::isfinite(options.cutoff) || options.cutoff <= 0) {
        throw std::runtime_error("cutoff must be a finite, positive number");
    }
    if (options.cutoff <= 1e-6) {
        throw std::runtime_error("cutoff is too small");
    }
}

void prepare_list(const VesinB200Sharded& sharded, VesinNeighborList* list) {
    if (list == nullptr) {
        throw std::runtime_error("`neighbors` can not be a NULL pointer");
    }
    if (list->device.type != VesinUnknownDevice && (list->device.type != VesinCUDA || list->device.device_id != sharded.device)) {
        throw std::runtime_error("`neighbors` was used on another device, free it first");
    }
    list->device = VesinDevice{VesinCUDA, sharded.device};
}

int neighbors_entry(
    VesinB200Sharded* sharded, const void* points, bool float_io, const int64_t* global_index, size_t n_owned, const void* box,
    const bool periodic[3], VesinOptions options, VesinNeighborList* list, const char** error_message
) {
    if (error_message == nullptr) {
        return 1;
    }
    try {
        if (sharded == nullptr) {
            throw std::runtime_error("`sharded` can not be a NULL pointer");
        }
        if (sharded->comm == nullptr) {
            throw std::runtime_error("this sharded list has no communicator: use vesin_b200_sharded_pack / vesin_b200_sharded_build");
        }
        check_options(options);
        prepare_list(*sharded, list);
        const Inputs inputs = gather_inputs(points, float_io, global_index, n_owned, box, periodic);
        const SlabGeometry geometry = slab_geometry(inputs.box, inputs.periodic, options.cutoff);
        CurrentDevice guard(sharded->device);
        check_on_device(*sharded, inputs);
        const bool timed = vb200::profiling_enabled();
        sharded->timed = false;
        // From here to the end of the exchange every rank must make the same NCCL calls:
        // nothing that can fail on one rank alone happens in between.
        if (timed) {
            SHARDED_CUDA(cudaEventRecord(sharded->timing[0], sharded->stream));
        }
        // The local build says when: it queues the sort of the owned points first, so that the
        // host time of the calls below is hidden behind it. Whatever happens in the build, the
        // exchange is queued exactly once on every rank (a rank that fails still takes part).
        bool exchanged = false;
        std::string exchange_error;
        const auto start_exchange = [&]() {
            if (exchanged) {
                return;
            }
            exchanged = true;
            try {
                pack(*sharded, inputs, geometry);
                if (timed) {
                    SHARDED_CUDA(cudaEventRecord(sharded->timing[1], sharded->stream));
                }
                exchange(*sharded);
                SHARDED_CUDA(cudaEventRecord(sharded->received, sharded->stream));
                if (timed) {
                    SHARDED_CUDA(cudaEventRecord(sharded->timing[2], sharded->stream));
                }
            } catch (const std::exception& e) {
                exchange_error = e.what(); // reported after the build has been unwound
            }
        };
        if (sharded->capacity == 0) {
            start_exchange(); // the first call agrees on the capacity (a collective): nothing before it
        }
        try {
            build(*sharded, inputs, geometry, /*wait_for_event=*/true, options, *list, start_exchange);
        } catch (...) {
            start_exchange();
            cudaStreamSynchronize(sharded->stream); // the messages may still be in flight
            throw;
        }
        if (!exchange_error.empty()) {
            cudaStreamSynchronize(sharded->stream);
            throw std::runtime_error(exchange_error);
        }
        if (timed) {
            SHARDED_CUDA(cudaStreamSynchronize(sharded->stream));
            float ms = 0.0f;
            SHARDED_CUDA(cudaEventElapsedTime(&ms, sharded->timing[0], sharded->timing[1]));
            sharded->pack_ms = ms;
            SHARDED_CUDA(cudaEventElapsedTime(&ms, sharded->timing[1], sharded->timing[2]));
            sharded->exchange_ms = ms;
            sharded->timed = true;
        }
    } catch (const std::bad_alloc&) {
        SHARDED_ERROR = "failed to allocate memory";
        *error_message = SHARDED_ERROR.c_str();
        return 1;
    } catch (const std::exception& e) {
        SHARDED_ERROR = e.what();
        *error_message = SHARDED_ERROR.c_str();
        return 1;
    }
    return 0;
}

template <typename Function>
int guarded(const char** error_message, Function&& function) {
    if (error_message == nullptr) {
        return 1;
    }
    try {
        function();
    } catch (const std::bad_alloc&) {
        SHARDED_ERROR = "failed to allocate memory";
        *error_message = SHARDED_ERROR.c_str();
        return 1;
    } catch (const std::exception& e) {
        SHARDED_ERROR = e.what();
        *error_message = SHARDED_ERROR.c_str();
        return 1;
    }
    return 0;
}

} // namespace

extern "C" int vesin_b200_slab_geometry(
    const double box[3][3], const bool periodic[3], double cutoff, int* axis, double inverse_column[3], double* reach,
    const char** error_message
) {
    return guarded(error_message, [&]() {
        if (box == nullptr || periodic == nullptr || axis == nullptr || inverse_column == nullptr || reach == nullptr) {
            throw std::runtime_error("vesin_b200_slab_geometry: NULL pointer argument");
        }
        if (!std::isfinite(cutoff) || cutoff <= 1e-6) {
            throw std::runtime_error("cutoff must be a finite number larger than 1e-6");
        }
        const SlabGeometry geometry = slab_geometry(reinterpret_cast<const double*>(box), periodic, cutoff);
        *axis = geometry.axis;
        for (int c = 0; c < 3; c++) {
            inverse_column[c] = geometry.inverse_column[c];
        }
        *reach = geometry.reach;
    });
}

extern "C" int vesin_b200_sharded_unique_id(unsigned char id[VESIN_B200_UNIQUE_ID_BYTES], const char** error_message) {
    return guarded(error_message, [&]() {
        if (id == nullptr) {
            throw std::runtime_error("`id` can not be a NULL pointer");
        }
        NcclUniqueId unique;
        check_nccl(nccl().GetUniqueId(&unique), "ncclGetUniqueId");
        std::memcpy(id, unique.internal, sizeof(unique.internal));
    });
}

extern "C" int vesin_b200_sharded_create(
    const unsigned char* id, int rank, int world_size, int device_id, VesinB200Sharded** sharded, const char** error_message
) {
    return guarded(error_message, [&]() {
        if (sharded == nullptr) {
            throw std::runtime_error("`sharded` can not be a NULL pointer");
        }
        *sharded = nullptr;
        if (world_size < 2 || rank < 0 || rank >= world_size) {
            throw std::runtime_error("a sharded list needs at least two ranks and 0 <= rank < world_size");
        }
        int device_count = 0;
        if (cudaGetDeviceCount(&device_count) != cudaSuccess || device_id < 0 || device_id >= device_count) {
            cudaGetLastError();
            throw std::runtime_error("device_id does not name a CUDA device of this process");
        }
        CurrentDevice guard(device_id);
        auto* created = new VesinB200Sharded();
        try {
            created->rank = rank;
            created->world = world_size;
            created->device = device_id;
            // blocking stream: ordered after what the caller queued on the legacy default stream
            SHARDED_CUDA(cudaStreamCreate(&created->stream));
            SHARDED_CUDA(cudaEventCreateWithFlags(&created->received, cudaEventDisableTiming));
            for (cudaEvent_t& event : created->timing) {
                SHARDED_CUDA(cudaEventCreate(&event));
            }
            SHARDED_CUDA(cudaMalloc(reinterpret_cast<void**>(&created->counts), 4 * sizeof(unsigned long long)));
            SHARDED_CUDA(cudaMemset(created->counts, 0, 4 * sizeof(unsigned long long)));
            if (id != nullptr) {
                NcclUniqueId unique;
                std::memcpy(unique.internal, id, sizeof(unique.internal));
                check_nccl(nccl().CommInitRank(&created->comm, world_size, unique, rank), "ncclCommInitRank");
            }
        } catch (...) {
            delete created;
            throw;
        }
        *sharded = created;
    });
}

extern "C" void vesin_b200_sharded_free(VesinB200Sharded* sharded) {
    delete sharded;
}

extern "C" int vesin_b200_sharded_set_halo_capacity(VesinB200Sharded* sharded, size_t records, const char** error_message) {
    return guarded(error_message, [&]() {
        if (sharded == nullptr) {
            throw std::runtime_error("`sharded` can not be a NULL pointer");
        }
        if (records == 0 || records >= (1ull << 30)) {
            throw std::runtime_error("the halo capacity must be positive and below 2^30 records");
        }
        CurrentDevice guard(sharded->device);
        SHARDED_CUDA(cudaStreamSynchronize(sharded->stream));
        allocate_messages(*sharded, records);
    });
}

extern "C" int vesin_b200_sharded_neighbors(
    VesinB200Sharded* sharded,
    const double (*points)[3],
    const int64_t* global_index,
    size_t n_owned,
    const double box[3][3],
    const bool periodic[3],
    VesinOptions options,
    VesinNeighborList* neighbors,
    const char** error_message
) {
    return neighbors_entry(sharded, points, false, global_index, n_owned, box, periodic, options, neighbors, error_message);
}

extern "C" int vesin_b200_sharded_neighbors_f32(
    VesinB200Sharded* sharded,
    const float (*points)[3],
    const int64_t* global_index,
    size_t n_owned,
    const float box[3][3],
    const bool periodic[3],
    VesinOptions options,
    VesinNeighborList* neighbors,
    const char** error_message
) {
    return neighbors_entry(sharded, points, true, global_index, n_owned, box, periodic, options, neighbors, error_message);
}

extern "C" int vesin_b200_sharded_pack(
    VesinB200Sharded* sharded,
    const double (*points)[3],
    const int64_t* global_index,
    size_t n_owned,
    const double box[3][3],
    const bool periodic[3],
    double cutoff,
    double* messages[4],
    size_t* rows,
    const char** error_message
) {
    return guarded(error_message, [&]() {
        if (sharded == nullptr || messages == nullptr || rows == nullptr) {
            throw std::runtime_error("vesin_b200_sharded_pack: NULL pointer argument");
        }
        if (!std::isfinite(cutoff) || cutoff <= 1e-6) {
            throw std::runtime_error("cutoff must be a finite number larger than 1e-6");
        }
        const Inputs inputs = gather_inputs(points, false, global_index, n_owned, box, periodic);
        const SlabGeometry geometry = slab_geometry(inputs.box, inputs.periodic, cutoff);
        CurrentDevice guard(sharded->device);
        check_on_device(*sharded, inputs);
        pack(*sharded, inputs, geometry);
        SHARDED_CUDA(cudaStreamSynchronize(sharded->stream));
        for (int k = 0; k < 4; k++) {
            messages[k] = sharded->messages[k];
        }
        *rows = sharded->capacity + 1;
    });
}

extern "C" int vesin_b200_sharded_build(
    VesinB200Sharded* sharded,
    const double (*points)[3],
    const int64_t* global_index,
    size_t n_owned,
    const double box[3][3],
    const bool periodic[3],
    VesinOptions options,
    VesinNeighborList* neighbors,
    const char** error_message
) {
    return guarded(error_message, [&]() {
        if (sharded == nullptr) {
            throw std::runtime_error("`sharded` can not be a NULL pointer");
        }
        if (sharded->capacity == 0) {
            throw std::runtime_error("no halo messages yet: call vesin_b200_sharded_pack first");
        }
        check_options(options);
        prepare_list(*sharded, neighbors);
        const Inputs inputs = gather_inputs(points, false, global_index, n_owned, box, periodic);
        const SlabGeometry geometry = slab_geometry(inputs.box, inputs.periodic, options.cutoff);
        CurrentDevice guard(sharded->device);
        check_on_device(*sharded, inputs);
        build(*sharded, inputs, geometry, /*wait_for_event=*/false, options, *neighbors);
    });
}

extern "C" int vesin_b200_sharded_stage_times(const VesinB200Sharded* sharded, double* pack_ms, double* exchange_ms) {
    if (sharded == nullptr || pack_ms == nullptr || exchange_ms == nullptr || !sharded->timed) {
        return 1;
    }
    *pack_ms = sharded->pack_ms;
    *exchange_ms = sharded->exchange_ms;
    return 0;
}
