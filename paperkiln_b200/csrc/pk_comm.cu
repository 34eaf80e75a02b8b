// Collective group of the C ABI: a sum all-reduce of fp32 gradient ranges between the ranks of a
// data-parallel job, issued asynchronously behind the compute stream so that the transfer of one
// transformer block's gradients overlaps the recompute + backward of the next block.
//
// Two backends behind one handle:
//   NCCL   one communicator per process (one process per GPU), a private communication stream,
//          ncclAllReduce in place. The library is opened at run time (libnccl.so.2: the copy the
//          process has already loaded, else the system's), so libpk itself has no link-time
//          dependency on it. Failure detection: ncclCommGetAsyncError is polled wherever the host
//          waits, a host-side time limit bounds every wait, and both lead to ncclCommAbort and a
//          PK_ERR_COMM / PK_ERR_TIMEOUT status -- never a hang, never a device trap.
//   file   CPU ranks exchanging host buffers through a directory (one file per rank and
//          collective, summed in ascending rank order; the files are left for the caller to
//          remove with the directory). It exists to exercise the host-side protocol -- ordering,
//          time limit, abort, use after abort -- without GPUs: a rank that is late is waited
//          for, a rank that never joins runs the others into their limit.
// The reference has no multi-GPU path; its nearest relative is gradient accumulation
// (tools/mtstudio.cpp:456-474), the same sum-of-scaled-gradients identity.
#include <dlfcn.h>
#include <nccl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "pk_common.cuh"

namespace pk {
namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int*) = nullptr;
};

NcclApi* nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h) {
            api.handle = h;
            api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
            api.CommInitRankConfig = reinterpret_cast<decltype(api.CommInitRankConfig)>(dlsym(h, "ncclCommInitRankConfig"));
            api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
            api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(dlsym(h, "ncclCommGetAsyncError"));
            api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(dlsym(h, "ncclCommAbort"));
            api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
            api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
            api.GetVersion = reinterpret_cast<decltype(api.GetVersion)>(dlsym(h, "ncclGetVersion"));
        }
    }
    const bool ok = api.handle && api.GetUniqueId && api.CommInitRankConfig && api.AllReduce && api.CommGetAsyncError &&
                    api.CommAbort && api.CommDestroy && api.GetErrorString;
    return ok ? &api : nullptr;
}

enum Backend { BACKEND_NCCL = 0, BACKEND_FILE = 1 };

struct Comm {
    int backend = BACKEND_NCCL;
    int rank = 0, world = 1;
    double timeout_s = 30.0;
    bool dead = false;             // aborted: every later call fails with PK_ERR_COMM
    int64_t launched = 0;          // collectives started so far
    // NCCL
    ncclComm_t nccl = nullptr;
    cudaStream_t stream = nullptr; // communication stream
    cudaEvent_t ev_ready = nullptr, ev_done = nullptr;
    bool pending = false;
    // file backend
    std::string dir;
    struct Pending {
        float* buf;
        int64_t count;
        int64_t seq;
    };
    std::vector<Pending> waiting;
};

double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

#define PK_NCCL(comm_expr)                                                                   \
    do {                                                                                     \
        ncclResult_t _r = (comm_expr);                                                       \
        if (_r != ncclSuccess && _r != ncclInProgress) {                                     \
            set_error("%s failed: %s", #comm_expr, nccl_api()->GetErrorString(_r));          \
            return PK_ERR_COMM;                                                              \
        }                                                                                    \
    } while (0)

int abort_comm(Comm* c) {
    if (c->dead) return PK_OK;
    c->dead = true;
    if (c->backend == BACKEND_NCCL && c->nccl) {
        NcclApi* api = nccl_api();
        if (api) api->CommAbort(c->nccl);   // frees the communicator and ends its kernels
        c->nccl = nullptr;
    }
    c->waiting.clear();
    return PK_OK;
}

// ---- file backend --------------------------------------------------------------------------
std::string part_path(const Comm* c, int64_t seq, int rank) {
    return c->dir + "/ar." + std::to_string(seq) + "." + std::to_string(rank);
}

int file_publish(Comm* c, const float* buf, int64_t count, int64_t seq) {
    const std::string path = part_path(c, seq, c->rank), tmp = path + ".tmp";
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if (!f) {
        set_error("pk_comm (file backend): cannot write %s", tmp.c_str());
        return PK_ERR_COMM;
    }
    const size_t n = std::fwrite(buf, sizeof(float), static_cast<size_t>(count), f);
    std::fclose(f);
    if (n != static_cast<size_t>(count) || std::rename(tmp.c_str(), path.c_str()) != 0) {
        set_error("pk_comm (file backend): cannot publish %s", path.c_str());
        return PK_ERR_COMM;
    }
    return PK_OK;
}

// Waits for every rank's part of collective `seq`, then sums them in ascending rank order.
int file_complete(Comm* c, float* buf, int64_t count, int64_t seq, double deadline) {
    std::vector<float> part(static_cast<size_t>(count)), acc(static_cast<size_t>(count), 0.0f);
    for (int r = 0; r < c->world; ++r) {
        const std::string path = part_path(c, seq, r);
        struct stat sb;
        while (stat(path.c_str(), &sb) != 0 || sb.st_size != static_cast<off_t>(count * sizeof(float))) {
            if (now_s() > deadline) {
                set_error("pk_comm_wait: rank %d did not join collective %lld within %.1f s", r, static_cast<long long>(seq),
                          c->timeout_s);
                return PK_ERR_TIMEOUT;
            }
            std::this_thread::sleep_for(std::chrono::milliseconds(1));
        }
        FILE* f = std::fopen(path.c_str(), "rb");
        const size_t n = f ? std::fread(part.data(), sizeof(float), static_cast<size_t>(count), f) : 0;
        if (f) std::fclose(f);
        if (n != static_cast<size_t>(count)) {
            set_error("pk_comm (file backend): short read of %s", path.c_str());
            return PK_ERR_COMM;
        }
        for (int64_t i = 0; i < count; ++i) acc[i] += part[i];
    }
    std::memcpy(buf, acc.data(), static_cast<size_t>(count) * sizeof(float));
    return PK_OK;   // the parts stay in the directory: another rank may not have read them yet
}

}  // namespace
}  // namespace pk

using namespace pk;

extern "C" {

int pk_comm_unique_id(void* id_h, size_t cap) {
    PK_REQUIRE(id_h != nullptr && cap >= sizeof(ncclUniqueId), "id buffer must hold 128 bytes");
    NcclApi* api = nccl_api();
    if (!api) {
        set_error("pk_comm_unique_id: libnccl.so.2 could not be opened");
        return PK_ERR_COMM;
    }
    ncclUniqueId id;
    PK_NCCL(api->GetUniqueId(&id));
    std::memcpy(id_h, &id, sizeof(id));
    return PK_OK;
}

int pk_comm_init(const void* id_h, int rank, int world, int max_ctas, void** comm_h) {
    PK_REQUIRE(id_h != nullptr && comm_h != nullptr, "null argument");
    PK_REQUIRE(world >= 1 && rank >= 0 && rank < world, "bad rank / world");
    *comm_h = nullptr;
    NcclApi* api = nccl_api();
    if (!api) {
        set_error("pk_comm_init: libnccl.so.2 could not be opened");
        return PK_ERR_COMM;
    }
    Comm* c = new Comm();
    c->backend = BACKEND_NCCL;
    c->rank = rank;
    c->world = world;
    ncclUniqueId id;
    std::memcpy(&id, id_h, sizeof(id));
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 1;
    if (max_ctas > 0) cfg.maxCTAs = max_ctas;   // fewer SMs taken from the kernels the transfer overlaps
    ncclResult_t r = api->CommInitRankConfig(&c->nccl, world, id, rank, &cfg);
    if (r != ncclSuccess) {
        set_error("ncclCommInitRankConfig failed: %s", api->GetErrorString(r));
        delete c;
        return PK_ERR_COMM;
    }
    cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_ready, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_done, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        set_error("pk_comm_init: %s", cudaGetErrorString(e));
        api->CommAbort(c->nccl);
        delete c;
        return PK_ERR_CUDA;
    }
    *comm_h = c;
    return PK_OK;
}

int pk_comm_init_file(const char* dir, int rank, int world, void** comm_h) {
    PK_REQUIRE(dir != nullptr && comm_h != nullptr, "null argument");
    PK_REQUIRE(world >= 1 && rank >= 0 && rank < world, "bad rank / world");
    struct stat sb;
    PK_REQUIRE(stat(dir, &sb) == 0 && S_ISDIR(sb.st_mode), "the exchange directory does not exist");
    Comm* c = new Comm();
    c->backend = BACKEND_FILE;
    c->rank = rank;
    c->world = world;
    c->dir = dir;
    *comm_h = c;
    return PK_OK;
}

int pk_comm_set_timeout(void* comm, double seconds) {
    PK_REQUIRE(comm != nullptr && seconds > 0.0, "bad argument");
    static_cast<Comm*>(comm)->timeout_s = seconds;
    return PK_OK;
}

int pk_comm_info(void* comm, int* rank_h, int* world_h, int* backend_h, int* alive_h) {
    PK_REQUIRE(comm != nullptr, "null communicator");
    Comm* c = static_cast<Comm*>(comm);
    if (rank_h) *rank_h = c->rank;
    if (world_h) *world_h = c->world;
    if (backend_h) *backend_h = c->backend;
    if (alive_h) *alive_h = c->dead ? 0 : 1;
    return PK_OK;
}

int pk_allreduce_async(void* comm, float* buf, int64_t count, void* compute_stream) {
    PK_REQUIRE(comm != nullptr, "null communicator");
    Comm* c = static_cast<Comm*>(comm);
    if (c->dead) {
        set_error("pk_allreduce_async: the communicator was aborted");
        return PK_ERR_COMM;
    }
    PK_REQUIRE(count >= 0 && (count == 0 || buf != nullptr), "bad buffer");
    if (count == 0) return PK_OK;
    if (c->backend == BACKEND_FILE) {
        const int64_t seq = c->launched++;
        const int rc = file_publish(c, buf, count, seq);
        if (rc != PK_OK) {
            abort_comm(c);
            return rc;
        }
        c->waiting.push_back({buf, count, seq});
        return PK_OK;
    }
    NcclApi* api = nccl_api();
    // the transfer starts once everything enqueued so far on the compute stream (the kernels that
    // produced buf) has finished, and not before
    PK_CHECK_CUDA(cudaEventRecord(c->ev_ready, as_stream(compute_stream)));
    PK_CHECK_CUDA(cudaStreamWaitEvent(c->stream, c->ev_ready, 0));
    ncclResult_t r = api->AllReduce(buf, buf, static_cast<size_t>(count), ncclFloat, ncclSum, c->nccl, c->stream);
    if (r != ncclSuccess) {
        set_error("ncclAllReduce failed: %s", api->GetErrorString(r));
        abort_comm(c);
        return PK_ERR_COMM;
    }
    ++c->launched;
    c->pending = true;
    return PK_OK;
}

// Orders the compute stream behind every collective started so far (no host block) and checks
// the communicator for an asynchronous error. File backend: completes the collectives (host).
int pk_comm_wait(void* comm, void* compute_stream) {
    PK_REQUIRE(comm != nullptr, "null communicator");
    Comm* c = static_cast<Comm*>(comm);
    if (c->dead) {
        set_error("pk_comm_wait: the communicator was aborted");
        return PK_ERR_COMM;
    }
    if (c->backend == BACKEND_FILE) {
        const double deadline = now_s() + c->timeout_s;
        for (const Comm::Pending& p : c->waiting) {
            const int rc = file_complete(c, p.buf, p.count, p.seq, deadline);
            if (rc != PK_OK) {
                abort_comm(c);
                return rc;
            }
        }
        c->waiting.clear();
        return PK_OK;
    }
    if (!c->pending) return PK_OK;
    PK_CHECK_CUDA(cudaEventRecord(c->ev_done, c->stream));
    PK_CHECK_CUDA(cudaStreamWaitEvent(as_stream(compute_stream), c->ev_done, 0));
    ncclResult_t async = ncclSuccess;
    PK_NCCL(nccl_api()->CommGetAsyncError(c->nccl, &async));
    if (async != ncclSuccess && async != ncclInProgress) {
        set_error("pk_comm_wait: the communicator reports %s", nccl_api()->GetErrorString(async));
        abort_comm(c);
        return PK_ERR_COMM;
    }
    return PK_OK;
}

// Host-blocking form: returns when every collective started so far has finished on the device,
// polling the communicator's asynchronous error state; gives up after the time limit
// (pk_comm_set_timeout, default 30 s), aborts the communicator and returns PK_ERR_TIMEOUT.
int pk_comm_wait_host(void* comm) {
    PK_REQUIRE(comm != nullptr, "null communicator");
    Comm* c = static_cast<Comm*>(comm);
    if (c->dead) {
        set_error("pk_comm_wait_host: the communicator was aborted");
        return PK_ERR_COMM;
    }
    if (c->backend == BACKEND_FILE) return pk_comm_wait(comm, nullptr);
    if (!c->pending) return PK_OK;
    PK_CHECK_CUDA(cudaEventRecord(c->ev_done, c->stream));
    const double deadline = now_s() + c->timeout_s;
    for (;;) {
        const cudaError_t q = cudaEventQuery(c->ev_done);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady) {
            set_error("pk_comm_wait_host: %s", cudaGetErrorString(q));
            abort_comm(c);
            return PK_ERR_CUDA;
        }
        ncclResult_t async = ncclSuccess;
        nccl_api()->CommGetAsyncError(c->nccl, &async);
        if (async != ncclSuccess && async != ncclInProgress) {
            set_error("pk_comm_wait_host: the communicator reports %s", nccl_api()->GetErrorString(async));
            abort_comm(c);
            return PK_ERR_COMM;
        }
        if (now_s() > deadline) {
            set_error("pk_comm_wait_host: collectives still running after %.1f s; communicator aborted", c->timeout_s);
            abort_comm(c);
            return PK_ERR_TIMEOUT;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    c->pending = false;
    return PK_OK;
}

int pk_comm_abort(void* comm) {
    PK_REQUIRE(comm != nullptr, "null communicator");
    return abort_comm(static_cast<Comm*>(comm));
}

int pk_comm_destroy(void* comm) {
    if (!comm) return PK_OK;
    Comm* c = static_cast<Comm*>(comm);
    if (c->backend == BACKEND_NCCL) {
        if (c->nccl && !c->dead) {
            if (c->stream) cudaStreamSynchronize(c->stream);
            NcclApi* api = nccl_api();
            if (api) api->CommDestroy(c->nccl);
        }
        if (c->ev_ready) cudaEventDestroy(c->ev_ready);
        if (c->ev_done) cudaEventDestroy(c->ev_done);
        if (c->stream) cudaStreamDestroy(c->stream);
    }
    delete c;
    return PK_OK;
}

}  // extern "C"
