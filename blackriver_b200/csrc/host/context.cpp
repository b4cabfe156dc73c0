#include "context.hpp"

#include <sys/stat.h>
#include <unistd.h>
#include <ctime>

#include <unistd.h>

#include <chrono>
#include <cstring>
#include <fstream>
#include <map>
#include <vector>
#include <thread>

namespace br {

int ComputingContext::cuda_device = -1;
cudaStream_t ComputingContext::cuda_stream = nullptr;
cudaStream_t ComputingContext::comm_stream = nullptr;
cudaEvent_t ComputingContext::compute_done = nullptr;
cudaEvent_t ComputingContext::comm_done = nullptr;
void* ComputingContext::cuda_workspace = nullptr;
void* ComputingContext::local_workspace = nullptr;
size_t ComputingContext::workspace_size = 0;
int ComputingContext::grad_accumulate = 0;
float ComputingContext::loss_scale = 1.0f;
int ComputingContext::verbose = 1;
bool ComputingContext::booted = false;
static bool g_owns_compute_stream = false;

static void boot_common(int device, size_t workspace_bytes) {
    // training switches start from their defaults on every boot (a previous user of the process may have set them)
    ComputingContext::grad_accumulate = 0;
    ComputingContext::loss_scale = 1.0f;
    ComputingContext::verbose = 1;
    ComputingContext::cuda_device = device;
    BR_CUDA_CHECK(cudaStreamCreateWithFlags(&ComputingContext::comm_stream, cudaStreamNonBlocking));
    BR_CUDA_CHECK(cudaEventCreateWithFlags(&ComputingContext::compute_done, cudaEventDisableTiming));
    BR_CUDA_CHECK(cudaEventCreateWithFlags(&ComputingContext::comm_done, cudaEventDisableTiming));
    ComputingContext::workspace_size = workspace_bytes;
    BR_CUDA_CHECK(cudaMalloc(&ComputingContext::cuda_workspace, workspace_bytes));
    BR_CUDA_CHECK(cudaMallocHost(&ComputingContext::local_workspace, workspace_bytes));
    ComputingContext::booted = true;
}

void ComputingContext::boot(int device, size_t workspace_bytes) {
    br_assert(!booted, "ComputingContext booted twice");
    BR_CUDA_CHECK(cudaSetDevice(device));
    BR_CUDA_CHECK(cudaStreamCreateWithFlags(&cuda_stream, cudaStreamNonBlocking));
    g_owns_compute_stream = true;
    boot_common(device, workspace_bytes);
}

void ComputingContext::boot_with_stream(int device, cudaStream_t compute, size_t workspace_bytes) {
    br_assert(!booted, "ComputingContext booted twice");
    BR_CUDA_CHECK(cudaSetDevice(device));
    cuda_stream = compute;
    g_owns_compute_stream = false;
    boot_common(device, workspace_bytes);
}

void ComputingContext::shutdown() {
    if (!booted) return;
    cudaStreamSynchronize(cuda_stream);
    cudaStreamSynchronize(comm_stream);
    cudaFree(cuda_workspace);
    cudaFreeHost(local_workspace);
    cudaEventDestroy(compute_done);
    cudaEventDestroy(comm_done);
    cudaStreamDestroy(comm_stream);
    if (g_owns_compute_stream) cudaStreamDestroy(cuda_stream);
    cuda_workspace = local_workspace = nullptr;
    cuda_stream = comm_stream = nullptr;
    workspace_size = 0;
    booted = false;
}

// ------------------------------------------------------------------------------------------
bool Profiler::enabled = false;
namespace {
struct ProfRec {
    const char* family;
    cudaEvent_t e0, e1;
};
std::vector<ProfRec> g_prof;
std::vector<cudaEvent_t> g_prof_pool;
cudaEvent_t prof_event() {
    if (!g_prof_pool.empty()) {
        cudaEvent_t e = g_prof_pool.back();
        g_prof_pool.pop_back();
        return e;
    }
    cudaEvent_t e;
    BR_CUDA_CHECK(cudaEventCreate(&e));
    return e;
}
}  // namespace

void Profiler::start() {
    for (auto& r : g_prof) {
        g_prof_pool.push_back(r.e0);
        g_prof_pool.push_back(r.e1);
    }
    g_prof.clear();
    enabled = true;
}

void Profiler::begin(const char* family) {
    if (!enabled) return;
    ProfRec r{family, prof_event(), prof_event()};
    BR_CUDA_CHECK(cudaEventRecord(r.e0, ComputingContext::cuda_stream));
    g_prof.push_back(r);
}

void Profiler::end() {
    if (!enabled || g_prof.empty()) return;
    BR_CUDA_CHECK(cudaEventRecord(g_prof.back().e1, ComputingContext::cuda_stream));
}

std::string Profiler::report_json() {
    enabled = false;
    if (ComputingContext::booted) BR_CUDA_CHECK(cudaStreamSynchronize(ComputingContext::cuda_stream));
    std::map<std::string, std::pair<double, long>> agg;
    for (auto& r : g_prof) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, r.e0, r.e1) == cudaSuccess) {
            auto& a = agg[r.family];
            a.first += ms;
            a.second += 1;
        }
    }
    std::ostringstream ss;
    ss << "{";
    bool first = true;
    for (auto& kv : agg) {
        if (!first) ss << ", ";
        first = false;
        ss << "\"" << kv.first << "\": {\"ms\": " << kv.second.first << ", \"calls\": " << kv.second.second << "}";
    }
    ss << "}";
    return ss.str();
}

// ------------------------------------------------------------------------------------------
int CollectiveContext::mpi_world = 1;
int CollectiveContext::mpi_rank = 0;
int CollectiveContext::nccl_world = 1;
int CollectiveContext::nccl_rank = 0;
ncclComm_t CollectiveContext::nccl_comm = nullptr;
ncclUniqueId CollectiveContext::nccl_id;
bool CollectiveContext::has_comm = false;
static std::chrono::steady_clock::time_point g_boot_time = std::chrono::steady_clock::now();

void CollectiveContext::boot_local(int rank, int world) {
    br_assert(world >= 1 && rank >= 0 && rank < world, "bad rank layout");
    mpi_rank = nccl_rank = rank;
    mpi_world = nccl_world = world;
    g_boot_time = std::chrono::steady_clock::now();
}

ncclUniqueId CollectiveContext::make_unique_id() {
    ncclUniqueId id;
    BR_NCCL_CHECK(ncclGetUniqueId(&id));
    return id;
}

void CollectiveContext::boot(int rank, int world, const ncclUniqueId& id) {
    boot_local(rank, world);
    nccl_id = id;
    if (world > 1) {
        BR_NCCL_CHECK(ncclCommInitRank(&nccl_comm, world, id, rank));
        has_comm = true;
    }
}

void CollectiveContext::boot_from_file(int rank, int world, const std::string& path, int timeout_s) {
    if (world == 1) {
        boot_local(rank, world);
        return;
    }
    ncclUniqueId id;
    if (rank == 0) {
        id = make_unique_id();
        std::string tmp = path + ".tmp";
        {
            std::ofstream out(tmp, std::ios::binary);
            out.write(reinterpret_cast<const char*>(&id), sizeof(id));
        }
        br_assert(::rename(tmp.c_str(), path.c_str()) == 0, "can't publish the NCCL id file");
    } else {
        // a file left behind by an earlier job under the same name must not be taken for this job's id:
        // only a file written since shortly before this rank started counts (the ranks of a job start together)
        const time_t not_before = ::time(nullptr) - 30;
        bool got = false;
        for (int i = 0; i < timeout_s * 20 && !got; i++) {
            struct stat st;
            if (::stat(path.c_str(), &st) == 0 && st.st_mtime >= not_before) {
                std::ifstream in(path, std::ios::binary);
                if (in && in.read(reinterpret_cast<char*>(&id), sizeof(id))) got = true;
            }
            if (!got) std::this_thread::sleep_for(std::chrono::milliseconds(50));
        }
        br_assert(got, "timed out waiting for the NCCL id file");
    }
    boot(rank, world, id);
    // every rank has read the id once the communicator exists: the publisher takes the file away again
    if (rank == 0) ::unlink(path.c_str());
}

void CollectiveContext::shutdown() {
    if (has_comm) {
        ncclCommDestroy(nccl_comm);
        has_comm = false;
        nccl_comm = nullptr;
    }
}

int CollectiveContext::now() {
    auto d = std::chrono::steady_clock::now() - g_boot_time;
    return (int)std::chrono::duration_cast<std::chrono::seconds>(d).count();
}

// ------------------------------------------------------------------------------------------
const size_t MemoryContext::page_size = 4096;
void* MemoryContext::root = nullptr;
size_t MemoryContext::total_size = 0;
size_t MemoryContext::currentp = 0;
bool MemoryContext::pinned = false;

void MemoryContext::boot(size_t total_bytes, bool pin) {
    br_assert(root == nullptr, "MemoryContext booted twice");
    total_size = (total_bytes + page_size - 1) / page_size * page_size;
    pinned = pin;
    if (pin) {
        BR_CUDA_CHECK(cudaMallocHost(&root, total_size));
    } else {
        root = ::aligned_alloc(page_size, total_size);
        br_assert(root != nullptr, "host arena allocation failed");
    }
    currentp = 0;
}

void* MemoryContext::alloc(size_t bytes) {
    br_assert(root != nullptr, "MemoryContext is not booted");
    size_t need = (bytes + page_size - 1) / page_size * page_size;
    if (need + currentp > total_size) {
        std::cerr << CollectiveContext::mpi_rank << ": arena used " << currentp << ", asked " << need << std::endl;
        br_panic("host arena exhausted");
    }
    void* p = static_cast<unsigned char*>(root) + currentp;
    currentp += need;
    return p;
}

void MemoryContext::shutdown() {
    if (!root) return;
    if (pinned) cudaFreeHost(root);
    else ::free(root);
    root = nullptr;
    total_size = currentp = 0;
}

}  // namespace br
