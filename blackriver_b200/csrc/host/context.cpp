#include "context.hpp"

#include <cuda.h>
#include <sys/stat.h>
#include <unistd.h>
#include <ctime>

#include "brk.h"

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
cudaStream_t ComputingContext::link_stream[2] = {nullptr, nullptr};
cudaEvent_t ComputingContext::compute_done = nullptr;
cudaEvent_t ComputingContext::comm_done = nullptr;
cudaStream_t ComputingContext::main_stream = nullptr;
std::vector<cudaEvent_t> ComputingContext::marks;
std::vector<char> ComputingContext::mark_set;
void* ComputingContext::cuda_workspace = nullptr;
void* ComputingContext::local_workspace = nullptr;
size_t ComputingContext::workspace_size = 0;
int ComputingContext::grad_accumulate = 0;
float ComputingContext::loss_scale = 1.0f;
int ComputingContext::verbose = 1;
int ComputingContext::nccl_on_comm_stream = 0;
bool ComputingContext::booted = false;
static bool g_owns_compute_stream = false;

static void boot_common(int device, size_t workspace_bytes) {
    // training switches start from their defaults on every boot (a previous user of the process may have set them)
    ComputingContext::grad_accumulate = 0;
    ComputingContext::loss_scale = 1.0f;
    ComputingContext::verbose = 1;
    ComputingContext::nccl_on_comm_stream = 0;
    ComputingContext::cuda_device = device;
    BR_CUDA_CHECK(cudaStreamCreateWithFlags(&ComputingContext::comm_stream, cudaStreamNonBlocking));
    for (int d = 0; d < 2; d++) BR_CUDA_CHECK(cudaStreamCreateWithFlags(&ComputingContext::link_stream[d], cudaStreamNonBlocking));
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
    while (PipeLinks::is_open) PipeLinks::close();
    for (int d = 0; d < 2; d++) {
        cudaStreamSynchronize(link_stream[d]);
        cudaStreamDestroy(link_stream[d]);
        link_stream[d] = nullptr;
    }
    cudaFree(cuda_workspace);
    cudaFreeHost(local_workspace);
    if (main_stream) {      // left in side mode by an interrupted script
        cuda_stream = main_stream;
        main_stream = nullptr;
    }
    for (cudaEvent_t e : marks) cudaEventDestroy(e);
    marks.clear();
    mark_set.clear();
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
    if (ComputingContext::booted) {
        BR_CUDA_CHECK(cudaStreamSynchronize(ComputingContext::cuda_stream));
        BR_CUDA_CHECK(cudaStreamSynchronize(ComputingContext::comm_stream));      // operators queued in side mode
    }
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
int CollectiveContext::dp_world = 1;
int CollectiveContext::dp_rank = 0;
ncclComm_t CollectiveContext::dp_comm = nullptr;
ncclComm_t CollectiveContext::job_comm = nullptr;
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

// The id file carries a job nonce in front of the 128 id bytes, so that a rank of a relaunched job can never take a
// file left by an earlier job under the same name for its own: the nonce is what the launcher gives every rank of one
// job alike (TORCHELASTIC_RUN_ID, else MASTER_PORT, else empty).
static std::string job_nonce() {
    for (const char* name : {"BR_JOB_ID", "TORCHELASTIC_RUN_ID", "MASTER_PORT"}) {
        const char* v = ::getenv(name);
        if (v && *v) return std::string(name) + "=" + v;
    }
    return "";
}

void CollectiveContext::boot_from_file(int rank, int world, const std::string& path, int timeout_s) {
    if (world == 1) {
        boot_local(rank, world);
        return;
    }
    ncclUniqueId id;
    char nonce[64] = {0};
    std::snprintf(nonce, sizeof(nonce), "%s", job_nonce().c_str());
    if (rank == 0) {
        ::unlink(path.c_str());          // whatever an earlier job left behind
        id = make_unique_id();
        std::string tmp = path + ".tmp";
        {
            std::ofstream out(tmp, std::ios::binary);
            out.write(nonce, sizeof(nonce));
            out.write(reinterpret_cast<const char*>(&id), sizeof(id));
        }
        br_assert(::rename(tmp.c_str(), path.c_str()) == 0, "can't publish the NCCL id file");
    } else {
        // only a file with this job's nonce, written since shortly before this rank started, counts
        const time_t not_before = ::time(nullptr) - 30;
        bool got = false;
        for (int i = 0; i < timeout_s * 20 && !got; i++) {
            struct stat st;
            if (::stat(path.c_str(), &st) == 0 && st.st_mtime >= not_before) {
                std::ifstream in(path, std::ios::binary);
                char seen[64];
                if (in && in.read(seen, sizeof(seen)) && std::memcmp(seen, nonce, sizeof(nonce)) == 0 &&
                    in.read(reinterpret_cast<char*>(&id), sizeof(id)))
                    got = true;
            }
            if (!got) std::this_thread::sleep_for(std::chrono::milliseconds(50));
        }
        br_assert(got, "timed out waiting for the NCCL id file");
    }
    boot(rank, world, id);
    // every rank has read the id once the communicator exists: the publisher takes the file away again
    if (rank == 0) ::unlink(path.c_str());
}

void CollectiveContext::split_replicas(int replicas) {
    br_assert(job_comm == nullptr, "the job is split into replicas already");
    br_assert(replicas >= 1 && mpi_world % replicas == 0, "the number of ranks is not a multiple of the replicas");
    if (replicas == 1) return;
    br_assert(has_comm, "split_replicas needs the job's communicator");
    const int stages = mpi_world / replicas;
    const int replica = mpi_rank / stages, stage = mpi_rank % stages;
    ncclComm_t pipe = nullptr, dp = nullptr;
    // every rank takes part in both splits; a pipeline of one stage needs no communicator of its own
    BR_NCCL_CHECK(ncclCommSplit(nccl_comm, stages > 1 ? replica : NCCL_SPLIT_NOCOLOR, stage, &pipe, nullptr));
    BR_NCCL_CHECK(ncclCommSplit(nccl_comm, stage, replica, &dp, nullptr));
    job_comm = nccl_comm;
    nccl_comm = pipe;
    has_comm = pipe != nullptr;
    nccl_rank = stage;
    nccl_world = stages;
    dp_comm = dp;
    dp_rank = replica;
    dp_world = replicas;
}

void CollectiveContext::shutdown() {
    if (dp_comm) ncclCommDestroy(dp_comm);
    dp_comm = nullptr;
    dp_world = 1;
    dp_rank = 0;
    if (has_comm && nccl_comm) ncclCommDestroy(nccl_comm);
    if (job_comm) ncclCommDestroy(job_comm);
    job_comm = nullptr;
    has_comm = false;
    nccl_comm = nullptr;
}

int CollectiveContext::now() {
    auto d = std::chrono::steady_clock::now() - g_boot_time;
    return (int)std::chrono::duration_cast<std::chrono::seconds>(d).count();
}

// ------------------------------------------------------------------------------------------
bool PipeLinks::is_open = false;
int PipeLinks::slots = 0;
size_t PipeLinks::slot_bytes = 0;

namespace {

typedef CUresult (*StreamWaitValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
StreamWaitValue32Fn g_wait_value = nullptr;

constexpr size_t LINK_HEADER = 4096;        // arrive[2][MAX_SLOTS] then ack[2][MAX_SLOTS], uint32

// One end of the links = one rank's view: its own block, its neighbours' blocks and its counters.  A process holds
// one end; a single-rank process that plays several ranks (tests) holds one per played rank and switches between them.
struct LinkEnd {
    unsigned char* local = nullptr;
    unsigned char* peer[2] = {nullptr, nullptr};   // [0] previous rank's block, [1] next rank's block
    bool mapped[2] = {false, false};               // opened through IPC (to be closed), not a block of this process
    uint32_t sent[2][PipeLinks::MAX_SLOTS];
    uint32_t received[2][PipeLinks::MAX_SLOTS];
    bool copy_pending[2] = {false, false};
};
std::vector<LinkEnd> g_ends;
LinkEnd* g_end = nullptr;                             // the end the next call works on
int g_emulated_ranks = 0;
int g_pending_rank = -1;
cudaEvent_t g_link_ready = nullptr;                   // compute stream -> transfer stream
cudaEvent_t g_copy_done[2] = {nullptr, nullptr};      // transfer stream -> compute stream
int g_link_users = 0;

inline uint32_t* arrive_flag(unsigned char* block, int side, int slot) {
    return reinterpret_cast<uint32_t*>(block) + side * PipeLinks::MAX_SLOTS + slot;
}
inline uint32_t* ack_flag(unsigned char* block, int dir, int slot) {
    return reinterpret_cast<uint32_t*>(block) + (2 + dir) * PipeLinks::MAX_SLOTS + slot;
}
inline unsigned char* window_of(unsigned char* block, int side, int slot) {
    return block + LINK_HEADER + ((size_t)side * PipeLinks::slots + slot) * PipeLinks::slot_bytes;
}
inline void wait_geq(cudaStream_t st, uint32_t* flag, uint32_t value) {
    CUresult r = g_wait_value((CUstream)st, (CUdeviceptr)(uintptr_t)flag, value, CU_STREAM_WAIT_VALUE_GEQ);
    br_assert(r == CUDA_SUCCESS, "cuStreamWaitValue32 failed");
}
inline void check_slot(int two, int slot) {
    br_assert(PipeLinks::is_open && g_end != nullptr, "io.link: the links are not open");
    br_assert((two == 0 || two == 1) && slot >= 0 && slot < PipeLinks::slots, "io.link: bad side / direction or slot");
}

}  // namespace

void PipeLinks::emulate(int ranks) {
    br_assert(CollectiveContext::nccl_world == 1 && ranks >= 1 && ranks <= 64, "io.link.emulate: a single-rank process plays 1..64 ranks");
    if (is_open) {
        br_assert((int)g_ends.size() == ranks, "io.link.emulate: the links are open for another number of played ranks");
        return;
    }
    g_emulated_ranks = ranks;
}

void PipeLinks::select(int rank) {
    if (!is_open) {            // remembered until io.link.open has made the ends
        g_pending_rank = rank;
        return;
    }
    br_assert(rank >= 0 && rank < (int)g_ends.size(), "io.link.rank: no such played rank");
    g_end = &g_ends[rank];
}

void PipeLinks::open(size_t bytes_per_slot, int nslots) {
    br_assert(ComputingContext::booted, "io.link.open needs the computing context");
    br_assert(nslots >= 1 && nslots <= MAX_SLOTS && bytes_per_slot > 0, "io.link.open: bad slot count or size");
    if (is_open) {
        // several stage scripts of one process (a test that plays all ranks itself) share the blocks
        br_assert(nslots == slots && (bytes_per_slot + 255) / 256 * 256 == slot_bytes, "io.link.open: already open with another geometry");
        g_link_users += 1;
        if (g_pending_rank >= 0) {
            int r = g_pending_rank;
            g_pending_rank = -1;
            select(r);
        }
        return;
    }
    if (!g_wait_value) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuStreamWaitValue32", &fn, cudaEnableDefault, &q);
        br_assert(e == cudaSuccess && q == cudaDriverEntryPointSuccess && fn != nullptr, "the driver offers no cuStreamWaitValue32");
        g_wait_value = reinterpret_cast<StreamWaitValue32Fn>(fn);
    }
    slots = nslots;
    slot_bytes = (bytes_per_slot + 255) / 256 * 256;
    const size_t total = LINK_HEADER + 2 * (size_t)slots * slot_bytes;
    cudaStream_t st = ComputingContext::cuda_stream;
    const int rank = CollectiveContext::nccl_rank, world = CollectiveContext::nccl_world;
    const int ends = (world == 1 && g_emulated_ranks > 1) ? g_emulated_ranks : 1;
    g_ends.assign(ends, LinkEnd());
    for (auto& e : g_ends) {
        BR_CUDA_CHECK(cudaMalloc(&e.local, total));
        BR_CUDA_CHECK(cudaMemsetAsync(e.local, 0, LINK_HEADER, st));
        std::memset(e.sent, 0, sizeof(e.sent));
        std::memset(e.received, 0, sizeof(e.received));
    }
    BR_CUDA_CHECK(cudaStreamSynchronize(st));
    if (world == 1 || !CollectiveContext::has_comm) {
        br_assert(world == 1, "io.link.open: several ranks need the NCCL communicator to exchange their memory handles");
        if (ends == 1) {
            g_ends[0].peer[0] = g_ends[0].peer[1] = g_ends[0].local;      // loop-back: both neighbours are this block
        } else {
            for (int r = 0; r < ends; r++) {
                if (r > 0) g_ends[r].peer[0] = g_ends[r - 1].local;
                if (r + 1 < ends) g_ends[r].peer[1] = g_ends[r + 1].local;
            }
        }
    } else {
        // every rank's IPC handle to every rank, through the communicator that exists anyway
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is 64 bytes");
        LinkEnd& e = g_ends[0];
        cudaIpcMemHandle_t mine;
        BR_CUDA_CHECK(cudaIpcGetMemHandle(&mine, e.local));
        unsigned char* table = nullptr;
        BR_CUDA_CHECK(cudaMalloc(&table, (size_t)world * 64));
        BR_CUDA_CHECK(cudaMemcpyAsync(table + (size_t)rank * 64, &mine, 64, cudaMemcpyHostToDevice, st));
        BR_NCCL_CHECK(ncclAllGather(table + (size_t)rank * 64, table, 64, ncclChar, CollectiveContext::nccl_comm, st));
        std::vector<cudaIpcMemHandle_t> all(world);
        BR_CUDA_CHECK(cudaMemcpyAsync(all.data(), table, (size_t)world * 64, cudaMemcpyDeviceToHost, st));
        BR_CUDA_CHECK(cudaStreamSynchronize(st));
        BR_CUDA_CHECK(cudaFree(table));
        unsigned char mine_ok = 1;
        for (int d = 0; d < 2; d++) {
            const int nb = d == 0 ? rank - 1 : rank + 1;
            if (nb < 0 || nb >= world) continue;
            void* p = nullptr;
            if (cudaIpcOpenMemHandle(&p, all[nb], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                cudaGetLastError();            // clear the error: the failure is reported below, by every rank alike
                mine_ok = 0;
                continue;
            }
            e.peer[d] = static_cast<unsigned char*>(p);
            e.mapped[d] = true;
        }
        // all ranks or none: a rank that could not map a neighbour makes every rank give up together, so that a caller
        // can fall back to another transport without the ranks disagreeing
        unsigned char* flags = nullptr;
        BR_CUDA_CHECK(cudaMalloc(&flags, (size_t)world));
        BR_CUDA_CHECK(cudaMemcpyAsync(flags + rank, &mine_ok, 1, cudaMemcpyHostToDevice, st));
        BR_NCCL_CHECK(ncclAllGather(flags + rank, flags, 1, ncclChar, CollectiveContext::nccl_comm, st));
        std::vector<unsigned char> oks(world);
        BR_CUDA_CHECK(cudaMemcpyAsync(oks.data(), flags, (size_t)world, cudaMemcpyDeviceToHost, st));
        BR_CUDA_CHECK(cudaStreamSynchronize(st));
        BR_CUDA_CHECK(cudaFree(flags));
        bool all_ok = true;
        for (unsigned char v : oks) all_ok = all_ok && v != 0;
        if (!all_ok) {
            for (int d = 0; d < 2; d++)
                if (e.mapped[d]) cudaIpcCloseMemHandle(e.peer[d]);
            // every rank has unmapped before anyone frees (same barrier as in close)
            if (ncclAllGather(e.local + 4 * (size_t)rank, e.local, 4, ncclChar, CollectiveContext::nccl_comm, st) == ncclSuccess)
                cudaStreamSynchronize(st);
            cudaFree(e.local);
            g_ends.clear();
            br_panic("io.link.open: a rank could not map its neighbour's memory (CUDA IPC or peer access unavailable)");
        }
    }
    g_end = &g_ends[0];
    BR_CUDA_CHECK(cudaEventCreateWithFlags(&g_link_ready, cudaEventDisableTiming));
    for (int d = 0; d < 2; d++) BR_CUDA_CHECK(cudaEventCreateWithFlags(&g_copy_done[d], cudaEventDisableTiming));
    is_open = true;
    g_link_users = 1;
    if (g_pending_rank >= 0) {
        int r = g_pending_rank;
        g_pending_rank = -1;
        select(r);
    }
}

void PipeLinks::close() {
    if (!is_open) return;
    if (--g_link_users > 0) return;
    cudaStreamSynchronize(ComputingContext::cuda_stream);
    for (int d = 0; d < 2; d++) cudaStreamSynchronize(ComputingContext::link_stream[d]);
    bool mapped = false;
    for (auto& e : g_ends)
        for (int d = 0; d < 2; d++)
            if (e.mapped[d]) {
                cudaIpcCloseMemHandle(e.peer[d]);
                mapped = true;
            }
    for (int d = 0; d < 2; d++) cudaEventDestroy(g_copy_done[d]);
    cudaEventDestroy(g_link_ready);
    // a block may only be freed once no neighbour maps it any more: every rank has unmapped before anyone frees
    if ((mapped || CollectiveContext::nccl_world > 1) && CollectiveContext::has_comm) {
        unsigned char* scratch = g_ends[0].local;      // the header is free now; world x 4 bytes fit it by far
        if (ncclAllGather(scratch + 4 * (size_t)CollectiveContext::nccl_rank, scratch, 4, ncclChar, CollectiveContext::nccl_comm,
                          ComputingContext::cuda_stream) == ncclSuccess)
            cudaStreamSynchronize(ComputingContext::cuda_stream);
    }
    for (auto& e : g_ends) cudaFree(e.local);
    g_ends.clear();
    g_end = nullptr;
    g_emulated_ranks = 0;
    is_open = false;
}

void* PipeLinks::window(int side, int slot) {
    check_slot(side, slot);
    return window_of(g_end->local, side, slot);
}

void PipeLinks::send(int dir, int slot, const void* src, size_t bytes) {
    check_slot(dir, slot);
    br_assert(bytes <= slot_bytes, "io.link.send: the tensor is larger than a window");
    LinkEnd& e = *g_end;
    unsigned char* peer = e.peer[dir];
    br_assert(peer != nullptr, "io.link.send: no neighbour in that direction");
    const int side = dir == 1 ? 0 : 1;         // what goes to the next rank lands in its side-0 window
    cudaStream_t ls = ComputingContext::link_stream[dir];
    BR_CUDA_CHECK(cudaEventRecord(g_link_ready, ComputingContext::cuda_stream));
    BR_CUDA_CHECK(cudaStreamWaitEvent(ls, g_link_ready, 0));
    wait_geq(ls, ack_flag(e.local, dir, slot), e.sent[dir][slot]);      // the previous content has been read
    BR_CUDA_CHECK(cudaMemcpyAsync(window_of(peer, side, slot), src, bytes, cudaMemcpyDefault, ls));
    e.sent[dir][slot] += 1;
    int st = brk_signal_u32(arrive_flag(peer, side, slot), e.sent[dir][slot], (void*)ls);
    br_assert(st == BRK_OK, "io.link.send: the signal kernel did not launch");
    BR_CUDA_CHECK(cudaEventRecord(g_copy_done[dir], ls));
    e.copy_pending[dir] = true;
}

void PipeLinks::fence(int dir) {
    check_slot(dir, 0);
    if (!g_end->copy_pending[dir]) return;
    // one event per direction serves all played ranks: it then stands for the latest copy of any of them, which is later
    BR_CUDA_CHECK(cudaStreamWaitEvent(ComputingContext::cuda_stream, g_copy_done[dir], 0));
    g_end->copy_pending[dir] = false;
}

void PipeLinks::wait(int side, int slot) {
    check_slot(side, slot);
    g_end->received[side][slot] += 1;
    wait_geq(ComputingContext::cuda_stream, arrive_flag(g_end->local, side, slot), g_end->received[side][slot]);
}

void PipeLinks::release(int side, int slot) {
    check_slot(side, slot);
    const int from = side == 0 ? 0 : 1;        // side-0 windows are filled by the previous rank
    unsigned char* peer = g_end->peer[from];
    br_assert(peer != nullptr, "io.link.release: no neighbour on that side");
    const int sender_dir = side == 0 ? 1 : 0;
    int st = brk_signal_u32(ack_flag(peer, sender_dir, slot), g_end->received[side][slot], (void*)ComputingContext::cuda_stream);
    br_assert(st == BRK_OK, "io.link.release: the signal kernel did not launch");
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
