// Process-wide runtime state: the device context (streams, events, scratch), the collective
// context (rank layout and the NCCL communicator) and the host memory arena.
//
// Same three singletons as the reference (blackriver/context.hpp:8-47) with these changes:
//  * one rank per GPU; there is no extra CPU-only feeder rank, so nccl_rank == mpi_rank;
//  * a compute stream plus a dedicated transfer stream with events between them, so stage
//    hand-offs overlap with compute; no cuBLAS / cuDNN handles (the kernels are our own);
//  * no MPI dependency: the NCCL unique id arrives from the launcher (a file, or bytes handed
//    in by an embedding process) and host tensors travel through NCCL via device staging.
#pragma once

#include <cuda_runtime.h>
#include <nccl.h>

#include <cstddef>
#include <string>

#include <vector>

#include "common.hpp"

namespace br {

struct ComputingContext {
    static int cuda_device;
    static cudaStream_t cuda_stream;   // compute
    static cudaStream_t comm_stream;   // staged host transfers
    static cudaStream_t link_stream[2];   // stage hand-offs of PipeLinks: [0] towards the previous rank, [1] towards the next
    static cudaEvent_t compute_done;   // recorded on cuda_stream before a send reads a tensor
    static cudaEvent_t comm_done;      // recorded on comm_stream after a recv wrote a tensor
    // Side mode (op.stream.side): cuda_stream is temporarily the transfer stream, so that every operator queued
    // meanwhile (the optimizer) runs beside what the compute stream is given next; main_stream then holds the compute
    // stream (nullptr outside side mode).  marks[i] are events recorded by op.event.record for op.event.wait.
    static cudaStream_t main_stream;
    static std::vector<cudaEvent_t> marks;
    static std::vector<char> mark_set;

    static void* cuda_workspace;       // device scratch handed to kernels that need it
    static void* local_workspace;      // pinned host scratch of the same size
    static size_t workspace_size;

    // training-step switches read by the device backend
    static int grad_accumulate;        // 1: op_linear_backward / op_layernorm_backward add into W_g, b_g (micro-batches)
    static float loss_scale;           // multiplies the loss gradient (fp16 gradients); Adam divides it out

    static int verbose;                // 1: op_loss_backward prints its "#### items loss" line like the reference
    static int nccl_on_comm_stream;    // 1: the io.nccl.* words queue on comm_stream (between op.stream.fork and op.stream.join)

    static bool booted;
    static void boot(int device, size_t workspace_bytes = (size_t)256 << 20);
    // adopt a stream owned by an embedding process (e.g. torch's current stream)
    static void boot_with_stream(int device, cudaStream_t compute, size_t workspace_bytes = (size_t)256 << 20);
    static void shutdown();
};

// Optional per-kernel-family timing of the device backend: when enabled, every kernel-library call
// made by the backend is bracketed by CUDA events on the compute stream; report() waits for the
// stream and returns the accumulated device time and call count per family.
struct Profiler {
    static bool enabled;
    static void start();                       // clears previous records
    static std::string report_json();          // {"family": {"ms": .., "calls": ..}, ...}; disables
    static void begin(const char* family);
    static void end();
};

struct CollectiveContext {
    static int mpi_world;   // number of ranks == number of GPUs in the job
    static int mpi_rank;
    static int nccl_world;  // same values; both names are kept because callers use both
    static int nccl_rank;
    static ncclComm_t nccl_comm;
    static ncclUniqueId nccl_id;
    static bool has_comm;
    // Data-parallel replicas (split_replicas): the job's ranks form `dp_world` replicas of a pipeline of nccl_world
    // stages; rank r of the job is stage r % stages of replica r / stages.  nccl_comm / nccl_rank / nccl_world then
    // describe this rank's pipeline (what every io.nccl.* hand-off and the stage links use), dp_comm joins the ranks
    // that hold the same stage in every replica, and mpi_rank / mpi_world keep the job-wide numbers.
    static int dp_world;
    static int dp_rank;
    static ncclComm_t dp_comm;
    static ncclComm_t job_comm;     // the communicator the two above were split from (nullptr when never split)

    // Rank layout only (no communicator): what host-only tools and tests need.
    static void boot_local(int rank, int world);
    // Creates the communicator from a unique id produced by make_unique_id() on rank 0.
    static void boot(int rank, int world, const ncclUniqueId& id);
    // Rendezvous through a file: rank 0 writes the id, the others poll for it (bounded wait).
    static void boot_from_file(int rank, int world, const std::string& path, int timeout_s = 120);
    static ncclUniqueId make_unique_id();
    // Splits the booted job into `replicas` equal pipelines (see dp_world above).  Collective over all ranks.
    static void split_replicas(int replicas);
    static void shutdown();
    static int now();  // whole seconds since boot, as the reference's echo prints
};

// One-sided stage hand-offs between neighbouring pipeline ranks of one node, replacing ncclSend / ncclRecv on the
// compute stream (blackriver/cuda_tensor.cpp:75-96) where transfers have to overlap compute.
//
// Every rank owns one device block, exported to its two neighbours through CUDA IPC:
//   * windows [2 sides][slots][slot_bytes]: side 0 is written by the previous rank (activations going forward),
//     side 1 by the next rank (gradients going backward); a slot is one micro-batch in flight;
//   * arrive[side][slot]: how many times that window has been filled (written by the sender after its copy);
//   * ack[dir][slot]: how many of this rank's sends in direction dir (1 = to the next rank, 0 = to the previous one)
//     the receiver has finished reading (written by the receiver).
// A send is a device-to-device copy into the neighbour's window on a transfer stream of its own (the copy engines
// move it; no SM runs a communication kernel) followed by a one-thread kernel that raises arrive; the consumer's
// compute stream waits for the counter with a stream memory operation (cuStreamWaitValue32), so no kernel spins
// either.  A sender never waits for its receiver except when it is about to overwrite a window the receiver has
// not released yet.  With one rank the block is its own neighbour in both directions (loop-back).
struct PipeLinks {
    static constexpr int MAX_SLOTS = 64;
    static bool is_open;
    static int slots;
    static size_t slot_bytes;

    // Collective over all ranks of the communicator.  Throws if CUDA IPC or stream memory operations are unavailable.
    static void open(size_t slot_bytes, int slots);
    // A single-rank process may play `ranks` pipeline ranks itself (tests on one GPU): called before open, it makes
    // open create one block per played rank, chained like real neighbours; select says whose turn it is.
    static void emulate(int ranks);
    static void select(int rank);
    static void close();
    static void* window(int side, int slot);                 // this rank's own window
    // queue: [after everything on the compute stream so far] copy `bytes` from src into the neighbour's window, raise arrive
    static void send(int dir, int slot, const void* src, size_t bytes);
    static void fence(int dir);                              // compute stream waits for the last copy queued in direction dir
    static void wait(int side, int slot);                    // compute stream waits for the next filling of window (side, slot)
    static void release(int side, int slot);                 // after the compute stream's work so far: the sender may overwrite it
};

struct MemoryContext {
    static const size_t page_size;
    static void* root;
    static size_t total_size;
    static size_t currentp;
    static bool pinned;

    // Bump allocator over one block, never freed piecewise (blackriver/context.cpp:96-121).
    // Requests are rounded UP to the page size (the reference rejects unaligned sizes).  With
    // pinned = true the block is page-locked so device copies from it are asynchronous.
    static void boot(size_t total_bytes, bool pinned = false);
    static void* alloc(size_t bytes);
    static void shutdown();
};

}  // namespace br
