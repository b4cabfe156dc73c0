// C ABI over the C++ host side (include/br_host.h).
#include "br_host.h"

#include <cstring>
#include <string>

#include "context.hpp"
#include "cpu_tensor.hpp"
#include "cuda_tensor.hpp"
#include "dag.hpp"
#include "nn.hpp"
#include "tensortype.hpp"

using namespace br;

static thread_local std::string g_error;

template <typename F>
static int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

extern "C" {

const char* brh_last_error(void) { return g_error.c_str(); }

int brh_context_boot(int device, void* stream, size_t workspace_bytes) {
    return guarded([&] {
        if (stream) ComputingContext::boot_with_stream(device, (cudaStream_t)stream, workspace_bytes);
        else ComputingContext::boot(device, workspace_bytes);
    });
}
int brh_context_shutdown(void) { return guarded([] { ComputingContext::shutdown(); }); }
void* brh_context_stream(void) { return (void*)ComputingContext::cuda_stream; }

int brh_collective_boot_local(int rank, int world) { return guarded([&] { CollectiveContext::boot_local(rank, world); }); }
int brh_collective_unique_id(char out[128]) {
    return guarded([&] {
        ncclUniqueId id = CollectiveContext::make_unique_id();
        static_assert(sizeof(id) == 128, "ncclUniqueId is 128 bytes");
        std::memcpy(out, &id, 128);
    });
}
int brh_collective_boot(int rank, int world, const char id_bytes[128]) {
    return guarded([&] {
        ncclUniqueId id;
        std::memcpy(&id, id_bytes, 128);
        CollectiveContext::boot(rank, world, id);
    });
}
int brh_collective_split(int replicas) { return guarded([&] { CollectiveContext::split_replicas(replicas); }); }
int brh_collective_shutdown(void) { return guarded([] { CollectiveContext::shutdown(); }); }

int brh_memory_boot(size_t total_bytes, int pinned) { return guarded([&] { MemoryContext::boot(total_bytes, pinned != 0); }); }
int brh_memory_shutdown(void) { return guarded([] { MemoryContext::shutdown(); }); }

void* brh_env_new(int hash_num) {
    Enviroment* env = nullptr;
    int rc = guarded([&] {
        env = new Enviroment(hash_num);
        load_nn_words(*env);
    });
    return rc == 0 ? env : nullptr;
}
void brh_env_free(void* env) { delete static_cast<Enviroment*>(env); }

#define ENV static_cast<Enviroment*>(env)

int brh_env_execute(void* env, const char* text) { return guarded([&] { ENV->execute(text); }); }
void* brh_env_build(void* env, const char* text) {
    DaG* dag = nullptr;
    int rc = guarded([&] { dag = ENV->build(text); });
    return rc == 0 ? dag : nullptr;
}
int brh_env_run(void* env, void* program) { return guarded([&] { ENV->run(static_cast<DaG*>(program)); }); }
void brh_program_free(void* program) { delete static_cast<DaG*>(program); }
int brh_env_change(void* env, int hash) { return guarded([&] { ENV->change((size_t)hash); }); }
int brh_env_current(void* env) { return (int)ENV->hashes_current(); }
int brh_env_stack_size(void* env) { return (int)ENV->stack().size(); }
int brh_env_stack_clear(void* env) { return guarded([&] { ENV->stack().clear(); }); }
int brh_env_pop_number(void* env, double* out) { return guarded([&] { *out = ENV->stack().pop_number(); }); }
int brh_env_pop_string(void* env, char* out, size_t cap) {
    return guarded([&] {
        std::string s = ENV->stack().pop_string();
        br_assert(s.size() + 1 <= cap, "string buffer too small");
        std::memcpy(out, s.c_str(), s.size() + 1);
    });
}
int brh_env_push_number(void* env, double v) { return guarded([&] { ENV->stack().push_number(v); }); }
int brh_env_push_string(void* env, const char* s) { return guarded([&] { ENV->stack().push_string(s); }); }
int brh_env_has(void* env, const char* name) { return ENV->hash().has(name) ? 1 : 0; }
int brh_env_get_number(void* env, const char* name, double* out) { return guarded([&] { *out = ENV->hash().find_number(name); }); }

int brh_env_tensor_info(void* env, const char* name, void** data, int* is_cuda, int* dtype, int* ndim, int64_t dims[8]) {
    return guarded([&] {
        tensor_t t = ENV->hash().find_tensor(name);
        br_assert(t->shape().dim() <= 8, "too many dimensions");
        if (data) *data = t->data();
        if (is_cuda) *is_cuda = t->is_cuda() ? 1 : 0;
        if (dtype) *dtype = (int)t->dtype();
        if (ndim) *ndim = (int)t->shape().dim();
        if (dims)
            for (size_t i = 0; i < t->shape().dim(); i++) dims[i] = (int64_t)t->shape()[(int)i];
    });
}

int brh_env_tensor_write(void* env, const char* name, const void* host, size_t bytes) {
    return guarded([&] {
        tensor_t t = ENV->hash().find_tensor(name);
        br_assert(bytes == t->bytes(), "byte count does not match the tensor");
        if (t->is_cuda()) {
            BR_CUDA_CHECK(cudaMemcpyAsync(t->data(), host, bytes, cudaMemcpyHostToDevice, ComputingContext::cuda_stream));
            BR_CUDA_CHECK(cudaStreamSynchronize(ComputingContext::cuda_stream));
        } else {
            std::memcpy(t->data(), host, bytes);
        }
    });
}

int brh_env_tensor_read(void* env, const char* name, void* host, size_t bytes) {
    return guarded([&] {
        tensor_t t = ENV->hash().find_tensor(name);
        br_assert(bytes == t->bytes(), "byte count does not match the tensor");
        if (t->is_cuda()) {
            BR_CUDA_CHECK(cudaMemcpyAsync(host, t->data(), bytes, cudaMemcpyDeviceToHost, ComputingContext::cuda_stream));
            BR_CUDA_CHECK(cudaStreamSynchronize(ComputingContext::cuda_stream));
        } else {
            std::memcpy(host, t->data(), bytes);
        }
    });
}

// Asynchronous host -> device write: the bytes are copied out of `host` into a pinned ring before the call returns and
// travel on the compute stream from there.  The ring is cut into quarters; entering a quarter waits (on the host) for
// the copies queued from it one lap earlier.
namespace {
constexpr size_t STAGE_BYTES = (size_t)16 << 20;
constexpr size_t STAGE_QUARTER = STAGE_BYTES / 4;
unsigned char* g_stage = nullptr;
size_t g_stage_head = 0;
cudaEvent_t g_stage_done[4] = {nullptr, nullptr, nullptr, nullptr};
bool g_stage_used[4] = {false, false, false, false};

unsigned char* stage_take(size_t bytes) {
    br_assert(bytes <= STAGE_QUARTER, "asynchronous tensor writes are limited to 4 MiB each");
    if (!g_stage) {
        BR_CUDA_CHECK(cudaMallocHost(&g_stage, STAGE_BYTES));
        for (auto& e : g_stage_done) BR_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    size_t q = g_stage_head / STAGE_QUARTER;
    if (g_stage_head + bytes > (q + 1) * STAGE_QUARTER) {      // does not fit the rest of this quarter: move on
        BR_CUDA_CHECK(cudaEventRecord(g_stage_done[q], ComputingContext::cuda_stream));
        g_stage_used[q] = true;
        q = (q + 1) % 4;
        g_stage_head = q * STAGE_QUARTER;
        if (g_stage_used[q]) BR_CUDA_CHECK(cudaEventSynchronize(g_stage_done[q]));
    }
    unsigned char* p = g_stage + g_stage_head;
    g_stage_head += (bytes + 63) / 64 * 64;
    return p;
}
}  // namespace

int brh_env_tensor_write_async(void* env, const char* name, const void* host, size_t bytes) {
    return guarded([&] {
        tensor_t t = ENV->hash().find_tensor(name);
        br_assert(bytes == t->bytes(), "byte count does not match the tensor");
        if (t->is_cuda()) {
            unsigned char* staged = stage_take(bytes);
            std::memcpy(staged, host, bytes);
            BR_CUDA_CHECK(cudaMemcpyAsync(t->data(), staged, bytes, cudaMemcpyHostToDevice, ComputingContext::cuda_stream));
        } else {
            std::memcpy(t->data(), host, bytes);
        }
    });
}

int brh_profile_start(void) { return guarded([] { Profiler::start(); }); }
int brh_profile_stop(char* out, size_t cap) {
    return guarded([&] {
        std::string j = Profiler::report_json();
        br_assert(j.size() + 1 <= cap, "profile buffer too small");
        std::memcpy(out, j.c_str(), j.size() + 1);
    });
}

float brh_last_loss(void) { return last_loss(); }

}  // extern "C"
