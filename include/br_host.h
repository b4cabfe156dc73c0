/*
 * br_host.h -- C ABI of libbr_host.so, the C++ host side (operator interface, tensor facade,
 * words machine, runtime contexts) for embedding processes: tests, benchmarks, other languages.
 * A C++ program links the classes directly (see blackriver_b200/csrc/host/train_bloom.cpp).
 *
 * All functions return 0 on success and -1 on failure unless stated otherwise; after a failure
 * brh_last_error() holds the message (the fatal checks of the C++ side surface here as errors
 * instead of terminating the process).
 */
#ifndef BR_HOST_H_
#define BR_HOST_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BRH_API __attribute__((visibility("default")))

BRH_API const char* brh_last_error(void);

/* Device context: blackriver/context.cpp:18-54 (ComputingContext::boot / shutdown).  `stream` may
 * be NULL (the library creates its compute stream) or a cudaStream_t owned by the caller. */
BRH_API int brh_context_boot(int device, void* stream, size_t workspace_bytes);
BRH_API int brh_context_shutdown(void);
BRH_API void* brh_context_stream(void);

/* Rank layout and NCCL communicator: blackriver/context.cpp:56-93 (CollectiveContext::boot), one
 * rank per GPU, the unique id handed over by the launcher instead of MPI_Bcast. */
BRH_API int brh_collective_boot_local(int rank, int world);
BRH_API int brh_collective_unique_id(char out[128]);
BRH_API int brh_collective_boot(int rank, int world, const char id[128]);
/* Data-parallel replicas of the pipeline (absent from the reference, whose one communicator is point-to-point only,
 * blackriver/context.cpp:56-80): splits the booted job of `world` ranks into `replicas` pipelines of world / replicas
 * stages each (rank r = stage r % stages of replica r / stages).  Afterwards the io.nccl.* hand-offs and the stage
 * links address pipeline stages, and io.nccl.allreduce sums a tensor over the replicas.  Collective: every rank calls
 * it with the same value; 1 is a no-op. */
BRH_API int brh_collective_split(int replicas);
BRH_API int brh_collective_shutdown(void);

/* Host arena: blackriver/context.cpp:96-121 (MemoryContext). */
BRH_API int brh_memory_boot(size_t total_bytes, int pinned);
BRH_API int brh_memory_shutdown(void);

/* Words machine: blackriver/dag.hpp:363-482 (Enviroment) with the op.* / io.* words of
 * blackriver/nn.cpp:339-371 registered. */
BRH_API void* brh_env_new(int hash_num);
BRH_API void brh_env_free(void* env);
BRH_API int brh_env_execute(void* env, const char* text);
/* Compile + link once, run many times (Enviroment::build / run, blackriver/dag.hpp:382-392): the
 * driver runs the same init program once per hash table.  %def bodies are registered by build. */
BRH_API void* brh_env_build(void* env, const char* text);
BRH_API int brh_env_run(void* env, void* program);
BRH_API void brh_program_free(void* program);
BRH_API int brh_env_change(void* env, int hash);
BRH_API int brh_env_current(void* env);
BRH_API int brh_env_stack_size(void* env);
BRH_API int brh_env_stack_clear(void* env);
BRH_API int brh_env_pop_number(void* env, double* out);
BRH_API int brh_env_pop_string(void* env, char* out, size_t cap);
BRH_API int brh_env_push_number(void* env, double v);
BRH_API int brh_env_push_string(void* env, const char* s);
BRH_API int brh_env_has(void* env, const char* name);            /* 1 / 0 */
BRH_API int brh_env_get_number(void* env, const char* name, double* out);
/* Tensor stored under `name` in the current hash table: storage address, placement
 * (1 = device), element type (0 f32, 2 f16, 3 i32: br::DataType), rank and dims. */
BRH_API int brh_env_tensor_info(void* env, const char* name, void** data, int* is_cuda, int* dtype, int* ndim, int64_t dims[8]);
/* Byte copies between caller host memory and the named tensor (synchronous). */
BRH_API int brh_env_tensor_write(void* env, const char* name, const void* host, size_t bytes);
BRH_API int brh_env_tensor_read(void* env, const char* name, void* host, size_t bytes);

/* Same write without waiting for the device: the bytes are copied out of `host` (into page-locked staging memory owned
 * by the library) before the call returns and reach the tensor in compute-stream order.  At most 4 MiB per call. */
BRH_API int brh_env_tensor_write_async(void* env, const char* name, const void* host, size_t bytes);

/* Per-kernel-family device timing of the backend (CUDA events around every kernel-library call).
 * brh_profile_stop waits for the stream, writes a JSON object {"family": {"ms":..,"calls":..}} into
 * `out` and switches profiling off. */
BRH_API int brh_profile_start(void);
BRH_API int brh_profile_stop(char* out, size_t cap);

/* Value returned by the most recent op.loss_backward word. */
BRH_API float brh_last_loss(void);

#ifdef __cplusplus
}
#endif
#endif /* BR_HOST_H_ */
