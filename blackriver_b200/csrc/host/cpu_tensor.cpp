#include "cpu_tensor.hpp"

#include <cuda_fp16.h>

#include <algorithm>
#include <cstring>

#include "cuda_tensor.hpp"

namespace br {

template <DataType DT>
CPUTensor<DT>::CPUTensor(const ShapeType& shape) {
    size_t bytes = std::max<size_t>(shape.numel() * DataType_size(DT), 1);
    if (MemoryContext::root != nullptr) {
        mem_ = MemoryContext::alloc(bytes);
        heap_ = false;
    } else {
        mem_ = ::aligned_alloc(64, (bytes + 63) / 64 * 64);
        br_assert(mem_ != nullptr, "host tensor allocation failed");
        heap_ = true;
    }
}

template <DataType DT>
CPUTensor<DT>::~CPUTensor() {
    if (heap_) ::free(mem_);
}

template <typename T>
static void print_edges(const T* p, size_t items, size_t last_dim) {
    size_t n = std::min<size_t>(last_dim, 8);
    std::cout << "--------------------------\nFirst " << n << " : ";
    for (size_t i = 0; i < n; i++) std::cout << p[i] << " ";
    std::cout << "\nLast " << n << " : ";
    for (size_t i = 0; i < n; i++) std::cout << p[items - n + i] << " ";
    std::cout << std::endl;
}

template <DataType DT>
ComputingReturn CPUTensor<DT>::io_dump(tensor_t self) {
    size_t last = self->shape().vec().back();
    if (DT == DataType::Float) print_edges((const float*)mem_, self->items(), last);
    else if (DT == DataType::Int) print_edges((const int*)mem_, self->items(), last);
    else {
        std::vector<float> tmp(self->items());
        for (size_t i = 0; i < tmp.size(); i++) tmp[i] = __half2float(((const __half*)mem_)[i]);
        print_edges(tmp.data(), tmp.size(), last);
    }
    return OP_OK;
}

// Raw little-endian file of the tensor's element type (blackriver/cpu_tensor.cpp:117-130).
// An fp16 tensor also accepts an fp32 file of the same element count and converts.
template <DataType DT>
ComputingReturn CPUTensor<DT>::io_load(tensor_t self, const char* fileName) {
    std::vector<unsigned char> raw;
    read_data(fileName, raw);
    if (raw.size() == self->bytes()) {
        std::memcpy(mem_, raw.data(), raw.size());
        return OP_OK;
    }
    if (DT == DataType::F16 && raw.size() == self->items() * 4) {
        const float* f = reinterpret_cast<const float*>(raw.data());
        for (size_t i = 0; i < self->items(); i++) ((__half*)mem_)[i] = __float2half(f[i]);
        return OP_OK;
    }
    return OP_INPUT_ERROR;
}

// Mirror of io_load (the reference leaves io_save unimplemented, blackriver/cpu_tensor.cpp:111-114).
template <DataType DT>
ComputingReturn CPUTensor<DT>::io_save(tensor_t self, const char* fileName) {
    std::ofstream out(fileName, std::ios::binary);
    if (!out) return OP_OUTPUT_ERROR;
    out.write(reinterpret_cast<const char*>(mem_), (std::streamsize)self->bytes());
    return out ? OP_OK : OP_OUTPUT_ERROR;
}

template <DataType DT>
ComputingReturn CPUTensor<DT>::io_mpi_bcast(tensor_t self, int root) {
    host_bcast(mem_, self->bytes(), root);
    return OP_OK;
}

template <DataType DT>
ComputingReturn CPUTensor<DT>::io_mpi_recv(tensor_t self, int source) {
    host_recv(mem_, self->bytes(), source);
    return OP_OK;
}

template <DataType DT>
ComputingReturn CPUTensor<DT>::io_mpi_send(tensor_t self, int dst) {
    host_send(mem_, self->bytes(), dst);
    return OP_OK;
}

template <DataType DT>
ComputingReturn CPUTensor<DT>::op_zero(tensor_t self) {
    std::memset(mem_, 0, self->bytes());
    return OP_OK;
}

template <DataType DT>
ComputingReturn CPUTensor<DT>::op_fill(tensor_t self, float value) {
    size_t n = self->items();
    if (DT == DataType::Float) std::fill_n((float*)mem_, n, value);
    else if (DT == DataType::Int) std::fill_n((int*)mem_, n, (int)value);
    else std::fill_n((__half*)mem_, n, __float2half(value));
    return OP_OK;
}

// self <- src; src on the host (memcpy) or on the device (copy on the compute stream, then wait:
// the destination may be pageable, cf. blackriver/cpu_tensor.cpp:30-32).
template <DataType DT>
ComputingReturn CPUTensor<DT>::op_copy(tensor_t self, tensor_t src) {
    if (src->dtype() != DT) return OP_INPUT_ERROR;
    if (src->is_cpu()) {
        std::memmove(mem_, src->data(), self->bytes());
        return OP_OK;
    }
    auto st = ComputingContext::cuda_stream;
    BR_CUDA_CHECK(cudaMemcpyAsync(mem_, src->data(), self->bytes(), cudaMemcpyDeviceToHost, st));
    BR_CUDA_CHECK(cudaStreamSynchronize(st));
    return OP_OK;
}

template <DataType DT>
ViewReturn CPUTensor<DT>::op_view(tensor_t self, size_t offset, const std::vector<size_t>& newShape) {
    ShapeType shape(newShape);
    void* p = static_cast<unsigned char*>(mem_) + offset * DataType_size(DT);
    return std::make_shared<TensorType>(new CPUTensor<DT>(p), shape);
}

template struct CPUTensor<DataType::Float>;
template struct CPUTensor<DataType::F16>;
template struct CPUTensor<DataType::Int>;

// ------------------------------------------------------------------------------------------
// host transport over NCCL, chunked through the device scratch
// ------------------------------------------------------------------------------------------
template <typename F>
static void staged(void* host, size_t bytes, bool to_device_first, bool from_device_after, F&& collective) {
    if (CollectiveContext::nccl_world <= 1) return;
    br_assert(CollectiveContext::has_comm && ComputingContext::booted, "host transport needs the device and the communicator");
    auto st = ComputingContext::comm_stream;
    unsigned char* h = static_cast<unsigned char*>(host);
    const size_t chunk = ComputingContext::workspace_size;
    for (size_t off = 0; off < bytes; off += chunk) {
        size_t n = std::min(chunk, bytes - off);
        if (to_device_first) BR_CUDA_CHECK(cudaMemcpyAsync(ComputingContext::cuda_workspace, h + off, n, cudaMemcpyHostToDevice, st));
        collective(ComputingContext::cuda_workspace, n, st);
        if (from_device_after) BR_CUDA_CHECK(cudaMemcpyAsync(h + off, ComputingContext::cuda_workspace, n, cudaMemcpyDeviceToHost, st));
        BR_CUDA_CHECK(cudaStreamSynchronize(st));
    }
}

void host_bcast(void* host, size_t bytes, int root) {
    bool is_root = CollectiveContext::nccl_rank == root;
    staged(host, bytes, is_root, !is_root, [&](void* d, size_t n, cudaStream_t st) {
        BR_NCCL_CHECK(ncclBroadcast(d, d, n, ncclChar, root, CollectiveContext::nccl_comm, st));
    });
}

void host_send(const void* host, size_t bytes, int dst) {
    staged(const_cast<void*>(host), bytes, true, false, [&](void* d, size_t n, cudaStream_t st) {
        BR_NCCL_CHECK(ncclSend(d, n, ncclChar, dst, CollectiveContext::nccl_comm, st));
    });
}

void host_recv(void* host, size_t bytes, int src) {
    staged(host, bytes, false, true, [&](void* d, size_t n, cudaStream_t st) {
        BR_NCCL_CHECK(ncclRecv(d, n, ncclChar, src, CollectiveContext::nccl_comm, st));
    });
}

tensor_t create_cpu_float(std::vector<size_t>& shape) {
    ShapeType s(shape);
    return std::make_shared<TensorType>(new CPUTensor<DataType::Float>(s), s);
}
tensor_t create_cpu_int(std::vector<size_t>& shape) {
    ShapeType s(shape);
    return std::make_shared<TensorType>(new CPUTensor<DataType::Int>(s), s);
}
tensor_t create_cpu_half(std::vector<size_t>& shape) {
    ShapeType s(shape);
    return std::make_shared<TensorType>(new CPUTensor<DataType::F16>(s), s);
}

}  // namespace br
