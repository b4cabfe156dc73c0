// Host tensor backend: storage, views, file IO and the host transport.  Like the reference's
// CPUTensor (blackriver/cpu_tensor.hpp:30-39) it carries no math: every op_* of the decoder
// answers OP_TODO_ERROR on a host tensor, so nothing can silently run on the CPU.
#pragma once

#include "context.hpp"
#include "tensortype.hpp"

namespace br {

template <DataType DT>
struct CPUTensor : public TransformerComputing {
    // owning: from the host arena when it is booted, from the heap otherwise
    explicit CPUTensor(const ShapeType& shape);
    // non-owning view
    explicit CPUTensor(void* mem) : mem_(mem), heap_(false) {}
    ~CPUTensor() override;

    void* data() { return mem_; }

    ComputingReturn io_dump(tensor_t self) override;
    ComputingReturn io_load(tensor_t self, const char* fileName) override;
    ComputingReturn io_save(tensor_t self, const char* fileName) override;
    ComputingReturn io_mpi_bcast(tensor_t self, int root) override;
    ComputingReturn io_mpi_recv(tensor_t self, int source) override;
    ComputingReturn io_mpi_send(tensor_t self, int dst) override;

    ComputingReturn op_zero(tensor_t self) override;
    ComputingReturn op_fill(tensor_t self, float value) override;
    ComputingReturn op_copy(tensor_t self, tensor_t src) override;
    ViewReturn op_view(tensor_t self, size_t offset, const std::vector<size_t>& newShape) override;

private:
    void* mem_;
    bool heap_;
};

// Host-memory transport between ranks, staged through device scratch and NCCL (stands in for
// the MPI_Bcast / MPI_Send / MPI_Recv calls of blackriver/cpu_tensor.cpp:133-152).  With one
// rank they are no-ops.
void host_bcast(void* host, size_t bytes, int root);
void host_send(const void* host, size_t bytes, int dst);
void host_recv(void* host, size_t bytes, int src);

}  // namespace br
