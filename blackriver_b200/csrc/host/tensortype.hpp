// TensorType: the facade every word and every driver talks to.
//
// It owns one backend object (host or device storage of one element type), forwards each
// operator of the TransformerComputing interface to it and treats any status other than OP_OK
// as fatal, which is the contract of the reference facade (blackriver/tensortype.hpp:135-313,
// blackriver/tensortype.cpp:8-213).  Additions over the reference: fp16 device tensors, int32
// device tensors and host fp16 tensors (the reference declares DataType::F16 but never builds
// one, tensortype.hpp:16-21), and a destructor that releases every backend kind.
#pragma once

#include <cstdint>
#include <memory>
#include <sstream>
#include <string>
#include <variant>
#include <vector>

#include "common.hpp"
#include "operators.hpp"

namespace br {

enum DataType {
    Float = 0,
    BF16 = 1,
    F16 = 2,
    Int = 3,
};

inline size_t DataType_size(DataType t) {
    switch (t) {
        case Float: case Int: return 4;
        case F16: case BF16: return 2;
    }
    br_panic("unknown data type");
}

inline const char* DataType_name(DataType t) {
    switch (t) {
        case Float: return "f32";
        case F16: return "f16";
        case BF16: return "bf16";
        case Int: return "i32";
    }
    br_panic("unknown data type");
}

// Row-major, contiguous, no strides.
struct ShapeType {
    ShapeType() = delete;
    explicit ShapeType(const std::vector<size_t>& dims) : dims_(dims) {
        numel_ = 1;
        for (size_t d : dims_) numel_ *= d;
    }
    size_t numel() const { return numel_; }
    const std::vector<size_t>& vec() const { return dims_; }
    const size_t* dims() const { return dims_.data(); }
    size_t dim() const { return dims_.size(); }
    size_t operator[](int i) const { return dims_[i]; }
    bool operator==(const ShapeType& o) const { return dims_ == o.dims_; }
    bool operator!=(const ShapeType& o) const { return dims_ != o.dims_; }
    std::string to_string() const {
        std::ostringstream ss;
        ss << "[";
        for (size_t d : dims_) ss << d << " ";
        ss << "]";
        return ss.str();
    }

private:
    std::vector<size_t> dims_;
    size_t numel_;
};

template <DataType DT> struct CPUTensor;
template <DataType DT> struct CUDATensor;
using cpu_float_t = CPUTensor<DataType::Float>;
using cpu_half_t = CPUTensor<DataType::F16>;
using cpu_int_t = CPUTensor<DataType::Int>;
using cuda_float_t = CUDATensor<DataType::Float>;
using cuda_half_t = CUDATensor<DataType::F16>;
using cuda_int_t = CUDATensor<DataType::Int>;

struct TensorType : public TransformerComputing {
    enum ImplType { CPU_FLOAT, CPU_HALF, CPU_INT, CUDA_FLOAT, CUDA_HALF, CUDA_INT };

    TensorType() = delete;
    TensorType(cpu_float_t* t, const ShapeType& s);
    TensorType(cpu_half_t* t, const ShapeType& s);
    TensorType(cpu_int_t* t, const ShapeType& s);
    TensorType(cuda_float_t* t, const ShapeType& s);
    TensorType(cuda_half_t* t, const ShapeType& s);
    TensorType(cuda_int_t* t, const ShapeType& s);
    ~TensorType() override;

    const ShapeType& shape() const { return shape_; }
    const DataType& dtype() const { return dtype_; }
    size_t items() const { return shape_.numel(); }
    size_t bytes() const { return shape_.numel() * DataType_size(dtype_); }
    size_t impl_index() const { return (size_t)kind_; }
    int64_t& marker() { return marker_; }

    // raw storage address: host memory for cpu tensors, device memory for cuda tensors
    void* data() const { return data_; }

    cpu_float_t* cpu_float();
    cpu_half_t* cpu_half();
    cpu_int_t* cpu_int();
    cuda_float_t* cuda_float();
    cuda_half_t* cuda_half();
    cuda_int_t* cuda_int();

    bool is_cpu() const { return kind_ == CPU_FLOAT || kind_ == CPU_HALF || kind_ == CPU_INT; }
    bool is_cuda() const { return !is_cpu(); }
    const char* device_name() const { return is_cpu() ? "cpu" : "cuda"; }
    bool same_impl(const tensor_t& o) const { return kind_ == o->kind_; }
    bool same_dtype(const tensor_t& o) const { return dtype_ == o->dtype_; }
    bool same_shape(const tensor_t& o) const { return shape_ == o->shape_; }
    std::string to_string() const;

    TransformerComputing* impl() { return impl_; }

    // TransformerComputing, forwarded to the backend
    ComputingReturn op_zero(tensor_t self) override;
    ComputingReturn op_fill(tensor_t self, float value) override;
    ComputingReturn op_copy(tensor_t self, tensor_t src) override;
    ViewReturn op_view(tensor_t self, size_t offset, const std::vector<size_t>& newShape) override;
    ComputingReturn op_add(tensor_t self, tensor_t b, tensor_t c) override;
    ComputingReturn op_mul(tensor_t self, tensor_t b, tensor_t c) override;
    ComputingReturn op_linear(tensor_t self, tensor_t w, tensor_t b, tensor_t y) override;
    ComputingReturn op_layernorm(tensor_t self, tensor_t mean, tensor_t var, tensor_t scale, tensor_t bias, tensor_t y, float eps) override;
    ComputingReturn op_transpos_0213(tensor_t self, tensor_t y) override;
    ComputingReturn op_qk(tensor_t self, tensor_t k, tensor_t qk) override;
    ComputingReturn op_softmax(tensor_t self, tensor_t out) override;
    ComputingReturn op_attn(tensor_t self, tensor_t v, tensor_t attn) override;
    ComputingReturn op_gelu(tensor_t self, tensor_t dst) override;
    ComputingReturn op_last_logits(tensor_t self, tensor_t mask, tensor_t lm_head, tensor_t output) override;
    LossReturn op_loss_backward(tensor_t self, tensor_t ids, tensor_t mask, tensor_t lm_head, tensor_t all_logits, tensor_t x_g, tensor_t lm_head_g) override;
    ComputingReturn op_layernorm_backward(tensor_t self, tensor_t scale, tensor_t bias, tensor_t var, tensor_t y, tensor_t dscale, tensor_t dbias, tensor_t din, float eps) override;
    ComputingReturn op_linear_backward(tensor_t self, tensor_t x, tensor_t weight, tensor_t bias, tensor_t x_g, tensor_t weight_g, tensor_t bias_g) override;
    ComputingReturn op_gelu_backward(tensor_t self, tensor_t x, tensor_t x_g) override;
    ComputingReturn op_attn_backward(tensor_t self, tensor_t attn, tensor_t v, tensor_t attn_g, tensor_t v_g) override;
    ComputingReturn op_softmax_backward(tensor_t self, tensor_t out, tensor_t x_g) override;
    ComputingReturn op_softmax_attn_backward(tensor_t self, tensor_t attn, tensor_t v, tensor_t attn_g, tensor_t v_g) override;
    ComputingReturn op_qk_backward(tensor_t self, tensor_t q, tensor_t k, tensor_t q_g, tensor_t k_g) override;

    ComputingReturn op_flash_attn(tensor_t self, tensor_t lens, tensor_t out, tensor_t lse, int heads) override;
    ComputingReturn op_flash_attn_backward(tensor_t self, tensor_t qkv, tensor_t out, tensor_t lse, tensor_t lens, tensor_t dqkv, int heads) override;
    ComputingReturn op_linear_residual(tensor_t self, tensor_t w, tensor_t bias, tensor_t residual, tensor_t y) override;
    ComputingReturn op_linear_gelu(tensor_t self, tensor_t w, tensor_t bias, tensor_t y, tensor_t y_gelu) override;
    ComputingReturn op_embed(tensor_t self, tensor_t table, tensor_t out) override;
    ComputingReturn op_embed_backward(tensor_t self, tensor_t ids, tensor_t table_g) override;
    ComputingReturn op_adam(tensor_t self, tensor_t grad, tensor_t master, tensor_t m, tensor_t v, float lr, float beta1, float beta2, float eps, int step, float grad_scale) override;
    ComputingReturn op_randn(tensor_t self, float mean, float std, uint64_t seed) override;
    LossReturn op_token_nll(tensor_t self, tensor_t ids, tensor_t mask, tensor_t lm_head, tensor_t all_logits, tensor_t out) override;
    ComputingReturn io_nccl_sendrecv(tensor_t self, tensor_t recv, int peer) override;
    ComputingReturn io_nccl_allreduce(tensor_t self) override;
    ComputingReturn op_layernorm_backward_residual(tensor_t self, tensor_t scale, tensor_t bias, tensor_t var, tensor_t y, tensor_t dscale, tensor_t dbias, tensor_t din, tensor_t residual, float eps) override;
    ComputingReturn op_linear_backward_x(tensor_t self, tensor_t weight, tensor_t x_g) override;
    ComputingReturn op_linear_backward_w(tensor_t self, tensor_t x, tensor_t weight_g, tensor_t bias_g) override;
    ComputingReturn op_loss_backward_async(tensor_t self, tensor_t ids, tensor_t mask, tensor_t lm_head, tensor_t all_logits, tensor_t x_g, tensor_t lm_head_g, tensor_t loss_out, int defer_weight) override;
    ComputingReturn op_loss_backward_w(tensor_t self, tensor_t x, tensor_t lm_head_g) override;

    ComputingReturn io_load(tensor_t self, const char* fileName) override;
    ComputingReturn io_save(tensor_t self, const char* fileName) override;
    ComputingReturn io_dump(tensor_t self) override;
    ComputingReturn io_mpi_bcast(tensor_t self, int root) override;
    ComputingReturn io_mpi_recv(tensor_t self, int source) override;
    ComputingReturn io_mpi_send(tensor_t self, int dst) override;
    ComputingReturn io_nccl_recv(tensor_t self, int source) override;
    ComputingReturn io_nccl_send(tensor_t self, int dst) override;

private:
    ShapeType shape_;
    DataType dtype_;
    int64_t marker_ = 0;
    ImplType kind_;
    TransformerComputing* impl_;
    void* data_;
};

// Factories.  The first three are the reference's (blackriver/tensortype.hpp:315-317).
tensor_t create_cuda_float(std::vector<size_t>& shape);
tensor_t create_cpu_float(std::vector<size_t>& shape);
tensor_t create_cpu_int(std::vector<size_t>& shape);
tensor_t create_cuda_half(std::vector<size_t>& shape);
tensor_t create_cuda_int(std::vector<size_t>& shape);
tensor_t create_cpu_half(std::vector<size_t>& shape);

}  // namespace br
