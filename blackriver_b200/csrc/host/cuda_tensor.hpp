// Device tensor backend: a thin shim that turns each operator of the TransformerComputing
// interface into calls of the C-ABI kernel library (include/brk.h).  It replaces the reference's
// CUDATensor (blackriver/cuda_tensor.hpp, blackriver/cuda_tensor.cpp), which drove cuBLASLt,
// cuDNN, OpenBLAS and the LightSeq-derived kernels.  There is no CPU fallback: a failing kernel
// call is returned as its status code and the facade turns it into a fatal error.
#pragma once

#include "context.hpp"
#include "tensortype.hpp"

namespace br {

template <DataType DT>
struct CUDATensor : public TransformerComputing {
    explicit CUDATensor(const ShapeType& shape);             // owning (cudaMalloc)
    explicit CUDATensor(void* mem) : mem_(mem), owner_(false) {}  // non-owning view
    ~CUDATensor() override;

    void* data() { return mem_; }

    ComputingReturn io_dump(tensor_t self) override;
    ComputingReturn io_load(tensor_t self, const char* fileName) override;
    ComputingReturn io_save(tensor_t self, const char* fileName) override;
    ComputingReturn io_nccl_send(tensor_t self, int dst) override;
    ComputingReturn io_nccl_recv(tensor_t self, int src) override;

    ComputingReturn op_zero(tensor_t self) override;
    ComputingReturn op_fill(tensor_t self, float value) override;
    ComputingReturn op_copy(tensor_t self, tensor_t src) override;
    ViewReturn op_view(tensor_t self, size_t offset, const std::vector<size_t>& newShape) override;
    ComputingReturn op_add(tensor_t self, tensor_t b, tensor_t c) override;
    ComputingReturn op_linear(tensor_t self, tensor_t w, tensor_t bias, tensor_t y) override;
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

private:
    void* mem_;
    bool owner_;
};

}  // namespace br
