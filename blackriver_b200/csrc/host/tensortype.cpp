#include "tensortype.hpp"

#include "cpu_tensor.hpp"
#include "cuda_tensor.hpp"

namespace br {

TensorType::TensorType(cpu_float_t* t, const ShapeType& s) : shape_(s), dtype_(Float), kind_(CPU_FLOAT), impl_(t), data_(t->data()) {}
TensorType::TensorType(cpu_half_t* t, const ShapeType& s) : shape_(s), dtype_(F16), kind_(CPU_HALF), impl_(t), data_(t->data()) {}
TensorType::TensorType(cpu_int_t* t, const ShapeType& s) : shape_(s), dtype_(Int), kind_(CPU_INT), impl_(t), data_(t->data()) {}
TensorType::TensorType(cuda_float_t* t, const ShapeType& s) : shape_(s), dtype_(Float), kind_(CUDA_FLOAT), impl_(t), data_(t->data()) {}
TensorType::TensorType(cuda_half_t* t, const ShapeType& s) : shape_(s), dtype_(F16), kind_(CUDA_HALF), impl_(t), data_(t->data()) {}
TensorType::TensorType(cuda_int_t* t, const ShapeType& s) : shape_(s), dtype_(Int), kind_(CUDA_INT), impl_(t), data_(t->data()) {}

TensorType::~TensorType() { delete impl_; }

#define BR_ACCESSOR(NAME, TYPE, KIND)                                   \
    TYPE* TensorType::NAME() {                                          \
        if (kind_ != KIND) br_panic("tensor is not a " #NAME " tensor"); \
        return static_cast<TYPE*>(impl_);                               \
    }
BR_ACCESSOR(cpu_float, cpu_float_t, CPU_FLOAT)
BR_ACCESSOR(cpu_half, cpu_half_t, CPU_HALF)
BR_ACCESSOR(cpu_int, cpu_int_t, CPU_INT)
BR_ACCESSOR(cuda_float, cuda_float_t, CUDA_FLOAT)
BR_ACCESSOR(cuda_half, cuda_half_t, CUDA_HALF)
BR_ACCESSOR(cuda_int, cuda_int_t, CUDA_INT)
#undef BR_ACCESSOR

std::string TensorType::to_string() const {
    std::ostringstream ss;
    ss << device_name() << ":" << DataType_name(dtype_) << ":" << marker_ << ":[";
    for (size_t i = 0; i < shape_.dim(); i++) ss << shape_[(int)i] << (i + 1 < shape_.dim() ? " " : "");
    ss << "]";
    return ss.str();
}

#define SELF_CHECK() br_assert(self.get() == this, "an operator must be invoked as t->op(t, ...)")

ComputingReturn TensorType::op_zero(tensor_t self) {
    SELF_CHECK();
    marker_ = 0;
    auto r = impl_->op_zero(self);
    op_check(r, "zero");
}

ComputingReturn TensorType::op_fill(tensor_t self, float value) {
    SELF_CHECK();
    auto r = impl_->op_fill(self, value);
    op_check(r, "fill");
}

ComputingReturn TensorType::op_copy(tensor_t self, tensor_t src) {
    SELF_CHECK();
    br_assert(items() == src->items(), "copy needs tensors of the same size");
    auto r = impl_->op_copy(self, src);
    op_check(r, "copy");
}

// One 0 in the requested shape stands for "whatever fits from the offset on"
// (blackriver/tensortype.cpp:28-58); the view must lie inside its parent.
ViewReturn TensorType::op_view(tensor_t self, size_t offset, const std::vector<size_t>& requested) {
    SELF_CHECK();
    std::vector<size_t> dims = requested;
    int open = -1;
    size_t known = 1;
    for (size_t i = 0; i < dims.size(); i++) {
        if (dims[i] == 0) {
            br_assert(open < 0, "a view may leave at most one dimension open");
            open = (int)i;
        } else {
            known *= dims[i];
        }
    }
    br_assert(offset <= items(), "view offset outside the tensor");
    if (open >= 0) dims[open] = (items() - offset) / known;
    ShapeType s(dims);
    br_assert(offset + s.numel() <= items(), "view reaches outside the tensor");
    auto r = impl_->op_view(self, offset, dims);
    if (r.index() == 0) {
        ComputingReturn code = std::get<0>(r);
        if (code != OP_OK) br_panic("view returned " + std::to_string((int)code));
    }
    return r;
}

ComputingReturn TensorType::op_add(tensor_t self, tensor_t b, tensor_t c) {
    SELF_CHECK();
    auto r = impl_->op_add(self, b, c);
    op_check(r, "add");
}
ComputingReturn TensorType::op_mul(tensor_t self, tensor_t b, tensor_t c) {
    SELF_CHECK();
    auto r = impl_->op_mul(self, b, c);
    op_check(r, "mul");
}
ComputingReturn TensorType::op_linear(tensor_t self, tensor_t w, tensor_t b, tensor_t y) {
    SELF_CHECK();
    auto r = impl_->op_linear(self, w, b, y);
    op_check(r, "linear");
}
ComputingReturn TensorType::op_layernorm(tensor_t self, tensor_t mean, tensor_t var, tensor_t scale, tensor_t bias, tensor_t y, float eps) {
    SELF_CHECK();
    auto r = impl_->op_layernorm(self, mean, var, scale, bias, y, eps);
    op_check(r, "layernorm");
}
ComputingReturn TensorType::op_transpos_0213(tensor_t self, tensor_t y) {
    SELF_CHECK();
    auto r = impl_->op_transpos_0213(self, y);
    op_check(r, "transpos_0213");
}
ComputingReturn TensorType::op_qk(tensor_t self, tensor_t k, tensor_t qk) {
    SELF_CHECK();
    auto r = impl_->op_qk(self, k, qk);
    op_check(r, "qk");
}
ComputingReturn TensorType::op_softmax(tensor_t self, tensor_t out) {
    SELF_CHECK();
    auto r = impl_->op_softmax(self, out);
    op_check(r, "softmax");
}
ComputingReturn TensorType::op_attn(tensor_t self, tensor_t v, tensor_t attn) {
    SELF_CHECK();
    auto r = impl_->op_attn(self, v, attn);
    op_check(r, "attn");
}
ComputingReturn TensorType::op_gelu(tensor_t self, tensor_t dst) {
    SELF_CHECK();
    auto r = impl_->op_gelu(self, dst);
    op_check(r, "gelu");
}
ComputingReturn TensorType::op_last_logits(tensor_t self, tensor_t mask, tensor_t lm_head, tensor_t output) {
    SELF_CHECK();
    auto r = impl_->op_last_logits(self, mask, lm_head, output);
    op_check(r, "last_logits");
}
LossReturn TensorType::op_loss_backward(tensor_t self, tensor_t ids, tensor_t mask, tensor_t lm_head, tensor_t all_logits, tensor_t x_g, tensor_t lm_head_g) {
    SELF_CHECK();
    auto r = impl_->op_loss_backward(self, ids, mask, lm_head, all_logits, x_g, lm_head_g);
    if (r.index() == 0) {
        ComputingReturn code = std::get<0>(r);
        if (code != OP_OK) br_panic("loss_backward returned " + std::to_string((int)code));
    }
    return r;
}
LossReturn TensorType::op_token_nll(tensor_t self, tensor_t ids, tensor_t mask, tensor_t lm_head, tensor_t all_logits, tensor_t out) {
    SELF_CHECK();
    auto r = impl_->op_token_nll(self, ids, mask, lm_head, all_logits, out);
    if (r.index() == 0) {
        ComputingReturn code = std::get<0>(r);
        if (code != OP_OK) br_panic("token_nll returned " + std::to_string((int)code));
    }
    return r;
}
ComputingReturn TensorType::op_layernorm_backward(tensor_t self, tensor_t scale, tensor_t bias, tensor_t var, tensor_t y, tensor_t dscale, tensor_t dbias, tensor_t din, float eps) {
    SELF_CHECK();
    auto r = impl_->op_layernorm_backward(self, scale, bias, var, y, dscale, dbias, din, eps);
    op_check(r, "layernorm_backward");
}
ComputingReturn TensorType::op_layernorm_backward_residual(tensor_t self, tensor_t scale, tensor_t bias, tensor_t var, tensor_t y, tensor_t dscale, tensor_t dbias, tensor_t din, tensor_t residual, float eps) {
    SELF_CHECK();
    auto r = impl_->op_layernorm_backward_residual(self, scale, bias, var, y, dscale, dbias, din, residual, eps);
    op_check(r, "layernorm_backward_residual");
}
ComputingReturn TensorType::op_linear_backward(tensor_t self, tensor_t x, tensor_t weight, tensor_t bias, tensor_t x_g, tensor_t weight_g, tensor_t bias_g) {
    SELF_CHECK();
    auto r = impl_->op_linear_backward(self, x, weight, bias, x_g, weight_g, bias_g);
    op_check(r, "linear_backward");
}
ComputingReturn TensorType::op_gelu_backward(tensor_t self, tensor_t x, tensor_t x_g) {
    SELF_CHECK();
    auto r = impl_->op_gelu_backward(self, x, x_g);
    op_check(r, "gelu_backward");
}
ComputingReturn TensorType::op_attn_backward(tensor_t self, tensor_t attn, tensor_t v, tensor_t attn_g, tensor_t v_g) {
    SELF_CHECK();
    auto r = impl_->op_attn_backward(self, attn, v, attn_g, v_g);
    op_check(r, "attn_backward");
}
ComputingReturn TensorType::op_softmax_backward(tensor_t self, tensor_t out, tensor_t x_g) {
    SELF_CHECK();
    auto r = impl_->op_softmax_backward(self, out, x_g);
    op_check(r, "softmax_backward");
}
ComputingReturn TensorType::op_softmax_attn_backward(tensor_t self, tensor_t attn, tensor_t v, tensor_t attn_g, tensor_t v_g) {
    SELF_CHECK();
    auto r = impl_->op_softmax_attn_backward(self, attn, v, attn_g, v_g);
    op_check(r, "softmax_attn_backward");
}
ComputingReturn TensorType::op_qk_backward(tensor_t self, tensor_t q, tensor_t k, tensor_t q_g, tensor_t k_g) {
    SELF_CHECK();
    auto r = impl_->op_qk_backward(self, q, k, q_g, k_g);
    op_check(r, "qk_backward");
}

ComputingReturn TensorType::op_flash_attn(tensor_t self, tensor_t lens, tensor_t out, tensor_t lse, int heads) {
    SELF_CHECK();
    auto r = impl_->op_flash_attn(self, lens, out, lse, heads);
    op_check(r, "flash_attn");
}
ComputingReturn TensorType::op_flash_attn_backward(tensor_t self, tensor_t qkv, tensor_t out, tensor_t lse, tensor_t lens, tensor_t dqkv, int heads) {
    SELF_CHECK();
    auto r = impl_->op_flash_attn_backward(self, qkv, out, lse, lens, dqkv, heads);
    op_check(r, "flash_attn_backward");
}
ComputingReturn TensorType::op_linear_residual(tensor_t self, tensor_t w, tensor_t bias, tensor_t residual, tensor_t y) {
    SELF_CHECK();
    auto r = impl_->op_linear_residual(self, w, bias, residual, y);
    op_check(r, "linear_residual");
}
ComputingReturn TensorType::op_linear_gelu(tensor_t self, tensor_t w, tensor_t bias, tensor_t y, tensor_t y_gelu) {
    SELF_CHECK();
    auto r = impl_->op_linear_gelu(self, w, bias, y, y_gelu);
    op_check(r, "linear_gelu");
}
ComputingReturn TensorType::op_embed(tensor_t self, tensor_t table, tensor_t out) {
    SELF_CHECK();
    // ids may live on the host: the math runs in the table's backend
    auto r = table->impl()->op_embed(self, table, out);
    op_check(r, "embed");
}
ComputingReturn TensorType::op_embed_backward(tensor_t self, tensor_t ids, tensor_t table_g) {
    SELF_CHECK();
    auto r = impl_->op_embed_backward(self, ids, table_g);
    op_check(r, "embed_backward");
}
ComputingReturn TensorType::op_adam(tensor_t self, tensor_t grad, tensor_t master, tensor_t m, tensor_t v, float lr, float beta1, float beta2, float eps, int step, float grad_scale) {
    SELF_CHECK();
    auto r = impl_->op_adam(self, grad, master, m, v, lr, beta1, beta2, eps, step, grad_scale);
    op_check(r, "adam");
}
ComputingReturn TensorType::op_randn(tensor_t self, float mean, float std, uint64_t seed) {
    SELF_CHECK();
    auto r = impl_->op_randn(self, mean, std, seed);
    op_check(r, "randn");
}

ComputingReturn TensorType::io_nccl_sendrecv(tensor_t self, tensor_t recv, int peer) {
    SELF_CHECK();
    auto r = impl_->io_nccl_sendrecv(self, recv, peer);
    op_check(r, "nccl_sendrecv");
}

ComputingReturn TensorType::io_nccl_allreduce(tensor_t self) {
    SELF_CHECK();
    auto r = impl_->io_nccl_allreduce(self);
    op_check(r, "nccl_allreduce");
}

ComputingReturn TensorType::op_linear_backward_x(tensor_t self, tensor_t weight, tensor_t x_g) {
    SELF_CHECK();
    auto r = impl_->op_linear_backward_x(self, weight, x_g);
    op_check(r, "linear_backward_x");
}
ComputingReturn TensorType::op_linear_backward_w(tensor_t self, tensor_t x, tensor_t weight_g, tensor_t bias_g) {
    SELF_CHECK();
    auto r = impl_->op_linear_backward_w(self, x, weight_g, bias_g);
    op_check(r, "linear_backward_w");
}
ComputingReturn TensorType::op_loss_backward_async(tensor_t self, tensor_t ids, tensor_t mask, tensor_t lm_head, tensor_t all_logits, tensor_t x_g, tensor_t lm_head_g, tensor_t loss_out, int defer_weight) {
    SELF_CHECK();
    auto r = impl_->op_loss_backward_async(self, ids, mask, lm_head, all_logits, x_g, lm_head_g, loss_out, defer_weight);
    op_check(r, "loss_backward_async");
}
ComputingReturn TensorType::op_loss_backward_w(tensor_t self, tensor_t x, tensor_t lm_head_g) {
    SELF_CHECK();
    auto r = impl_->op_loss_backward_w(self, x, lm_head_g);
    op_check(r, "loss_backward_w");
}

ComputingReturn TensorType::io_load(tensor_t self, const char* fileName) {
    SELF_CHECK();
    auto r = impl_->io_load(self, fileName);
    op_check(r, "load");
}
ComputingReturn TensorType::io_save(tensor_t self, const char* fileName) {
    SELF_CHECK();
    auto r = impl_->io_save(self, fileName);
    op_check(r, "save");
}
ComputingReturn TensorType::io_dump(tensor_t self) {
    SELF_CHECK();
    auto r = impl_->io_dump(self);
    op_check(r, "dump");
}
ComputingReturn TensorType::io_mpi_bcast(tensor_t self, int root) {
    SELF_CHECK();
    auto r = impl_->io_mpi_bcast(self, root);
    op_check(r, "mpi_bcast");
}
ComputingReturn TensorType::io_mpi_recv(tensor_t self, int source) {
    SELF_CHECK();
    auto r = impl_->io_mpi_recv(self, source);
    op_check(r, "mpi_recv");
}
ComputingReturn TensorType::io_mpi_send(tensor_t self, int dst) {
    SELF_CHECK();
    auto r = impl_->io_mpi_send(self, dst);
    op_check(r, "mpi_send");
}
ComputingReturn TensorType::io_nccl_recv(tensor_t self, int source) {
    SELF_CHECK();
    auto r = impl_->io_nccl_recv(self, source);
    op_check(r, "nccl_recv");
}
ComputingReturn TensorType::io_nccl_send(tensor_t self, int dst) {
    SELF_CHECK();
    auto r = impl_->io_nccl_send(self, dst);
    op_check(r, "nccl_send");
}

}  // namespace br
