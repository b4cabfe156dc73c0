// The tensor-operator interface of BlackRiver: the drop-in boundary.
//
// Method names, argument order, argument meaning and return conventions are those of
// br::TransformerComputing in the reference (blackriver/operators.hpp:20-112); scripts and
// word bindings written against the reference call these unchanged.  Every method gets the
// tensor it is invoked on a second time as `self` (a shared_ptr to the same object), outputs
// are caller-allocated tensors, and the default implementation answers OP_TODO_ERROR so that a
// backend only overrides what it supports.
#pragma once

#include <cstdint>
#include <memory>
#include <variant>
#include <vector>

namespace br {

struct TensorType;
using tensor_t = std::shared_ptr<TensorType>;

// blackriver/operators.hpp:12-18.  The kernel library's status codes reuse these values.
enum ComputingReturn {
    OP_OK = 0,
    OP_TODO_ERROR = -1,
    OP_INPUT_ERROR = -2,
    OP_OUTPUT_ERROR = -3,
    OP_ATTR_ERROR = -4,
};

using ViewReturn = std::variant<ComputingReturn, tensor_t>;
using LossReturn = std::variant<ComputingReturn, float>;

struct TransformerComputing {
    virtual ~TransformerComputing() = default;

    // ---- io: files, host transport, device transport (operators.hpp:21-44) ----
    virtual ComputingReturn io_load(tensor_t self, const char* fileName) { return OP_TODO_ERROR; }
    virtual ComputingReturn io_save(tensor_t self, const char* fileName) { return OP_TODO_ERROR; }
    virtual ComputingReturn io_dump(tensor_t self) { return OP_TODO_ERROR; }
    virtual ComputingReturn io_mpi_bcast(tensor_t self, int root) { return OP_TODO_ERROR; }
    virtual ComputingReturn io_mpi_recv(tensor_t self, int source) { return OP_TODO_ERROR; }
    virtual ComputingReturn io_mpi_send(tensor_t self, int dst) { return OP_TODO_ERROR; }
    virtual ComputingReturn io_nccl_recv(tensor_t self, int source) { return OP_TODO_ERROR; }
    virtual ComputingReturn io_nccl_send(tensor_t self, int dst) { return OP_TODO_ERROR; }

    // ---- storage ops (operators.hpp:46-57) ----
    virtual ComputingReturn op_zero(tensor_t self) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_fill(tensor_t self, float value) { return OP_TODO_ERROR; }
    // copies `src` INTO self (the reference names the parameter dst in one place and src in another;
    // every caller passes the source, nn.cpp:71-78)
    virtual ComputingReturn op_copy(tensor_t self, tensor_t src) { return OP_TODO_ERROR; }
    // non-owning view of `self` at an element offset; one 0 in newShape means "infer"
    virtual ViewReturn op_view(tensor_t self, size_t offset, const std::vector<size_t>& newShape) { return OP_TODO_ERROR; }

    // ---- forward math (operators.hpp:58-87) ----
    virtual ComputingReturn op_add(tensor_t self, tensor_t b, tensor_t c) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_mul(tensor_t self, tensor_t b, tensor_t c) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_linear(tensor_t self, tensor_t w, tensor_t bias, tensor_t y) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_layernorm(tensor_t self, tensor_t mean, tensor_t var, tensor_t scale, tensor_t bias,
                                         tensor_t y, float eps) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_transpos_0213(tensor_t self, tensor_t y) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_qk(tensor_t self, tensor_t k, tensor_t qk) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_softmax(tensor_t self, tensor_t out) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_attn(tensor_t self, tensor_t v, tensor_t attn) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_gelu(tensor_t self, tensor_t dst) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_last_logits(tensor_t self, tensor_t mask, tensor_t lm_head, tensor_t output) { return OP_TODO_ERROR; }

    // ---- loss and backward math (operators.hpp:88-111) ----
    virtual LossReturn op_loss_backward(tensor_t self, tensor_t ids, tensor_t mask, tensor_t lm_head, tensor_t all_logits,
                                        tensor_t x_g, tensor_t lm_head_g) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_layernorm_backward(tensor_t self, tensor_t scale, tensor_t bias, tensor_t var, tensor_t y,
                                                  tensor_t dscale, tensor_t dbias, tensor_t din, float eps) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_linear_backward(tensor_t self, tensor_t x, tensor_t weight, tensor_t bias, tensor_t x_g,
                                               tensor_t weight_g, tensor_t bias_g) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_gelu_backward(tensor_t self, tensor_t x, tensor_t x_g) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_attn_backward(tensor_t self, tensor_t attn, tensor_t v, tensor_t attn_g, tensor_t v_g) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_softmax_backward(tensor_t self, tensor_t out, tensor_t x_g) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_softmax_attn_backward(tensor_t self, tensor_t attn, tensor_t v, tensor_t attn_g, tensor_t v_g) { return OP_TODO_ERROR; }
    virtual ComputingReturn op_qk_backward(tensor_t self, tensor_t q, tensor_t k, tensor_t q_g, tensor_t k_g) { return OP_TODO_ERROR; }

    // ---- extensions: not part of the reference interface (operators.hpp there ends above) ----
    // Fused attention on the fused QKV projection.  self = qkv [B,T,3H] (q | k | v thirds), lens = int
    // [B] valid lengths (host or device), out [B,T,H], lse [B,heads,T] fp32.  Stands for the
    // transpos_0213 x3 / querykey / add alibi / add xmask / softmax / attn / transpos_0213 chain.
    virtual ComputingReturn op_flash_attn(tensor_t self, tensor_t lens, tensor_t out, tensor_t lse, int heads) { return OP_TODO_ERROR; }
    // self = d_out [B,T,H]; writes dqkv [B,T,3H].
    virtual ComputingReturn op_flash_attn_backward(tensor_t self, tensor_t qkv, tensor_t out, tensor_t lse, tensor_t lens,
                                                   tensor_t dqkv, int heads) { return OP_TODO_ERROR; }
    // y = x W^T + b + residual  (op_linear followed by op_add, in the GEMM epilogue)
    virtual ComputingReturn op_linear_residual(tensor_t self, tensor_t w, tensor_t bias, tensor_t residual, tensor_t y) { return OP_TODO_ERROR; }
    // y = x W^T + b ; y_gelu = bloom_gelu(y)  (op_linear followed by op_gelu, in the GEMM epilogue)
    virtual ComputingReturn op_linear_gelu(tensor_t self, tensor_t w, tensor_t bias, tensor_t y, tensor_t y_gelu) { return OP_TODO_ERROR; }
    // self = ids (int, host or device) ; out[i,:] = table[ids[i],:]   (the feeder rank's gather, on the device)
    virtual ComputingReturn op_embed(tensor_t self, tensor_t table, tensor_t out) { return OP_TODO_ERROR; }
    // self = dx ; table_g[ids[i],:] += dx[i,:]
    virtual ComputingReturn op_embed_backward(tensor_t self, tensor_t ids, tensor_t table_g) { return OP_TODO_ERROR; }
    // self = working weights (fp16 or fp32) ; Adam on fp32 master / m / v, gradient multiplied by grad_scale
    virtual ComputingReturn op_adam(tensor_t self, tensor_t grad, tensor_t master, tensor_t m, tensor_t v, float lr, float beta1,
                                    float beta2, float eps, int step, float grad_scale) { return OP_TODO_ERROR; }
    // simultaneous exchange with one peer: send self, receive into `recv` (one NCCL group, so two ranks
    // that both call it towards each other cannot block one another)
    virtual ComputingReturn io_nccl_sendrecv(tensor_t self, tensor_t recv, int peer) { return OP_TODO_ERROR; }
    // op_layernorm_backward with the residual branch folded in: din = residual + (input gradient of the LayerNorm);
    // residual may be din
    virtual ComputingReturn op_layernorm_backward_residual(tensor_t self, tensor_t scale, tensor_t bias, tensor_t var, tensor_t y,
                                                           tensor_t dscale, tensor_t dbias, tensor_t din, tensor_t residual, float eps) {
        return OP_TODO_ERROR;
    }
    // self <- sum of self over the data-parallel replicas (in place; nothing to do with one replica)
    virtual ComputingReturn io_nccl_allreduce(tensor_t self) { return OP_TODO_ERROR; }
    // self[i] ~ N(mean, std), seeded
    virtual ComputingReturn op_randn(tensor_t self, float mean, float std, uint64_t seed) { return OP_TODO_ERROR; }
    // forward-only scoring: out[b, t] (fp32) = NLL of ids[b, t+1] given position t of self [batch, tokens, hidden], 0 where the
    // pair (t, t+1) is not counted (same target rule as op_loss_backward); returns the mean over the counted positions
    virtual LossReturn op_token_nll(tensor_t self, tensor_t ids, tensor_t mask, tensor_t lm_head, tensor_t all_logits, tensor_t out) {
        return OP_TODO_ERROR;
    }
    // The two halves of op_linear_backward, so that a pipeline stage can hand x_g to its predecessor before it spends
    // time on its own weight gradients: self = dy ; x_g = dy W (overwritten)
    virtual ComputingReturn op_linear_backward_x(tensor_t self, tensor_t weight, tensor_t x_g) { return OP_TODO_ERROR; }
    // self = dy ; b_g = sum_n dy ; W_g = dy^T x (overwritten, or added to under op.accumulate)
    virtual ComputingReturn op_linear_backward_w(tensor_t self, tensor_t x, tensor_t weight_g, tensor_t bias_g) { return OP_TODO_ERROR; }
    // op_loss_backward without a host round trip: the 1/items factor is formed on the device and the mean loss goes to
    // loss_out[0] (device fp32) instead of being returned.  With defer_weight != 0 (needs a logits band covering every
    // row) the LM-head weight gradient is left out; op_loss_backward_w adds it later from the band, which then still
    // holds the logits' gradient.
    virtual ComputingReturn op_loss_backward_async(tensor_t self, tensor_t ids, tensor_t mask, tensor_t lm_head, tensor_t all_logits,
                                                   tensor_t x_g, tensor_t lm_head_g, tensor_t loss_out, int defer_weight) { return OP_TODO_ERROR; }
    // self = the band holding dlogits [rows, vocab] ; lm_head_g += dlogits^T x
    virtual ComputingReturn op_loss_backward_w(tensor_t self, tensor_t x, tensor_t lm_head_g) { return OP_TODO_ERROR; }
};

}  // namespace br
