#include "cuda_tensor.hpp"

#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <utility>
#include <vector>

#include "brk.h"
#include "cpu_tensor.hpp"

namespace br {

namespace {

inline cudaStream_t stream() { return ComputingContext::cuda_stream; }
// NCCL transfers go to the transfer stream while a script has forked it (op.stream.fork ... op.stream.join)
inline cudaStream_t nccl_stream() { return ComputingContext::nccl_on_comm_stream ? ComputingContext::comm_stream : ComputingContext::cuda_stream; }
inline void* sptr() { return (void*)ComputingContext::cuda_stream; }

template <DataType DT> constexpr int brk_dtype() { return DT == DataType::F16 ? BRK_F16 : BRK_F32; }

// status of the kernel library -> operator status (the first four codes coincide)
inline ComputingReturn ret(int st) {
    if (st == BRK_OK) return OP_OK;
    if (st == BRK_CUDA_ERROR) {
        std::cerr << "kernel library: " << brk_last_cuda_error() << std::endl;
        return OP_OUTPUT_ERROR;
    }
    return (ComputingReturn)st;
}

struct ProfScope {
    explicit ProfScope(const char* family) { Profiler::begin(family); }
    ~ProfScope() { Profiler::end(); }
};

// all operands of a math op must be device tensors of the op's element type
template <DataType DT>
inline bool dev_ok(std::initializer_list<tensor_t> ts) {
    for (auto& t : ts)
        if (!t || !t->is_cuda() || t->dtype() != DT) return false;
    return true;
}

inline void dims4(const ShapeType& s, int64_t out[4]) {
    br_assert(s.dim() <= 4, "at most 4 dimensions");
    size_t pad = 4 - s.dim();
    for (size_t i = 0; i < 4; i++) out[i] = i < pad ? 1 : (int64_t)s[(int)(i - pad)];
}

// carve aligned pieces out of the device scratch
struct Scratch {
    unsigned char* p = (unsigned char*)ComputingContext::cuda_workspace;
    size_t left = ComputingContext::workspace_size;
    void* take(size_t bytes) {
        size_t need = (bytes + 255) / 256 * 256;
        br_assert(need <= left, "device scratch exhausted");
        void* r = p;
        p += need;
        left -= need;
        return r;
    }
};

// int32 tensor -> device pointer; host tensors are staged through `scratch`
inline const int32_t* int_on_device(const tensor_t& t, Scratch& sc) {
    if (t->is_cuda()) return (const int32_t*)t->data();
    int32_t* d = (int32_t*)sc.take(t->bytes());
    BR_CUDA_CHECK(cudaMemcpyAsync(d, t->data(), t->bytes(), cudaMemcpyHostToDevice, stream()));
    return d;
}

// One GEMM, routed to the tensor-core kernel when the element type is fp16 and the layout meets
// TMA's rules (single problem, alpha 1, beta 0 or 1), otherwise to the general SIMT kernel.
template <DataType DT>
inline int gemm_any(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int ta, int tb, int64_t lda,
                    int64_t ldb, int64_t ldc, float beta, const void* bias) {
    ProfScope prof(DT == DataType::F16 ? "gemm_f16" : "gemm_f32");
    if (DT == DataType::F16 && (beta == 0.0f || beta == 1.0f) && brk_gemm_f16_supported(m, n, k, ta, tb, lda, ldb, a, b))
        return brk_gemm_f16(a, b, c, m, n, k, ta, tb, lda, ldb, ldc, bias, nullptr, 0, nullptr, 0, beta == 1.0f ? 1 : 0, sptr());
    return brk_gemm(a, b, c, m, n, k, ta, tb, lda, ldb, ldc, 1, 0, 0, 0, 1.0f, beta, bias, brk_dtype<DT>(), sptr());
}

}  // namespace

template <DataType DT>
CUDATensor<DT>::CUDATensor(const ShapeType& shape) : owner_(true) {
    BR_CUDA_CHECK(cudaMalloc(&mem_, std::max<size_t>(shape.numel() * DataType_size(DT), 16)));
}

template <DataType DT>
CUDATensor<DT>::~CUDATensor() {
    if (owner_ && mem_) cudaFree(mem_);
}

// ---- io ----------------------------------------------------------------------------------------
template <DataType DT>
ComputingReturn CUDATensor<DT>::io_dump(tensor_t self) {
    size_t n = std::min<size_t>(self->shape().vec().back(), 8);
    const size_t es = DataType_size(DT);
    unsigned char first[32], last[32];
    BR_CUDA_CHECK(cudaMemcpyAsync(first, mem_, n * es, cudaMemcpyDeviceToHost, stream()));
    BR_CUDA_CHECK(cudaMemcpyAsync(last, (unsigned char*)mem_ + (self->items() - n) * es, n * es, cudaMemcpyDeviceToHost, stream()));
    BR_CUDA_CHECK(cudaStreamSynchronize(stream()));
    auto val = [&](unsigned char* b, size_t i) -> double {
        if (DT == DataType::Float) return ((float*)b)[i];
        if (DT == DataType::Int) return ((int*)b)[i];
        return __half2float(((__half*)b)[i]);
    };
    std::cout << "--------------------------\nFirst " << n << " : ";
    for (size_t i = 0; i < n; i++) std::cout << val(first, i) << " ";
    std::cout << "\nLast " << n << " : ";
    for (size_t i = 0; i < n; i++) std::cout << val(last, i) << " ";
    std::cout << std::endl;
    return OP_OK;
}

// Raw file -> device (blackriver/cuda_tensor.cpp:57-72).  fp16 tensors also accept fp32 files.
template <DataType DT>
ComputingReturn CUDATensor<DT>::io_load(tensor_t self, const char* fileName) {
    std::vector<unsigned char> raw;
    read_data(fileName, raw);
    std::vector<__half> conv;
    const void* src = raw.data();
    if (raw.size() != self->bytes()) {
        if (!(DT == DataType::F16 && raw.size() == self->items() * 4)) return OP_INPUT_ERROR;
        conv.resize(self->items());
        const float* f = reinterpret_cast<const float*>(raw.data());
        for (size_t i = 0; i < conv.size(); i++) conv[i] = __float2half(f[i]);
        src = conv.data();
    }
    BR_CUDA_CHECK(cudaMemcpyAsync(mem_, src, self->bytes(), cudaMemcpyHostToDevice, stream()));
    BR_CUDA_CHECK(cudaStreamSynchronize(stream()));  // the staging vectors die with this frame
    return OP_OK;
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::io_save(tensor_t self, const char* fileName) {
    std::vector<unsigned char> raw(self->bytes());
    BR_CUDA_CHECK(cudaMemcpyAsync(raw.data(), mem_, raw.size(), cudaMemcpyDeviceToHost, stream()));
    BR_CUDA_CHECK(cudaStreamSynchronize(stream()));
    std::ofstream out(fileName, std::ios::binary);
    if (!out) return OP_OUTPUT_ERROR;
    out.write(reinterpret_cast<const char*>(raw.data()), (std::streamsize)raw.size());
    return out ? OP_OK : OP_OUTPUT_ERROR;
}

// Stage hand-off on the compute stream, in program order with the kernels around it
// (blackriver/cuda_tensor.cpp:75-96).  The overlapped pipeline does not use these: it moves activations and
// gradients with the one-sided io.link.* words (PipeLinks), which never occupy the compute stream.
template <DataType DT>
ComputingReturn CUDATensor<DT>::io_nccl_send(tensor_t self, int dst) {
    if (!CollectiveContext::has_comm) return OP_ATTR_ERROR;
    BR_NCCL_CHECK(ncclSend(mem_, self->bytes(), ncclChar, dst, CollectiveContext::nccl_comm, stream()));
    return OP_OK;
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::io_nccl_recv(tensor_t self, int src) {
    if (!CollectiveContext::has_comm) return OP_ATTR_ERROR;
    BR_NCCL_CHECK(ncclRecv(mem_, self->bytes(), ncclChar, src, CollectiveContext::nccl_comm, stream()));
    return OP_OK;
}

// ---- storage -------------------------------------------------------------------------------------
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_zero(tensor_t self) {
    BR_CUDA_CHECK(cudaMemsetAsync(mem_, 0, self->bytes(), stream()));
    return OP_OK;
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_fill(tensor_t self, float value) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    return ret(brk_fill(mem_, value, (int64_t)self->items(), brk_dtype<DT>(), sptr()));
}

// self <- src from host or device memory (blackriver/cuda_tensor.cpp:127-144); a dtype change
// between fp32 and fp16 device tensors converts.
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_copy(tensor_t self, tensor_t src) {
    if (src->dtype() == DT) {
        auto kind = src->is_cpu() ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
        BR_CUDA_CHECK(cudaMemcpyAsync(mem_, src->data(), self->bytes(), kind, stream()));
        return OP_OK;
    }
    if (src->is_cuda() && DT != DataType::Int && src->dtype() != DataType::Int) {
        int sd = src->dtype() == DataType::F16 ? BRK_F16 : BRK_F32;
        return ret(brk_cast(src->data(), sd, mem_, brk_dtype<DT>(), (int64_t)self->items(), sptr()));
    }
    return OP_INPUT_ERROR;
}

template <DataType DT>
ViewReturn CUDATensor<DT>::op_view(tensor_t self, size_t offset, const std::vector<size_t>& newShape) {
    ShapeType shape(newShape);
    void* p = static_cast<unsigned char*>(mem_) + offset * DataType_size(DT);
    return std::make_shared<TensorType>(new CUDATensor<DT>(p), shape);
}

// ---- forward math ----------------------------------------------------------------------------------
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_add(tensor_t self, tensor_t b, tensor_t c) {
    ProfScope prof("add");
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({b})) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({c}) || c->items() != self->items()) return OP_OUTPUT_ERROR;
    if (self->shape().dim() > 4 || b->shape().dim() > 4) return OP_INPUT_ERROR;
    int64_t ad[4], bd[4];
    dims4(self->shape(), ad);
    dims4(b->shape(), bd);
    return ret(brk_add_bcast(mem_, b->data(), c->data(), ad, bd, brk_dtype<DT>(), sptr()));
}

// y[n,o] = sum_i x[n,i] w[o,i] + b[o]   (blackriver/cuda_tensor.cpp:147-193)
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_linear(tensor_t self, tensor_t w, tensor_t bias, tensor_t y) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({w, bias}) || w->shape().dim() != 2) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({y})) return OP_OUTPUT_ERROR;
    int64_t in = (int64_t)self->shape().vec().back();
    int64_t out = (int64_t)w->shape()[0];
    if ((int64_t)w->shape()[1] != in || (int64_t)bias->items() != out) return OP_INPUT_ERROR;
    int64_t n = (int64_t)self->items() / in;
    if ((int64_t)y->items() != n * out) return OP_OUTPUT_ERROR;
    return ret(gemm_any<DT>(mem_, w->data(), y->data(), n, out, in, 0, 1, in, in, out, 0.0f, bias->data()));
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_layernorm(tensor_t self, tensor_t mean, tensor_t var, tensor_t scale, tensor_t bias, tensor_t y, float eps) {
    ProfScope prof("layernorm_fwd");
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({scale, bias})) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({y}) || !dev_ok<DataType::Float>({mean, var})) return OP_OUTPUT_ERROR;
    int64_t hidden = (int64_t)self->shape().vec().back();
    int64_t rows = (int64_t)self->items() / hidden;
    if ((int64_t)scale->items() != hidden || (int64_t)bias->items() != hidden) return OP_INPUT_ERROR;
    if ((int64_t)mean->items() < rows || (int64_t)var->items() < rows || y->items() != self->items()) return OP_OUTPUT_ERROR;
    return ret(brk_layernorm_fwd(mem_, scale->data(), bias->data(), y->data(), (float*)mean->data(), (float*)var->data(), rows,
                                 hidden, eps, brk_dtype<DT>(), sptr()));
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_transpos_0213(tensor_t self, tensor_t y) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->shape().dim() != 4) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({y}) || y->items() != self->items()) return OP_OUTPUT_ERROR;
    auto& s = self->shape();
    return ret(brk_transpose_0213(mem_, y->data(), s[0], s[1], s[2], s[3], brk_dtype<DT>(), sptr()));
}

// S = Q K^T / sqrt(d) per (batch, head)   (blackriver/cuda_tensor.cpp:278-330)
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_qk(tensor_t self, tensor_t k, tensor_t qk) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->shape().dim() != 4 || !dev_ok<DT>({k}) || !self->same_shape(k)) return OP_INPUT_ERROR;
    auto& s = self->shape();
    int64_t bh = s[0] * s[1], t = s[2], d = s[3];
    if (!dev_ok<DT>({qk}) || (int64_t)qk->items() != bh * t * t) return OP_OUTPUT_ERROR;
    float alpha = (float)(1.0 / std::sqrt((double)d));
    return ret(brk_gemm(mem_, k->data(), qk->data(), t, t, d, 0, 1, d, d, t, bh, t * d, t * d, t * t, alpha, 0.0f, nullptr,
                        brk_dtype<DT>(), sptr()));
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_softmax(tensor_t self, tensor_t out) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({out}) || out->items() != self->items()) return OP_OUTPUT_ERROR;
    int64_t cols = (int64_t)self->shape().vec().back();
    return ret(brk_softmax_fwd(mem_, out->data(), (int64_t)self->items() / cols, cols, brk_dtype<DT>(), sptr()));
}

// O = P V   (blackriver/cuda_tensor.cpp:359-398)
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_attn(tensor_t self, tensor_t v, tensor_t attn) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->shape().dim() != 4 || !dev_ok<DT>({v}) || v->shape().dim() != 4) return OP_INPUT_ERROR;
    auto& s = self->shape();
    int64_t bh = s[0] * s[1], t = s[2], d = v->shape()[3];
    if (!dev_ok<DT>({attn}) || attn->items() != v->items()) return OP_OUTPUT_ERROR;
    return ret(brk_gemm(mem_, v->data(), attn->data(), t, d, t, 0, 0, t, d, d, bh, t * t, t * d, t * d, 1.0f, 0.0f, nullptr,
                        brk_dtype<DT>(), sptr()));
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_gelu(tensor_t self, tensor_t dst) {
    ProfScope prof("gelu_fwd");
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({dst}) || dst->items() != self->items()) return OP_OUTPUT_ERROR;
    return ret(brk_gelu_fwd(mem_, dst->data(), (int64_t)self->items(), brk_dtype<DT>(), sptr()));
}

// out[b] = W_lm x[b, t*], t* = first i with mask[i+1] == 0, or 0 when there is none
// (blackriver/cuda_tensor.cpp:415-462; a full-length row therefore reads token 0, as there).
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_last_logits(tensor_t self, tensor_t mask_, tensor_t lm_head, tensor_t output) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->shape().dim() != 3 || !dev_ok<DT>({lm_head}) || !mask_ || !mask_->is_cpu() || mask_->dtype() != DataType::Int) return OP_INPUT_ERROR;
    int64_t batch = self->shape()[0], tokens = self->shape()[1], hidden = self->shape()[2];
    int64_t vocab = lm_head->shape()[0];
    if (!dev_ok<DT>({output}) || (int64_t)output->items() != batch * vocab) return OP_OUTPUT_ERROR;
    const int* mask = (const int*)mask_->data();
    const size_t es = DataType_size(DT);
    for (int64_t b = 0; b < batch; b++) {
        const int* m = mask + b * tokens;
        int64_t target = 0;
        for (int64_t i = 0; i < tokens - 1; i++)
            if (m[i + 1] == 0) { target = i; break; }
        const unsigned char* x = (const unsigned char*)mem_ + (b * tokens + target) * hidden * es;
        unsigned char* dst = (unsigned char*)output->data() + b * vocab * es;
        int st = brk_gemm(x, lm_head->data(), dst, 1, vocab, hidden, 0, 1, hidden, hidden, vocab, 1, 0, 0, 0, 1.0f, 0.0f, nullptr,
                          brk_dtype<DT>(), sptr());
        if (st != BRK_OK) return ret(st);
    }
    return OP_OK;
}

// ---- loss ------------------------------------------------------------------------------------------
// Shifted causal-LM cross-entropy with its gradients (blackriver/cuda_tensor.cpp:465-697).
// x = self [B,T,H] (after ln_f); ids, mask [B,T] int32 on the host or on the device; lm_head
// [V,H]; all_logits is device scratch for bands of logits ([rows,V], rows >= 1); x_g [B,T,H] is
// overwritten; lm_head_g [V,H] is ACCUMULATED into, on the device or (as in the reference) on the
// host.  Returns the mean NLL over counted positions (the reference returns the same magnitude
// with the opposite sign).  Everything stays on the device: one logits GEMM, one fused
// log-softmax/NLL/gradient kernel and two gradient GEMMs per band, no per-band synchronisation.
template <DataType DT>
LossReturn CUDATensor<DT>::op_loss_backward(tensor_t self, tensor_t ids_, tensor_t mask_, tensor_t lm_head, tensor_t all_logits,
                                            tensor_t x_g, tensor_t lm_head_g) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->shape().dim() != 3 || !dev_ok<DT>({lm_head, all_logits})) return OP_INPUT_ERROR;
    if (!ids_ || !mask_ || ids_->dtype() != DataType::Int || mask_->dtype() != DataType::Int) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({x_g}) || x_g->items() != self->items() || !lm_head_g || lm_head_g->items() != lm_head->items()) return OP_OUTPUT_ERROR;
    const int batch = (int)self->shape()[0], tokens = (int)self->shape()[1];
    const int64_t hidden = self->shape()[2], vocab = lm_head->shape()[0];
    const int64_t n = (int64_t)batch * tokens;
    if ((int64_t)ids_->items() < n || (int64_t)mask_->items() < n) return OP_INPUT_ERROR;
    const int64_t band = std::min<int64_t>((int64_t)all_logits->items() / vocab, n);
    if (band < 1) return OP_ATTR_ERROR;
    constexpr int dt = brk_dtype<DT>();
    const size_t es = DataType_size(DT);

    Scratch sc;
    int32_t* d_ids = (int32_t*)sc.take(n * 4);
    int32_t* d_mask = (int32_t*)sc.take(n * 4);
    int32_t* d_target = (int32_t*)sc.take(n * 4);
    int32_t* d_count = (int32_t*)sc.take(4);
    float* d_rowloss = (float*)sc.take(n * 4);
    float* d_total = (float*)sc.take(4);
    auto kind = [](tensor_t& t) { return t->is_cpu() ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice; };
    BR_CUDA_CHECK(cudaMemcpyAsync(d_ids, ids_->data(), n * 4, kind(ids_), stream()));
    BR_CUDA_CHECK(cudaMemcpyAsync(d_mask, mask_->data(), n * 4, kind(mask_), stream()));
    int st = brk_loss_targets(d_ids, d_mask, d_target, d_count, batch, tokens, sptr());
    if (st != BRK_OK) return ret(st);
    int items = 0;
    BR_CUDA_CHECK(cudaMemcpyAsync(&items, d_count, 4, cudaMemcpyDeviceToHost, stream()));
    BR_CUDA_CHECK(cudaStreamSynchronize(stream()));
    BR_CUDA_CHECK(cudaMemsetAsync(x_g->data(), 0, x_g->bytes(), stream()));
    if (items == 0) return 0.0f;
    const float scale = ComputingContext::loss_scale / (float)items;

    // the weight gradient accumulates on the device; a host-resident gradient gets a device twin
    void* d_wg = lm_head_g->data();
    void* twin = nullptr;
    if (lm_head_g->is_cpu()) {
        if (lm_head_g->dtype() != DT) return OP_OUTPUT_ERROR;
        BR_CUDA_CHECK(cudaMalloc(&twin, lm_head_g->bytes()));
        BR_CUDA_CHECK(cudaMemcpyAsync(twin, lm_head_g->data(), lm_head_g->bytes(), cudaMemcpyHostToDevice, stream()));
        d_wg = twin;
    } else if (lm_head_g->dtype() != DT) {
        return OP_OUTPUT_ERROR;
    }

    void* logits = all_logits->data();
    for (int64_t r0 = 0; r0 < n && st == BRK_OK; r0 += band) {
        const int64_t rows = std::min(band, n - r0);
        const unsigned char* x = (const unsigned char*)mem_ + r0 * hidden * es;
        unsigned char* dx = (unsigned char*)x_g->data() + r0 * hidden * es;
        // logits = x W^T
        st = gemm_any<DT>(x, lm_head->data(), logits, rows, vocab, hidden, 0, 1, hidden, hidden, vocab, 0.0f, nullptr);
        // row losses and dlogits (in place)
        if (st == BRK_OK) { ProfScope prof("nll_fwd_bwd"); st = brk_logsoftmax_nll_fwd_bwd(logits, d_target + r0, d_rowloss + r0, logits, rows, vocab, scale, dt, sptr()); }
        // x_g = dlogits W
        if (st == BRK_OK) st = gemm_any<DT>(logits, lm_head->data(), dx, rows, hidden, vocab, 0, 0, vocab, hidden, hidden, 0.0f, nullptr);
        // W_g += dlogits^T x
        if (st == BRK_OK) st = gemm_any<DT>(logits, x, d_wg, vocab, hidden, rows, 1, 0, vocab, hidden, hidden, 1.0f, nullptr);
    }
    if (st == BRK_OK) st = brk_sum_f32(d_rowloss, d_total, n, sptr());
    float total = 0.0f;
    if (st == BRK_OK) {
        BR_CUDA_CHECK(cudaMemcpyAsync(&total, d_total, 4, cudaMemcpyDeviceToHost, stream()));
        if (twin) BR_CUDA_CHECK(cudaMemcpyAsync(lm_head_g->data(), twin, lm_head_g->bytes(), cudaMemcpyDeviceToHost, stream()));
        BR_CUDA_CHECK(cudaStreamSynchronize(stream()));
    }
    if (twin) cudaFree(twin);
    if (st != BRK_OK) return ret(st);
    float loss = total / (float)items;
    if (ComputingContext::verbose) std::cout << "#################  " << items << " " << loss << std::endl;
    return loss;
}

// op_loss_backward queued without a host round trip (the reference synchronises twice per group of rows,
// blackriver/cuda_tensor.cpp:569-577 and 686-691): the number of counted positions stays on the device, the gradient
// factor loss_scale / items is formed inside the log-softmax kernel and the mean loss is left in loss_out[0].
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_loss_backward_async(tensor_t self, tensor_t ids_, tensor_t mask_, tensor_t lm_head, tensor_t all_logits,
                                                       tensor_t x_g, tensor_t lm_head_g, tensor_t loss_out, int defer_weight) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->shape().dim() != 3 || !dev_ok<DT>({lm_head, all_logits})) return OP_INPUT_ERROR;
    if (!ids_ || !mask_ || ids_->dtype() != DataType::Int || mask_->dtype() != DataType::Int) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({x_g, lm_head_g}) || x_g->items() != self->items() || lm_head_g->items() != lm_head->items()) return OP_OUTPUT_ERROR;
    if (!dev_ok<DataType::Float>({loss_out}) || loss_out->items() < 1) return OP_OUTPUT_ERROR;
    const int batch = (int)self->shape()[0], tokens = (int)self->shape()[1];
    const int64_t hidden = self->shape()[2], vocab = lm_head->shape()[0];
    const int64_t n = (int64_t)batch * tokens;
    if ((int64_t)ids_->items() < n || (int64_t)mask_->items() < n) return OP_INPUT_ERROR;
    const int64_t band = std::min<int64_t>((int64_t)all_logits->items() / vocab, n);
    if (band < 1 || (defer_weight && band < n)) return OP_ATTR_ERROR;
    constexpr int dt = brk_dtype<DT>();
    const size_t es = DataType_size(DT);

    Scratch sc;
    const int32_t* d_ids = int_on_device(ids_, sc);
    const int32_t* d_mask = int_on_device(mask_, sc);
    int32_t* d_target = (int32_t*)sc.take(n * 4);
    int32_t* d_count = (int32_t*)sc.take(4);
    float* d_rowloss = (float*)sc.take(n * 4);
    int st = brk_loss_targets(d_ids, d_mask, d_target, d_count, batch, tokens, sptr());
    void* logits = all_logits->data();
    for (int64_t r0 = 0; r0 < n && st == BRK_OK; r0 += band) {
        const int64_t rows = std::min(band, n - r0);
        const unsigned char* x = (const unsigned char*)mem_ + r0 * hidden * es;
        unsigned char* dx = (unsigned char*)x_g->data() + r0 * hidden * es;
        st = gemm_any<DT>(x, lm_head->data(), logits, rows, vocab, hidden, 0, 1, hidden, hidden, vocab, 0.0f, nullptr);
        if (st == BRK_OK) {
            ProfScope prof("nll_fwd_bwd");
            st = brk_logsoftmax_nll_fwd_bwd_counted(logits, d_target + r0, d_rowloss + r0, logits, rows, vocab, ComputingContext::loss_scale,
                                                    d_count, dt, sptr());
        }
        if (st == BRK_OK) st = gemm_any<DT>(logits, lm_head->data(), dx, rows, hidden, vocab, 0, 0, vocab, hidden, hidden, 0.0f, nullptr);
        if (st == BRK_OK && !defer_weight)
            st = gemm_any<DT>(logits, x, lm_head_g->data(), vocab, hidden, rows, 1, 0, vocab, hidden, hidden, 1.0f, nullptr);
    }
    if (st == BRK_OK) st = brk_sum_div_f32(d_rowloss, d_count, (float*)loss_out->data(), n, sptr());
    return ret(st);
}

// lm_head_g += dlogits^T x, the weight-gradient GEMM that op_loss_backward_async left out
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_loss_backward_w(tensor_t self, tensor_t x, tensor_t lm_head_g) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({x}) || x->shape().dim() != 3) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({lm_head_g}) || lm_head_g->shape().dim() != 2) return OP_OUTPUT_ERROR;
    const int64_t n = (int64_t)(x->shape()[0] * x->shape()[1]), hidden = x->shape()[2];
    const int64_t vocab = lm_head_g->shape()[0];
    if ((int64_t)lm_head_g->shape()[1] != hidden || (int64_t)self->items() < n * vocab) return OP_INPUT_ERROR;
    return ret(gemm_any<DT>(mem_, x->data(), lm_head_g->data(), vocab, hidden, n, 1, 0, vocab, hidden, hidden, 1.0f, nullptr));
}

// Forward-only scoring over the LM head (no counterpart in the reference, whose only inference hook is op_last_logits):
// the same banded logits GEMM and target rule as op_loss_backward, row losses only.
template <DataType DT>
LossReturn CUDATensor<DT>::op_token_nll(tensor_t self, tensor_t ids_, tensor_t mask_, tensor_t lm_head, tensor_t all_logits, tensor_t out) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->shape().dim() != 3 || !dev_ok<DT>({lm_head, all_logits})) return OP_INPUT_ERROR;
    if (!ids_ || !mask_ || ids_->dtype() != DataType::Int || mask_->dtype() != DataType::Int) return OP_INPUT_ERROR;
    const int batch = (int)self->shape()[0], tokens = (int)self->shape()[1];
    const int64_t hidden = self->shape()[2], vocab = lm_head->shape()[0];
    const int64_t n = (int64_t)batch * tokens;
    if (!dev_ok<DataType::Float>({out}) || (int64_t)out->items() != n) return OP_OUTPUT_ERROR;
    if ((int64_t)ids_->items() < n || (int64_t)mask_->items() < n) return OP_INPUT_ERROR;
    const int64_t band = std::min<int64_t>((int64_t)all_logits->items() / vocab, n);
    if (band < 1) return OP_ATTR_ERROR;
    constexpr int dt = brk_dtype<DT>();
    const size_t es = DataType_size(DT);

    Scratch sc;
    int32_t* d_ids = (int32_t*)sc.take(n * 4);
    int32_t* d_mask = (int32_t*)sc.take(n * 4);
    int32_t* d_target = (int32_t*)sc.take(n * 4);
    int32_t* d_count = (int32_t*)sc.take(4);
    float* d_total = (float*)sc.take(4);
    auto kind = [](tensor_t& t) { return t->is_cpu() ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice; };
    BR_CUDA_CHECK(cudaMemcpyAsync(d_ids, ids_->data(), n * 4, kind(ids_), stream()));
    BR_CUDA_CHECK(cudaMemcpyAsync(d_mask, mask_->data(), n * 4, kind(mask_), stream()));
    int st = brk_loss_targets(d_ids, d_mask, d_target, d_count, batch, tokens, sptr());
    float* row_loss = (float*)out->data();
    for (int64_t r0 = 0; r0 < n && st == BRK_OK; r0 += band) {
        const int64_t rows = std::min(band, n - r0);
        const unsigned char* x = (const unsigned char*)mem_ + r0 * hidden * es;
        st = gemm_any<DT>(x, lm_head->data(), all_logits->data(), rows, vocab, hidden, 0, 1, hidden, hidden, vocab, 0.0f, nullptr);
        if (st == BRK_OK) st = brk_logsoftmax_nll_fwd(all_logits->data(), d_target + r0, row_loss + r0, nullptr, rows, vocab, dt, sptr());
    }
    if (st == BRK_OK) st = brk_sum_f32(row_loss, d_total, n, sptr());
    if (st != BRK_OK) return ret(st);
    int items = 0;
    float total = 0.0f;
    BR_CUDA_CHECK(cudaMemcpyAsync(&items, d_count, 4, cudaMemcpyDeviceToHost, stream()));
    BR_CUDA_CHECK(cudaMemcpyAsync(&total, d_total, 4, cudaMemcpyDeviceToHost, stream()));
    BR_CUDA_CHECK(cudaStreamSynchronize(stream()));
    return items > 0 ? total / (float)items : 0.0f;
}

// ---- backward math -----------------------------------------------------------------------------------
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_layernorm_backward(tensor_t self, tensor_t scale, tensor_t bias, tensor_t var, tensor_t y,
                                                      tensor_t dscale, tensor_t dbias, tensor_t din, float eps) {
    ProfScope prof("layernorm_bwd");
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({scale, bias, y}) || !dev_ok<DataType::Float>({var})) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({dscale, dbias, din}) || din->items() != self->items()) return OP_OUTPUT_ERROR;
    int64_t hidden = (int64_t)self->shape().vec().back();
    int64_t rows = (int64_t)self->items() / hidden;
    if ((int64_t)var->items() < rows || y->items() != self->items()) return OP_INPUT_ERROR;
    size_t need = brk_layernorm_bwd_workspace_bytes(rows, hidden);
    if (need > ComputingContext::workspace_size) return OP_ATTR_ERROR;
    return ret(brk_layernorm_bwd(mem_, scale->data(), bias->data(), (const float*)var->data(), y->data(), dscale->data(),
                                 dbias->data(), din->data(), rows, hidden, eps, ComputingContext::cuda_workspace,
                                 ComputingContext::workspace_size, ComputingContext::grad_accumulate, brk_dtype<DT>(), sptr()));
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_layernorm_backward_residual(tensor_t self, tensor_t scale, tensor_t bias, tensor_t var, tensor_t y,
                                                               tensor_t dscale, tensor_t dbias, tensor_t din, tensor_t residual,
                                                               float eps) {
    ProfScope prof("layernorm_bwd");
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({scale, bias, y, residual}) || !dev_ok<DataType::Float>({var})) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({dscale, dbias, din}) || din->items() != self->items()) return OP_OUTPUT_ERROR;
    int64_t hidden = (int64_t)self->shape().vec().back();
    int64_t rows = (int64_t)self->items() / hidden;
    if ((int64_t)var->items() < rows || y->items() != self->items() || residual->items() != self->items()) return OP_INPUT_ERROR;
    size_t need = brk_layernorm_bwd_workspace_bytes(rows, hidden);
    if (need > ComputingContext::workspace_size) return OP_ATTR_ERROR;
    return ret(brk_layernorm_bwd_residual(mem_, scale->data(), bias->data(), (const float*)var->data(), y->data(), residual->data(),
                                          dscale->data(), dbias->data(), din->data(), rows, hidden, eps,
                                          ComputingContext::cuda_workspace, ComputingContext::workspace_size,
                                          ComputingContext::grad_accumulate, brk_dtype<DT>(), sptr()));
}

// b_g = sum_n dy ; W_g = dy^T x ; x_g = dy W, all overwritten, W_g before x_g because x_g may be x
// (blackriver/cuda_tensor.cpp:731-812; bloomz-7b/train.words:198)
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_linear_backward(tensor_t self, tensor_t x, tensor_t weight, tensor_t bias, tensor_t x_g,
                                                   tensor_t weight_g, tensor_t bias_g) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({x, weight}) || weight->shape().dim() != 2) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({x_g, weight_g, bias_g})) return OP_OUTPUT_ERROR;
    int64_t out = (int64_t)weight->shape()[0], in = (int64_t)weight->shape()[1];
    int64_t n = (int64_t)self->items() / out;
    if ((int64_t)x->items() != n * in) return OP_INPUT_ERROR;
    if (x_g->items() != x->items() || weight_g->items() != weight->items() || (int64_t)bias_g->items() != out) return OP_OUTPUT_ERROR;
    constexpr int dt = brk_dtype<DT>();
    const int acc = ComputingContext::grad_accumulate;
    int st;
    { ProfScope prof("colsum"); st = brk_colsum_ws(mem_, bias_g->data(), n, out, acc, dt, ComputingContext::cuda_workspace, ComputingContext::workspace_size, sptr()); }
    if (st == BRK_OK) st = gemm_any<DT>(mem_, x->data(), weight_g->data(), out, in, n, 1, 0, out, in, in, acc ? 1.0f : 0.0f, nullptr);
    if (st == BRK_OK) st = gemm_any<DT>(mem_, weight->data(), x_g->data(), n, in, out, 0, 0, out, in, in, 0.0f, nullptr);
    return ret(st);
}

// x_g = dy W alone: the part of op_linear_backward that the previous pipeline stage waits for
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_linear_backward_x(tensor_t self, tensor_t weight, tensor_t x_g) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({weight}) || weight->shape().dim() != 2) return OP_INPUT_ERROR;
    int64_t out = (int64_t)weight->shape()[0], in = (int64_t)weight->shape()[1];
    if (self->items() % out != 0) return OP_INPUT_ERROR;
    int64_t n = (int64_t)self->items() / out;
    if (!dev_ok<DT>({x_g}) || (int64_t)x_g->items() != n * in) return OP_OUTPUT_ERROR;
    return ret(gemm_any<DT>(mem_, weight->data(), x_g->data(), n, in, out, 0, 0, out, in, in, 0.0f, nullptr));
}

// b_g = sum_n dy ; W_g = dy^T x: the part nothing downstream waits for (it can run any time before the optimizer)
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_linear_backward_w(tensor_t self, tensor_t x, tensor_t weight_g, tensor_t bias_g) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({x})) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({weight_g, bias_g}) || weight_g->shape().dim() != 2) return OP_OUTPUT_ERROR;
    int64_t out = (int64_t)weight_g->shape()[0], in = (int64_t)weight_g->shape()[1];
    if (self->items() % out != 0 || (int64_t)bias_g->items() != out) return OP_INPUT_ERROR;
    int64_t n = (int64_t)self->items() / out;
    if ((int64_t)x->items() != n * in) return OP_INPUT_ERROR;
    constexpr int dt = brk_dtype<DT>();
    const int acc = ComputingContext::grad_accumulate;
    int st;
    { ProfScope prof("colsum"); st = brk_colsum_ws(mem_, bias_g->data(), n, out, acc, dt, ComputingContext::cuda_workspace, ComputingContext::workspace_size, sptr()); }
    if (st == BRK_OK) st = gemm_any<DT>(mem_, x->data(), weight_g->data(), out, in, n, 1, 0, out, in, in, acc ? 1.0f : 0.0f, nullptr);
    return ret(st);
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_gelu_backward(tensor_t self, tensor_t x, tensor_t x_g) {
    ProfScope prof("gelu_bwd");
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({x}) || x->items() != self->items()) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({x_g}) || x_g->items() != self->items()) return OP_OUTPUT_ERROR;
    return ret(brk_gelu_bwd(mem_, x->data(), x_g->data(), (int64_t)self->items(), brk_dtype<DT>(), sptr()));
}

// dV = P^T dO ; dP = dO V^T   (blackriver/cuda_tensor.cpp:831-888)
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_attn_backward(tensor_t self, tensor_t attn, tensor_t v, tensor_t attn_g, tensor_t v_g) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->shape().dim() != 4 || !dev_ok<DT>({attn, v}) || !self->same_shape(v)) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({attn_g, v_g}) || attn_g->items() != attn->items() || v_g->items() != v->items()) return OP_OUTPUT_ERROR;
    auto& s = self->shape();
    int64_t bh = s[0] * s[1], t = s[2], d = s[3];
    constexpr int dt = brk_dtype<DT>();
    int st = brk_gemm(attn->data(), mem_, v_g->data(), t, d, t, 1, 0, t, d, d, bh, t * t, t * d, t * d, 1.0f, 0.0f, nullptr, dt, sptr());
    if (st == BRK_OK) st = brk_gemm(mem_, v->data(), attn_g->data(), t, t, d, 0, 1, d, d, t, bh, t * d, t * d, t * t, 1.0f, 0.0f, nullptr, dt, sptr());
    return ret(st);
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_softmax_backward(tensor_t self, tensor_t out, tensor_t x_g) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({out}) || out->items() != self->items()) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({x_g}) || x_g->items() != self->items()) return OP_OUTPUT_ERROR;
    int64_t cols = (int64_t)self->shape().vec().back();
    return ret(brk_softmax_bwd(mem_, out->data(), x_g->data(), (int64_t)self->items() / cols, cols, brk_dtype<DT>(), sptr()));
}

// dV = P^T dO ; dS = P o (dP - sum P o dP) with dP = dO V^T ; attn_g may be attn itself
// (blackriver/cuda_tensor.cpp:921-1002; bloomz-7b/train.words:217).  dP is produced in bands of
// (batch, head) groups inside the device scratch, so dS can overwrite P band by band.
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_softmax_attn_backward(tensor_t self, tensor_t attn, tensor_t v, tensor_t attn_g, tensor_t v_g) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->shape().dim() != 4 || !dev_ok<DT>({attn, v}) || !self->same_shape(v)) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({attn_g, v_g}) || attn_g->items() != attn->items() || v_g->items() != v->items()) return OP_OUTPUT_ERROR;
    auto& s = self->shape();
    int64_t bh = s[0] * s[1], t = s[2], d = s[3];
    constexpr int dt = brk_dtype<DT>();
    const size_t es = DataType_size(DT);
    int st = brk_gemm(attn->data(), mem_, v_g->data(), t, d, t, 1, 0, t, d, d, bh, t * t, t * d, t * d, 1.0f, 0.0f, nullptr, dt, sptr());
    int64_t group = (int64_t)(ComputingContext::workspace_size / ((size_t)t * t * es));
    if (group < 1) return OP_ATTR_ERROR;
    group = std::min(group, bh);
    void* dp = ComputingContext::cuda_workspace;
    for (int64_t g0 = 0; g0 < bh && st == BRK_OK; g0 += group) {
        int64_t g = std::min(group, bh - g0);
        const unsigned char* dout = (const unsigned char*)mem_ + g0 * t * d * es;
        const unsigned char* vv = (const unsigned char*)v->data() + g0 * t * d * es;
        const unsigned char* p = (const unsigned char*)attn->data() + g0 * t * t * es;
        unsigned char* ds = (unsigned char*)attn_g->data() + g0 * t * t * es;
        st = brk_gemm(dout, vv, dp, t, t, d, 0, 1, d, d, t, g, t * d, t * d, t * t, 1.0f, 0.0f, nullptr, dt, sptr());
        if (st == BRK_OK) st = brk_softmax_bwd(dp, p, ds, g * t, t, dt, sptr());
    }
    return ret(st);
}

// dQ = dS K / sqrt(d) ; dK = dS^T Q / sqrt(d)   (blackriver/cuda_tensor.cpp:1005-1063)
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_qk_backward(tensor_t self, tensor_t q, tensor_t k, tensor_t q_g, tensor_t k_g) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->shape().dim() != 4 || !dev_ok<DT>({q, k}) || q->shape().dim() != 4 || !q->same_shape(k)) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({q_g, k_g}) || q_g->items() != q->items() || k_g->items() != k->items()) return OP_OUTPUT_ERROR;
    auto& s = q->shape();
    int64_t bh = s[0] * s[1], t = s[2], d = s[3];
    if ((int64_t)self->items() != bh * t * t) return OP_INPUT_ERROR;
    float alpha = (float)(1.0 / std::sqrt((double)d));
    constexpr int dt = brk_dtype<DT>();
    int st = brk_gemm(mem_, k->data(), q_g->data(), t, d, t, 0, 0, t, d, d, bh, t * t, t * d, t * d, alpha, 0.0f, nullptr, dt, sptr());
    if (st == BRK_OK) st = brk_gemm(mem_, q->data(), k_g->data(), t, d, t, 1, 0, t, d, d, bh, t * t, t * d, t * d, alpha, 0.0f, nullptr, dt, sptr());
    return ret(st);
}

// ---- extensions ------------------------------------------------------------------------------------------
namespace {

// ALiBi slopes of the reference formula (blackriver/train_bloom.cpp:61-66) as fp32 on the device, cached
// per head count for the life of the process.
const float* device_slopes(int heads) {
    static std::vector<std::pair<int, float*>> cache;
    for (auto& e : cache)
        if (e.first == heads) return e.second;
    std::vector<double> sd(heads);
    brk_alibi_slopes(heads, sd.data());
    std::vector<float> sf(sd.begin(), sd.end());
    float* d = nullptr;
    BR_CUDA_CHECK(cudaMalloc(&d, heads * sizeof(float)));
    BR_CUDA_CHECK(cudaMemcpyAsync(d, sf.data(), heads * sizeof(float), cudaMemcpyHostToDevice, stream()));
    BR_CUDA_CHECK(cudaStreamSynchronize(stream()));
    cache.emplace_back(heads, d);
    return d;
}

}  // namespace

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_flash_attn(tensor_t self, tensor_t lens, tensor_t out, tensor_t lse, int heads) {
    ProfScope prof("attention_fwd");
    if (DT != DataType::F16) return OP_TODO_ERROR;   // the fp32 parity path keeps the unfused operator chain
    if (self->shape().dim() != 3 || heads <= 0) return OP_INPUT_ERROR;
    const int batch = (int)self->shape()[0], tokens = (int)self->shape()[1];
    const int64_t h3 = (int64_t)self->shape()[2];
    if (h3 % 3 != 0 || (h3 / 3) % heads != 0) return OP_INPUT_ERROR;
    const int64_t hidden = h3 / 3;
    const int d = (int)(hidden / heads);
    if (!dev_ok<DT>({out}) || (int64_t)out->items() != (int64_t)batch * tokens * hidden) return OP_OUTPUT_ERROR;
    if (!dev_ok<DataType::Float>({lse}) || (int64_t)lse->items() < (int64_t)batch * heads * tokens) return OP_OUTPUT_ERROR;
    if (lens && (lens->dtype() != DataType::Int || (int)lens->items() < batch)) return OP_INPUT_ERROR;
    Scratch sc;
    const int32_t* dlens = lens ? int_on_device(lens, sc) : nullptr;
    const __half* q = (const __half*)mem_;
    return ret(brk_flash_attn_fwd(q, q + hidden, q + 2 * hidden, h3, out->data(), hidden, (float*)lse->data(), dlens,
                                  device_slopes(heads), batch, tokens, heads, d, sptr()));
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_flash_attn_backward(tensor_t self, tensor_t qkv, tensor_t out, tensor_t lse, tensor_t lens,
                                                       tensor_t dqkv, int heads) {
    ProfScope prof("attention_bwd");
    if (DT != DataType::F16) return OP_TODO_ERROR;
    if (!dev_ok<DT>({qkv, out}) || qkv->shape().dim() != 3 || heads <= 0 || !dev_ok<DataType::Float>({lse})) return OP_INPUT_ERROR;
    const int batch = (int)qkv->shape()[0], tokens = (int)qkv->shape()[1];
    const int64_t h3 = (int64_t)qkv->shape()[2], hidden = h3 / 3;
    if (h3 % 3 != 0 || hidden % heads != 0) return OP_INPUT_ERROR;
    const int d = (int)(hidden / heads);
    if (self->items() != out->items() || (int64_t)out->items() != (int64_t)batch * tokens * hidden) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({dqkv}) || dqkv->items() != qkv->items()) return OP_OUTPUT_ERROR;
    if (lens && (lens->dtype() != DataType::Int || (int)lens->items() < batch)) return OP_INPUT_ERROR;
    Scratch sc;
    const int32_t* dlens = lens ? int_on_device(lens, sc) : nullptr;
    size_t need = brk_flash_attn_bwd_workspace_bytes(batch, tokens, heads);
    void* ws = sc.take(need);
    const __half* q = (const __half*)qkv->data();
    __half* g = (__half*)dqkv->data();
    return ret(brk_flash_attn_bwd(q, q + hidden, q + 2 * hidden, h3, out->data(), mem_, hidden, (const float*)lse->data(), g,
                                  g + hidden, g + 2 * hidden, h3, dlens, device_slopes(heads), batch, tokens, heads, d, ws, need, sptr()));
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_linear_residual(tensor_t self, tensor_t w, tensor_t bias, tensor_t residual, tensor_t y) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({w, bias, residual}) || w->shape().dim() != 2) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({y})) return OP_OUTPUT_ERROR;
    int64_t in = (int64_t)self->shape().vec().back(), out = (int64_t)w->shape()[0];
    int64_t n = (int64_t)self->items() / in;
    if ((int64_t)w->shape()[1] != in || (int64_t)bias->items() != out || (int64_t)residual->items() != n * out) return OP_INPUT_ERROR;
    if ((int64_t)y->items() != n * out) return OP_OUTPUT_ERROR;
    ProfScope prof(DT == DataType::F16 ? "gemm_f16" : "gemm_f32");
    if (DT == DataType::F16 && brk_gemm_f16_supported(n, out, in, 0, 1, in, in, mem_, w->data()))
        return ret(brk_gemm_f16(mem_, w->data(), y->data(), n, out, in, 0, 1, in, in, out, bias->data(), residual->data(), out,
                                nullptr, 0, 0, sptr()));
    int st = brk_gemm(mem_, w->data(), y->data(), n, out, in, 0, 1, in, in, out, 1, 0, 0, 0, 1.0f, 0.0f, bias->data(), brk_dtype<DT>(), sptr());
    int64_t dims[4] = {1, 1, n, out};
    if (st == BRK_OK) st = brk_add_bcast(y->data(), residual->data(), y->data(), dims, dims, brk_dtype<DT>(), sptr());
    return ret(st);
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_linear_gelu(tensor_t self, tensor_t w, tensor_t bias, tensor_t y, tensor_t y_gelu) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({w, bias}) || w->shape().dim() != 2) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({y, y_gelu})) return OP_OUTPUT_ERROR;
    int64_t in = (int64_t)self->shape().vec().back(), out = (int64_t)w->shape()[0];
    int64_t n = (int64_t)self->items() / in;
    if ((int64_t)w->shape()[1] != in || (int64_t)bias->items() != out) return OP_INPUT_ERROR;
    if ((int64_t)y->items() != n * out || y_gelu->items() != y->items()) return OP_OUTPUT_ERROR;
    ProfScope prof(DT == DataType::F16 ? "gemm_f16" : "gemm_f32");
    if (DT == DataType::F16 && brk_gemm_f16_supported(n, out, in, 0, 1, in, in, mem_, w->data()))
        return ret(brk_gemm_f16(mem_, w->data(), y->data(), n, out, in, 0, 1, in, in, out, bias->data(), nullptr, 0, y_gelu->data(), out,
                                0, sptr()));
    int st = brk_gemm(mem_, w->data(), y->data(), n, out, in, 0, 1, in, in, out, 1, 0, 0, 0, 1.0f, 0.0f, bias->data(), brk_dtype<DT>(), sptr());
    if (st == BRK_OK) st = brk_gelu_fwd(y->data(), y_gelu->data(), n * out, brk_dtype<DT>(), sptr());
    return ret(st);
}

// self = ids; the call is routed here through the TABLE's backend, so DT is the table's type
template <DataType DT>
ComputingReturn CUDATensor<DT>::op_embed(tensor_t self, tensor_t table, tensor_t out) {
    ProfScope prof("embedding");
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (self->dtype() != DataType::Int || table->shape().dim() != 2) return OP_INPUT_ERROR;
    const int64_t n = (int64_t)self->items(), vocab = (int64_t)table->shape()[0], hidden = (int64_t)table->shape()[1];
    if (!dev_ok<DT>({out}) || (int64_t)out->items() != n * hidden) return OP_OUTPUT_ERROR;
    Scratch sc;
    const int32_t* ids = int_on_device(self, sc);
    return ret(brk_embedding_gather(table->data(), ids, out->data(), n, hidden, vocab, brk_dtype<DT>(), sptr()));
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_embed_backward(tensor_t self, tensor_t ids_, tensor_t table_g) {
    ProfScope prof("embedding");
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!ids_ || ids_->dtype() != DataType::Int) return OP_INPUT_ERROR;
    if (!dev_ok<DT>({table_g}) || table_g->shape().dim() != 2) return OP_OUTPUT_ERROR;
    const int64_t n = (int64_t)ids_->items(), vocab = (int64_t)table_g->shape()[0], hidden = (int64_t)table_g->shape()[1];
    if ((int64_t)self->items() != n * hidden) return OP_INPUT_ERROR;
    Scratch sc;
    const int32_t* ids = int_on_device(ids_, sc);
    return ret(brk_embedding_scatter_add(mem_, ids, table_g->data(), n, hidden, vocab, brk_dtype<DT>(), sptr()));
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_adam(tensor_t self, tensor_t grad, tensor_t master, tensor_t m, tensor_t v, float lr, float beta1,
                                        float beta2, float eps, int step, float grad_scale) {
    ProfScope prof("adam");
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (!dev_ok<DT>({grad}) || !dev_ok<DataType::Float>({master, m, v})) return OP_INPUT_ERROR;
    const int64_t n = (int64_t)self->items();
    if ((int64_t)grad->items() != n || (int64_t)master->items() != n || (int64_t)m->items() != n || (int64_t)v->items() != n) return OP_INPUT_ERROR;
    // fp16 working weights are refreshed by the kernel; fp32 working weights are a copy of the master
    void* w16 = DT == DataType::F16 ? mem_ : nullptr;
    int st = brk_adam_step(master->data(), m->data(), v->data(), grad->data(), brk_dtype<DT>(), w16, n, lr, beta1, beta2, eps, step,
                           grad_scale, sptr());
    if (st == BRK_OK && DT == DataType::Float && master->data() != mem_)
        BR_CUDA_CHECK(cudaMemcpyAsync(mem_, master->data(), self->bytes(), cudaMemcpyDeviceToDevice, stream()));
    return ret(st);
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::io_nccl_sendrecv(tensor_t self, tensor_t recv, int peer) {
    if (!CollectiveContext::has_comm) return OP_ATTR_ERROR;
    if (!recv || !recv->is_cuda()) return OP_OUTPUT_ERROR;
    BR_NCCL_CHECK(ncclGroupStart());
    BR_NCCL_CHECK(ncclSend(mem_, self->bytes(), ncclChar, peer, CollectiveContext::nccl_comm, nccl_stream()));
    BR_NCCL_CHECK(ncclRecv(recv->data(), recv->bytes(), ncclChar, peer, CollectiveContext::nccl_comm, nccl_stream()));
    BR_NCCL_CHECK(ncclGroupEnd());
    return OP_OK;
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::io_nccl_allreduce(tensor_t self) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    if (CollectiveContext::dp_world <= 1) return OP_OK;
    if (!CollectiveContext::dp_comm) return OP_ATTR_ERROR;
    BR_NCCL_CHECK(ncclAllReduce(mem_, mem_, self->items(), DT == DataType::F16 ? ncclHalf : ncclFloat, ncclSum,
                                CollectiveContext::dp_comm, nccl_stream()));
    return OP_OK;
}

template <DataType DT>
ComputingReturn CUDATensor<DT>::op_randn(tensor_t self, float mean, float std, uint64_t seed) {
    if (DT == DataType::Int) return OP_TODO_ERROR;
    return ret(brk_init_normal(mem_, (int64_t)self->items(), mean, std, seed, brk_dtype<DT>(), sptr()));
}

template struct CUDATensor<DataType::Float>;
template struct CUDATensor<DataType::F16>;
template struct CUDATensor<DataType::Int>;

tensor_t create_cuda_float(std::vector<size_t>& shape) {
    ShapeType s(shape);
    return std::make_shared<TensorType>(new CUDATensor<DataType::Float>(s), s);
}
tensor_t create_cuda_half(std::vector<size_t>& shape) {
    ShapeType s(shape);
    return std::make_shared<TensorType>(new CUDATensor<DataType::F16>(s), s);
}
tensor_t create_cuda_int(std::vector<size_t>& shape) {
    ShapeType s(shape);
    return std::make_shared<TensorType>(new CUDATensor<DataType::Int>(s), s);
}

}  // namespace br
