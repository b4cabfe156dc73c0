#include "nn.hpp"

#include <array>

#include "brk.h"
#include "context.hpp"
#include "cuda_tensor.hpp"
#include "tensortype.hpp"

namespace br {
namespace {

// Pops N tensors; the result is in PUSH order (index 0 = pushed first = deepest).
template <size_t N>
std::array<tensor_t, N> pop_tensors(Stack& stack) {
    std::array<tensor_t, N> t;
    for (size_t i = N; i-- > 0;) t[i] = stack.pop_tensor();
    return t;
}

std::vector<size_t> pop_shape(Stack& stack) {
    std::vector<size_t> shape;
    for (double v : stack.pop_number_list()) shape.push_back((size_t)v);
    return shape;
}

#define BR_WORD(NAME, BODY)                        \
    struct NAME : public NativeWord {              \
        void run(Stack& stack) override { BODY }   \
        NWORD_CREATOR_DEFINE_LR(NAME)              \
    };

// ( -- )  wait for the compute stream
BR_WORD(Sync, {
    (void)stack;
    if (ComputingContext::booted) {
        BR_CUDA_CHECK(cudaStreamSynchronize(ComputingContext::cuda_stream));
        BR_CUDA_CHECK(cudaStreamSynchronize(ComputingContext::comm_stream));
        for (int d = 0; d < 2; d++) BR_CUDA_CHECK(cudaStreamSynchronize(ComputingContext::link_stream[d]));
    }
})

// ( d1 .. dn n device dtype -- t )   device: "cuda" | "cpu"; dtype: "float" | "half" | "int"
BR_WORD(Create, {
    std::string dtype = stack.pop_string();
    std::string device = stack.pop_string();
    auto shape = pop_shape(stack);
    tensor_t t;
    if (device == "cuda" && dtype == "float") t = create_cuda_float(shape);
    else if (device == "cuda" && dtype == "half") t = create_cuda_half(shape);
    else if (device == "cuda" && dtype == "int") t = create_cuda_int(shape);
    else if (device == "cpu" && dtype == "float") t = create_cpu_float(shape);
    else if (device == "cpu" && dtype == "half") t = create_cpu_half(shape);
    else if (device == "cpu" && dtype == "int") t = create_cpu_int(shape);
    else br_panic("op.create: unsupported device/dtype " + device + "/" + dtype);
    stack.push_tensor(t);
})

BR_WORD(Zero, {
    tensor_t t = stack.pop_tensor();
    t->op_zero(t);
})

// ( t value -- )
BR_WORD(Fill, {
    double value = stack.pop_number();
    tensor_t t = stack.pop_tensor();
    t->op_fill(t, (float)value);
})

// ( t offset d1 .. dn n -- view )
BR_WORD(View, {
    auto shape = pop_shape(stack);
    size_t offset = (size_t)stack.pop_number();
    tensor_t t = stack.pop_tensor();
    auto r = t->op_view(t, offset, shape);
    stack.push_tensor(std::get<1>(r));
})

// ( dst src -- )
BR_WORD(Copy, {
    auto t = pop_tensors<2>(stack);
    t[0]->op_copy(t[0], t[1]);
})

// ( x w b y -- )
BR_WORD(Linear, {
    auto t = pop_tensors<4>(stack);
    t[0]->op_linear(t[0], t[1], t[2], t[3]);
})

// ( x mean var scale bias y eps -- )
BR_WORD(Layernorm, {
    float eps = (float)stack.pop_number();
    auto t = pop_tensors<6>(stack);
    t[0]->op_layernorm(t[0], t[1], t[2], t[3], t[4], t[5], eps);
})

// ( x y -- )
BR_WORD(Transpos0213, {
    auto t = pop_tensors<2>(stack);
    t[0]->op_transpos_0213(t[0], t[1]);
})

// ( q k qk -- )
BR_WORD(QueryKey, {
    auto t = pop_tensors<3>(stack);
    t[0]->op_qk(t[0], t[1], t[2]);
})

// ( a b c -- )  c = a + b
BR_WORD(Add, {
    auto t = pop_tensors<3>(stack);
    t[0]->op_add(t[0], t[1], t[2]);
})

// ( x out -- )
BR_WORD(Softmax, {
    auto t = pop_tensors<2>(stack);
    t[0]->op_softmax(t[0], t[1]);
})

// ( probs v out -- )
BR_WORD(Attn, {
    auto t = pop_tensors<3>(stack);
    t[0]->op_attn(t[0], t[1], t[2]);
})

// ( x out -- )
BR_WORD(Gelu, {
    auto t = pop_tensors<2>(stack);
    t[0]->op_gelu(t[0], t[1]);
})

// ( x mask lm_head out -- )
BR_WORD(LastLogits, {
    auto t = pop_tensors<4>(stack);
    t[0]->op_last_logits(t[0], t[1], t[2], t[3]);
})

// ( x ids mask lm_head workspace x_g lm_head_g -- )   the reference word drops the loss value
// (blackriver/nn.cpp:178-190); it is kept here for last_loss()
float g_last_loss = 0.0f;
BR_WORD(LossBackward, {
    auto t = pop_tensors<7>(stack);
    auto r = t[0]->op_loss_backward(t[0], t[1], t[2], t[3], t[4], t[5], t[6]);
    if (r.index() == 1) g_last_loss = std::get<1>(r);
})

// ( x ids mask lm_head workspace out -- )   forward-only scoring; the mean is kept for last_loss()
BR_WORD(TokenNll, {
    auto t = pop_tensors<6>(stack);
    auto r = t[0]->op_token_nll(t[0], t[1], t[2], t[3], t[4], t[5]);
    if (r.index() == 1) g_last_loss = std::get<1>(r);
})

// ( dy scale bias var y dscale dbias din eps -- )
BR_WORD(LayernormBackward, {
    float eps = (float)stack.pop_number();
    auto t = pop_tensors<8>(stack);
    t[0]->op_layernorm_backward(t[0], t[1], t[2], t[3], t[4], t[5], t[6], t[7], eps);
})

// ( dy scale bias var y dscale dbias din residual eps -- )  din = residual + the LayerNorm's input gradient
BR_WORD(LayernormBackwardResidual, {
    float eps = (float)stack.pop_number();
    auto t = pop_tensors<9>(stack);
    t[0]->op_layernorm_backward_residual(t[0], t[1], t[2], t[3], t[4], t[5], t[6], t[7], t[8], eps);
})

// ( dy x w b x_g w_g b_g -- )
BR_WORD(LinearBackward, {
    auto t = pop_tensors<7>(stack);
    t[0]->op_linear_backward(t[0], t[1], t[2], t[3], t[4], t[5], t[6]);
})

// ( dy x x_g -- )
BR_WORD(GeluBackward, {
    auto t = pop_tensors<3>(stack);
    t[0]->op_gelu_backward(t[0], t[1], t[2]);
})

// ( dy attn v attn_g v_g -- )
BR_WORD(AttnBackward, {
    auto t = pop_tensors<5>(stack);
    t[0]->op_attn_backward(t[0], t[1], t[2], t[3], t[4]);
})

// ( dy out x_g -- )
BR_WORD(SoftmaxBackward, {
    auto t = pop_tensors<3>(stack);
    t[0]->op_softmax_backward(t[0], t[1], t[2]);
})

// ( dy attn v attn_g v_g -- )
BR_WORD(SoftmaxAttnBackward, {
    auto t = pop_tensors<5>(stack);
    t[0]->op_softmax_attn_backward(t[0], t[1], t[2], t[3], t[4]);
})

// ( dS q k q_g k_g -- )
BR_WORD(QueryKeyBackward, {
    auto t = pop_tensors<5>(stack);
    t[0]->op_qk_backward(t[0], t[1], t[2], t[3], t[4]);
})

// ---- extension words ----
// ( qkv lens out lse heads -- )
BR_WORD(FlashAttn, {
    int heads = (int)stack.pop_number();
    auto t = pop_tensors<4>(stack);
    t[0]->op_flash_attn(t[0], t[1], t[2], t[3], heads);
})
// ( dout qkv out lse lens dqkv heads -- )
BR_WORD(FlashAttnBackward, {
    int heads = (int)stack.pop_number();
    auto t = pop_tensors<6>(stack);
    t[0]->op_flash_attn_backward(t[0], t[1], t[2], t[3], t[4], t[5], heads);
})
// ( x w b residual y -- )
BR_WORD(LinearResidual, {
    auto t = pop_tensors<5>(stack);
    t[0]->op_linear_residual(t[0], t[1], t[2], t[3], t[4]);
})
// ( x w b y y_gelu -- )
BR_WORD(LinearGelu, {
    auto t = pop_tensors<5>(stack);
    t[0]->op_linear_gelu(t[0], t[1], t[2], t[3], t[4]);
})
// ( ids table out -- )
BR_WORD(Embed, {
    auto t = pop_tensors<3>(stack);
    t[0]->op_embed(t[0], t[1], t[2]);
})
// ( dx ids table_g -- )
BR_WORD(EmbedBackward, {
    auto t = pop_tensors<3>(stack);
    t[0]->op_embed_backward(t[0], t[1], t[2]);
})
// ( w grad master m v lr beta1 beta2 eps step grad_scale -- )
BR_WORD(Adam, {
    float gscale = (float)stack.pop_number();
    int step = (int)stack.pop_number();
    float eps = (float)stack.pop_number();
    float b2 = (float)stack.pop_number();
    float b1 = (float)stack.pop_number();
    float lr = (float)stack.pop_number();
    auto t = pop_tensors<5>(stack);
    t[0]->op_adam(t[0], t[1], t[2], t[3], t[4], lr, b1, b2, eps, step, gscale);
})
// ( t mean std seed -- )
BR_WORD(Randn, {
    uint64_t seed = (uint64_t)stack.pop_number();
    float std = (float)stack.pop_number();
    float mean = (float)stack.pop_number();
    tensor_t t = stack.pop_tensor();
    t->op_randn(t, mean, std, seed);
})
// ( send_t recv_t peer -- )  grouped send + receive with one peer
BR_WORD(IoNcclSendRecv, {
    int peer = (int)stack.pop_number();
    auto t = pop_tensors<2>(stack);
    t[0]->io_nccl_sendrecv(t[0], t[1], peer);
})
// ( tensor -- )  the tensor becomes its sum over the data-parallel replicas
BR_WORD(IoNcclAllReduce, {
    tensor_t t = stack.pop_tensor();
    t->io_nccl_allreduce(t);
})
// ( -- replica replicas )  this rank's place among the data-parallel replicas
BR_WORD(IoReplica, {
    stack.push_number(CollectiveContext::dp_rank);
    stack.push_number(CollectiveContext::dp_world);
})
// ( flag -- )  1: weight / bias gradients are added to, 0: overwritten (the reference behaviour)
BR_WORD(Accumulate, { ComputingContext::grad_accumulate = stack.pop_number() != 0.0 ? 1 : 0; })
// ( value -- )  factor applied to the loss gradient
BR_WORD(LossScale, { ComputingContext::loss_scale = (float)stack.pop_number(); })
// ( flag -- )  0 silences the per-call loss line of op.loss_backward
BR_WORD(Verbose, { ComputingContext::verbose = stack.pop_number() != 0.0 ? 1 : 0; })
// ( -- loss )  value of the most recent op.loss_backward
BR_WORD(LastLoss, { stack.push_number((double)g_last_loss); })

// ( dy w x_g -- )  first half of op.linear_backward
BR_WORD(LinearBackwardX, {
    auto t = pop_tensors<3>(stack);
    t[0]->op_linear_backward_x(t[0], t[1], t[2]);
})
// ( dy x w_g b_g -- )  second half of op.linear_backward
BR_WORD(LinearBackwardW, {
    auto t = pop_tensors<4>(stack);
    t[0]->op_linear_backward_w(t[0], t[1], t[2], t[3]);
})
// ( x ids mask lm_head workspace x_g lm_head_g loss_out defer -- )  op.loss_backward without a host round trip
BR_WORD(LossBackwardAsync, {
    int defer = (int)stack.pop_number();
    auto t = pop_tensors<8>(stack);
    t[0]->op_loss_backward_async(t[0], t[1], t[2], t[3], t[4], t[5], t[6], t[7], defer);
})
// ( workspace x lm_head_g -- )  the LM-head weight gradient a deferring op.loss_backward_async left out
BR_WORD(LossBackwardW, {
    auto t = pop_tensors<3>(stack);
    t[0]->op_loss_backward_w(t[0], t[1], t[2]);
})
// ( -- code )  waits for the device; 0 when no tensor-core kernel gave up a bounded wait and no optimizer launch met a
// non-finite gradient since the last query, else 256 * (Adam status) + 16 * (GEMM status) + (attention status)
BR_WORD(KernelStatus, {
    int code = 0;
    if (ComputingContext::booted) {
        BR_CUDA_CHECK(cudaStreamSynchronize(ComputingContext::cuda_stream));
        code = 256 * brk_adam_status() + 16 * brk_gemm_f16_status() + brk_flash_attn_status();
    }
    stack.push_number((double)code);
})

// ( -- )  the transfer stream continues from the compute stream's present position, and the io.nccl.* words that follow
// queue on it: the transfer then runs beside whatever the compute stream is given next
BR_WORD(StreamFork, {
    (void)stack;
    BR_CUDA_CHECK(cudaEventRecord(ComputingContext::compute_done, ComputingContext::cuda_stream));
    BR_CUDA_CHECK(cudaStreamWaitEvent(ComputingContext::comm_stream, ComputingContext::compute_done, 0));
    ComputingContext::nccl_on_comm_stream = 1;
})
// ( -- )  the compute stream waits for what was queued on the transfer stream since the fork
BR_WORD(StreamJoin, {
    (void)stack;
    BR_CUDA_CHECK(cudaEventRecord(ComputingContext::comm_done, ComputingContext::comm_stream));
    BR_CUDA_CHECK(cudaStreamWaitEvent(ComputingContext::cuda_stream, ComputingContext::comm_done, 0));
    ComputingContext::nccl_on_comm_stream = 0;
})

// ( flag -- )  1: from here on every operator (and io.nccl.* word) queues on the transfer stream, which first waits for
// what the compute stream has been given so far; 0: back to the compute stream, which does NOT wait for the side work --
// whoever needs a result of it waits for an event recorded there (op.event.record / op.event.wait) or joins
// (op.stream.join).  Used to run the optimizer beside the next step's first forward.
BR_WORD(StreamSide, {
    const bool on = stack.pop_number() != 0.0;
    if (!ComputingContext::booted) return;
    if (on) {
        br_assert(ComputingContext::main_stream == nullptr, "op.stream.side: already on the side stream");
        BR_CUDA_CHECK(cudaEventRecord(ComputingContext::compute_done, ComputingContext::cuda_stream));
        BR_CUDA_CHECK(cudaStreamWaitEvent(ComputingContext::comm_stream, ComputingContext::compute_done, 0));
        ComputingContext::main_stream = ComputingContext::cuda_stream;
        ComputingContext::cuda_stream = ComputingContext::comm_stream;
    } else {
        br_assert(ComputingContext::main_stream != nullptr, "op.stream.side: not on the side stream");
        ComputingContext::cuda_stream = ComputingContext::main_stream;
        ComputingContext::main_stream = nullptr;
    }
})
// ( id -- )  marks the present position of the stream operators are queued on
BR_WORD(EventRecord, {
    const int id = (int)stack.pop_number();
    br_assert(id >= 0 && id < 4096, "op.event.record: id out of range");
    if (!ComputingContext::booted) return;
    auto& marks = ComputingContext::marks;
    while ((int)marks.size() <= id) {
        cudaEvent_t e;
        BR_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        marks.push_back(e);
        ComputingContext::mark_set.push_back(0);
    }
    BR_CUDA_CHECK(cudaEventRecord(marks[id], ComputingContext::cuda_stream));
    ComputingContext::mark_set[id] = 1;
})
// ( id -- )  the compute stream waits for mark id (nothing to wait for if it was never recorded)
BR_WORD(EventWait, {
    const int id = (int)stack.pop_number();
    if (id >= 0 && id < (int)ComputingContext::marks.size() && ComputingContext::mark_set[id]) {
        cudaStream_t compute = ComputingContext::main_stream ? ComputingContext::main_stream : ComputingContext::cuda_stream;
        BR_CUDA_CHECK(cudaStreamWaitEvent(compute, ComputingContext::marks[id], 0));
    }
})

// ---- one-sided stage hand-offs (PipeLinks) ----
// ( bytes_per_slot slots -- )  collective over all ranks
BR_WORD(LinkOpen, {
    int slots = (int)stack.pop_number();
    size_t bytes = (size_t)stack.pop_number();
    PipeLinks::open(bytes, slots);
})
BR_WORD(LinkClose, { (void)stack; PipeLinks::close(); })
// ( ranks -- )  before io.link.open, single-rank process only: play that many pipeline ranks in this process
BR_WORD(LinkEmulate, { PipeLinks::emulate((int)stack.pop_number()); })
// ( rank -- )  the played rank the following io.link words act for
BR_WORD(LinkRank, { PipeLinks::select((int)stack.pop_number()); })
// ( side slot d1 .. dn n dtype -- t )  this rank's window as a tensor; side 0 = from the previous rank, 1 = from the next
BR_WORD(LinkWindow, {
    std::string dtype = stack.pop_string();
    auto shape = pop_shape(stack);
    int slot = (int)stack.pop_number();
    int side = (int)stack.pop_number();
    ShapeType s(shape);
    void* mem = PipeLinks::window(side, slot);
    tensor_t t;
    if (dtype == "half") t = std::make_shared<TensorType>(new CUDATensor<DataType::F16>(mem), s);
    else if (dtype == "float") t = std::make_shared<TensorType>(new CUDATensor<DataType::Float>(mem), s);
    else br_panic("io.link.window: dtype must be half or float");
    br_assert(t->bytes() <= PipeLinks::slot_bytes, "io.link.window: the shape does not fit a window");
    stack.push_tensor(t);
})
// ( t dir slot -- )  dir 1 = to the next rank, 0 = to the previous rank
BR_WORD(LinkSend, {
    int slot = (int)stack.pop_number();
    int dir = (int)stack.pop_number();
    tensor_t t = stack.pop_tensor();
    br_assert(t->is_cuda(), "io.link.send moves device tensors");
    PipeLinks::send(dir, slot, t->data(), t->bytes());
})
// ( dir -- )  the compute stream waits until the last tensor sent in that direction has left its buffer
BR_WORD(LinkFence, { PipeLinks::fence((int)stack.pop_number()); })
// ( side slot -- )
BR_WORD(LinkWait, {
    int slot = (int)stack.pop_number();
    int side = (int)stack.pop_number();
    PipeLinks::wait(side, slot);
})
BR_WORD(LinkRelease, {
    int slot = (int)stack.pop_number();
    int side = (int)stack.pop_number();
    PipeLinks::release(side, slot);
})

BR_WORD(IoDump, {
    tensor_t t = stack.pop_tensor();
    t->io_dump(t);
})

// ( t file -- )
BR_WORD(IoLoad, {
    std::string file = stack.pop_string();
    tensor_t t = stack.pop_tensor();
    t->io_load(t, file.c_str());
})

BR_WORD(IoSave, {
    std::string file = stack.pop_string();
    tensor_t t = stack.pop_tensor();
    t->io_save(t, file.c_str());
})

// ( t peer -- )
BR_WORD(IoMpiRecv, {
    int peer = (int)stack.pop_number();
    tensor_t t = stack.pop_tensor();
    t->io_mpi_recv(t, peer);
})
BR_WORD(IoMpiSend, {
    int peer = (int)stack.pop_number();
    tensor_t t = stack.pop_tensor();
    t->io_mpi_send(t, peer);
})
BR_WORD(IoMpiBcast, {
    int root = (int)stack.pop_number();
    tensor_t t = stack.pop_tensor();
    t->io_mpi_bcast(t, root);
})
BR_WORD(IoNcclRecv, {
    int peer = (int)stack.pop_number();
    tensor_t t = stack.pop_tensor();
    t->io_nccl_recv(t, peer);
})
BR_WORD(IoNcclSend, {
    int peer = (int)stack.pop_number();
    tensor_t t = stack.pop_tensor();
    t->io_nccl_send(t, peer);
})

}  // namespace

float last_loss() { return g_last_loss; }

void load_nn_words(Enviroment& env) {
    env.insert_native_word("io.dump", IoDump::creator);
    env.insert_native_word("io.load", IoLoad::creator);
    env.insert_native_word("io.save", IoSave::creator);
    env.insert_native_word("io.mpi.bcast", IoMpiBcast::creator);
    env.insert_native_word("io.mpi.recv", IoMpiRecv::creator);
    env.insert_native_word("io.mpi.send", IoMpiSend::creator);
    env.insert_native_word("io.nccl.send", IoNcclSend::creator);
    env.insert_native_word("io.nccl.recv", IoNcclRecv::creator);

    env.insert_native_word("io.nccl.sendrecv", IoNcclSendRecv::creator);
    env.insert_native_word("io.nccl.allreduce", IoNcclAllReduce::creator);
    env.insert_native_word("io.replica", IoReplica::creator);
    env.insert_native_word("op.flash_attn", FlashAttn::creator);
    env.insert_native_word("op.flash_attn_backward", FlashAttnBackward::creator);
    env.insert_native_word("op.linear_residual", LinearResidual::creator);
    env.insert_native_word("op.linear_gelu", LinearGelu::creator);
    env.insert_native_word("op.embed", Embed::creator);
    env.insert_native_word("op.embed_backward", EmbedBackward::creator);
    env.insert_native_word("op.adam", Adam::creator);
    env.insert_native_word("op.token_nll", TokenNll::creator);
    env.insert_native_word("op.randn", Randn::creator);
    env.insert_native_word("op.accumulate", Accumulate::creator);
    env.insert_native_word("op.loss_scale", LossScale::creator);
    env.insert_native_word("op.last_loss", LastLoss::creator);
    env.insert_native_word("op.verbose", Verbose::creator);

    env.insert_native_word("op.linear_backward_x", LinearBackwardX::creator);
    env.insert_native_word("op.linear_backward_w", LinearBackwardW::creator);
    env.insert_native_word("op.loss_backward_async", LossBackwardAsync::creator);
    env.insert_native_word("op.loss_backward_w", LossBackwardW::creator);
    env.insert_native_word("op.kernel_status", KernelStatus::creator);
    env.insert_native_word("op.stream.fork", StreamFork::creator);
    env.insert_native_word("op.stream.join", StreamJoin::creator);
    env.insert_native_word("op.stream.side", StreamSide::creator);
    env.insert_native_word("op.event.record", EventRecord::creator);
    env.insert_native_word("op.event.wait", EventWait::creator);
    env.insert_native_word("io.link.open", LinkOpen::creator);
    env.insert_native_word("io.link.close", LinkClose::creator);
    env.insert_native_word("io.link.emulate", LinkEmulate::creator);
    env.insert_native_word("io.link.rank", LinkRank::creator);
    env.insert_native_word("io.link.window", LinkWindow::creator);
    env.insert_native_word("io.link.send", LinkSend::creator);
    env.insert_native_word("io.link.fence", LinkFence::creator);
    env.insert_native_word("io.link.wait", LinkWait::creator);
    env.insert_native_word("io.link.release", LinkRelease::creator);

    env.insert_native_word("op.sync", Sync::creator);
    env.insert_native_word("op.create", Create::creator);
    env.insert_native_word("op.zero", Zero::creator);
    env.insert_native_word("op.fill", Fill::creator);
    env.insert_native_word("op.view", View::creator);
    env.insert_native_word("op.copy", Copy::creator);
    env.insert_native_word("op.linear", Linear::creator);
    env.insert_native_word("op.layernorm", Layernorm::creator);
    env.insert_native_word("op.transpos_0213", Transpos0213::creator);
    env.insert_native_word("op.add", Add::creator);
    env.insert_native_word("op.querykey", QueryKey::creator);
    env.insert_native_word("op.softmax", Softmax::creator);
    env.insert_native_word("op.attn", Attn::creator);
    env.insert_native_word("op.gelu", Gelu::creator);
    env.insert_native_word("op.last_logits", LastLogits::creator);
    env.insert_native_word("op.loss_backward", LossBackward::creator);
    env.insert_native_word("op.layernorm_backward", LayernormBackward::creator);
    env.insert_native_word("op.layernorm_backward_residual", LayernormBackwardResidual::creator);
    env.insert_native_word("op.linear_backward", LinearBackward::creator);
    env.insert_native_word("op.gelu_backward", GeluBackward::creator);
    env.insert_native_word("op.attn_backward", AttnBackward::creator);
    env.insert_native_word("op.softmax_backward", SoftmaxBackward::creator);
    env.insert_native_word("op.softmax_attn_backward", SoftmaxAttnBackward::creator);
    env.insert_native_word("op.qk_backward", QueryKeyBackward::creator);
}

}  // namespace br
