"""Fine-tune driver over the C++ host side: builds a BLOOM-shaped model (or one pipeline stage of
it) with the generated words scripts and runs training steps made of micro-batches.

It plays the role of the reference's driver (blackriver/train_bloom.cpp: BloomInput feeding ids
and masks, BloomAttentions running the words) with one rank per GPU: rank r owns a contiguous
block of layers, the first rank also the embedding, the last rank the final LayerNorm, the tied
LM head and the loss.  Each step runs every micro-batch forward and backward through the pipeline
(activations of the micro-batches in flight are kept in slots; schedule.py fixes the order of the
tasks on every rank), sums the two copies of the tied-table gradient, and applies Adam.
Everything that computes is a word executed by the words machine on device tensors.
"""
import numpy as np

from . import host, schedule, words

LM_HEAD_COST_IN_LAYERS = 4.3      # measured step time of final LayerNorm + 250880-way head + loss, in 7b1 decoder layers


def partition_layers(n_layers, world, head_cost=LM_HEAD_COST_IN_LAYERS, n_micro=16):
    """Contiguous layer counts per stage.  The last stage also carries the final LayerNorm, the LM head and the loss,
    worth `head_cost` layers, so it gets correspondingly fewer layers -- none at all when the head alone already fills
    a stage's share (7b1 on 8 GPUs).  Among the near-even splits the one with the shortest simulated step of the
    overlapped schedule is taken (schedule.choose_partition); every stage but the last keeps at least one layer."""
    if world == 1:
        return [n_layers]
    unit = sum(schedule.LAYER_COST) * head_cost / sum(schedule.HEAD_COST)
    head = tuple(c * unit for c in schedule.HEAD_COST)
    return schedule.choose_partition(n_layers, world, n_micro, head_cost=head)


def make_microbatches(n_micro, batch, tokens, vocab, min_len, seed, pad_id=3):
    """Seeded synthetic token ids with right padding: (ids, mask, lens) per micro-batch."""
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n_micro):
        ids = rng.integers(0, vocab, (batch, tokens)).astype(np.int32)
        lens = rng.integers(min_len, tokens + 1, batch).astype(np.int32)
        mask = (np.arange(tokens)[None, :] < lens[:, None]).astype(np.int32)
        ids[mask == 0] = pad_id
        out.append((ids, mask, lens))
    return out


def replica_layout(rank, world, replicas, n_micro):
    """(replica, stage, stages, micro-batches per replica) of job rank `rank`: stage-major inside a replica, so the
    stages of one pipeline are neighbouring ranks (and neighbouring GPUs)."""
    if replicas < 1 or world % replicas or n_micro % replicas:
        raise ValueError(f"{world} ranks / {n_micro} micro-batches do not divide into {replicas} replicas")
    stages = world // replicas
    return rank // stages, rank % stages, stages, n_micro // replicas


def replica_share(microbatches, replica, replicas):
    """The micro-batches of a step that replica `replica` works on: every replicas-th, starting at its own number."""
    return list(microbatches[replica::replicas])


def pack_inputs(mb):
    """ids [B,T], mask [B,T], lens [B] of one micro-batch as the int32 buffer the stage scripts call "inp"."""
    ids, mask, lens = mb
    return np.concatenate([np.asarray(ids, np.int32).ravel(), np.asarray(mask, np.int32).ravel(), np.asarray(lens, np.int32).ravel()])


class Trainer:
    """One pipeline stage (or the whole model) driven through the words machine.

    world == 1: every micro-batch forward then backward.  world > 1 with overlap (the default): the stage's work is cut
    into forward / input-gradient / weight-gradient tasks per micro-batch, executed in the static order that
    schedule.build lays out for this rank, with one-sided hand-offs between neighbours (io.link.*), and stages may end
    between the attention half and the MLP half of a layer (split_layers) so that the ranks carry equal shares; with
    overlap=False the plain order (all forwards, then all backwards) over NCCL send / receive on the compute stream
    and whole layers per stage.
    Nothing in a step waits for the device except one check before the optimizer: the status words of the tensor-core
    kernels are read (an update computed from a kernel that gave up a wait is refused) together with the losses."""

    def __init__(self, hidden, heads, vocab, n_layers, batch, tokens, n_micro, rank=0, world=1, dtype="half", seed=0,
                 loss_scale=1024.0, lr=1e-4, logits_rows=None, init_std=0.02, verbose=False, head_cost=LM_HEAD_COST_IN_LAYERS,
                 overlap=None, n_slots=None, activation_budget=56 << 30, play_all_ranks=False, split_layers=True, replicas=1,
                 async_optimizer=False, early_exchange=False):
        # data-parallel replicas: the job's ranks form `replicas` pipelines of world / replicas stages; each replica
        # takes every replicas-th micro-batch of a step and the gradients are summed over the replicas before Adam.
        # From here on rank / world / n_micro describe this rank's pipeline and its share of the micro-batches.
        self.job_rank, self.job_world, self.replicas = rank, world, int(replicas)
        self.total_micro = n_micro
        if self.replicas > 1:
            self.replica, rank, world, n_micro = replica_layout(rank, world, self.replicas, n_micro)
        else:
            self.replica = 0
        self.rank, self.world, self.n_micro = rank, world, n_micro
        self.batch, self.tokens = batch, tokens
        self.loss_scale, self.lr = float(loss_scale), float(lr)
        self.first, self.last = rank == 0, rank == world - 1
        self.overlap = ((world > 1) if overlap is None else (bool(overlap) and world > 1)) and n_micro > 1
        if self.overlap and not play_all_ranks and not self._links_available():
            import sys
            print(f"rank {rank}: one-sided links unavailable (CUDA IPC / peer access); using NCCL hand-offs and the plain schedule",
                  file=sys.stderr)
            self.overlap = False
        # stage boundaries in half-layer units (2 per layer); the plain schedule keeps whole layers
        unit = sum(schedule.LAYER_COST) * head_cost / sum(schedule.HEAD_COST)
        head = tuple(c * unit for c in schedule.HEAD_COST)
        # the early exchange of the tied table's gradient (see below) lets a rank's deferred weight-gradient tasks run in
        # the time it would otherwise wait for the next step's first micro-batch, so the partition is then chosen for
        # the steady-state step time of consecutive steps; every rank derives the same answer from the same arguments
        self.early_exchange = False
        steady = self.overlap and bool(early_exchange) and self.replicas == 1 and not async_optimizer and not play_all_ranks
        self.bounds = schedule.choose_partition_units(n_layers, world, n_micro, head_cost=head,
                                                      whole_layers=not (self.overlap and split_layers), steady=steady)
        self.counts = [(self.bounds[r + 1] - self.bounds[r]) / 2 for r in range(world)]      # layers per stage, halves count 0.5
        u0, u1 = self.bounds[rank], self.bounds[rank + 1]
        first_layer = u0 // 2
        kinds = []
        for layer in range(first_layer, (u1 + 1) // 2 if u1 > u0 else first_layer):
            kinds.append(("A" if u0 <= 2 * layer < u1 else "") + ("M" if u0 <= 2 * layer + 1 < u1 else ""))
        self.kinds = kinds
        # share of a whole layer's GEMM FLOPs in each half: QKV + dense are 4 of the 12 h x h blocks
        self.gemm_layers = sum((4 if "A" in k else 0) + (8 if "M" in k else 0) for k in kinds) / 12.0
        my_layers = len(kinds)
        if world == 1:
            self.n_slots = 1
        elif not self.overlap:
            self.n_slots = n_micro        # all forwards run before the first backward: every micro-batch stays alive
        elif n_slots is not None:
            self.n_slots = max(2, min(int(n_slots), n_micro))
        else:
            act = batch * tokens * hidden * (2 if dtype == "half" else 4)
            self.n_slots = schedule.n_slots_for(world, n_micro, [int(c + 0.5) for c in self.counts], 23 * act, activation_budget)
        self.env = host.Env(my_layers + 1)
        kw = dict(hidden=hidden, heads=heads, vocab=vocab, n_layers=my_layers, batch=batch, tokens=tokens, dtype=dtype,
                  first_stage=self.first, last_stage=self.last, logits_rows=logits_rows, init_std=init_std, seed=seed,
                  layer_offset=first_layer, n_slots=self.n_slots, n_micro=n_micro, kinds=kinds,
                  prev_rank=None if self.first else rank - 1, next_rank=None if self.last else rank + 1)
        # play_all_ranks: this single-rank process holds the Trainers of every rank of the pipeline (a test on one GPU
        # that interleaves their task lists itself); the links then keep one block per played rank
        self.played = bool(play_all_ranks) and self.overlap
        # async_optimizer: Adam (and the tied-table exchange) are queued on the transfer stream and the next step's first
        # forward waits, layer by layer, for the parameters it reads, so the update runs beside that forward
        self.async_optimizer = bool(async_optimizer)
        self._grads_clean = True          # zero_grads ran at initialisation; the asynchronous optimizer clears them itself
        self.env.execute(words.fused_words(overlap=self.overlap, async_optimizer=self.async_optimizer, **kw))
        if self.played:
            self.env.execute(f"{world} io.link.emulate {rank} io.link.rank")
        self.env.execute("build_model init_model zero_grads")
        self.env.execute(f"{self.loss_scale} op.loss_scale {1 if verbose else 0} op.verbose")
        e = self.env
        S = self.n_slots
        self.tasks = []          # (program, micro-batch to feed or None) in execution order
        self._programs = []

        def prog(text):
            h = e.build(text)
            self._programs.append(h)
            return h

        if world == 1:
            self.order = None
            for k in range(n_micro):
                self.tasks.append((prog("slot_0 stage_forward"), k))
                self.tasks.append((prog(f'slot_0 "loss@{k}" stage_backward_async'), k))
        elif not self.overlap:
            self.order = None
            for k in range(n_micro):
                self.tasks.append((prog(f"slot_{k % S} stage_forward"), k))
            for k in range(n_micro):
                self.tasks.append((prog(f'slot_{k % S} "loss@{k}" stage_backward_async'), k))
        else:
            costs = self.stage_costs = schedule.stage_costs_units(self.bounds, head_cost=head)
            orders, self.simulated_step = schedule.build(world, n_micro, costs, S)
            schedule.check(orders, n_micro, S)          # raises on a dependency or slot conflict before anything is queued
            self.order = orders[rank]
            self.simulated_efficiency = schedule.efficiency(self.simulated_step, costs, n_micro)
            # the last rank takes the LM-head part of its weight-gradient tasks first and starts the exchange of the tied
            # table's gradient before the layers' parts (schedule.expand_last_rank): the first rank, whose next step
            # needs the updated table, then does not wait for this rank's deferred work
            self.early_exchange = steady and self.last and not self.first
            if self.early_exchange:
                self.order = schedule.expand_last_rank(self.order)
            for t in self.order:
                slot = t.k % S
                if t.kind == "F":
                    self.tasks.append((prog(f"slot_{slot} stage_f"), t.k))
                elif t.kind == "B":
                    self.tasks.append((prog(f'slot_{slot} "loss@{t.k}" stage_b'), t.k))
                elif t.kind == "H":
                    self.tasks.append((prog(f"slot_{slot} stage_h"), None))
                elif t.kind == "X":
                    self.tasks.append((prog("0 sync_tied_start"), None))
                elif self.early_exchange:
                    self.tasks.append((prog(f"slot_{slot} stage_wl"), None))
                else:
                    self.tasks.append((prog(f"slot_{slot} stage_w"), None))
        self.p_begin = prog("zero_grads 1 op.accumulate")
        self.p_begin_clean = prog("1 op.accumulate")
        self.p_sync = prog("op.sync")
        self.p_status = prog("op.kernel_status")
        self.p_score = None          # built on first use
        self.step_no = 0
        self.losses = []

    @staticmethod
    def _links_available():
        """Opens and closes a minimal set of link windows.  io.link.open fails on every rank or on none (the ranks
        exchange their results), so all ranks reach the same answer."""
        probe = host.Env(1)
        try:
            probe.execute("256 2 io.link.open io.link.close")
            return True
        except host.HostError:
            return False
        finally:
            probe.close()

    def _feed(self, packed):
        e = self.env
        e.change(0)
        e.write_async("inp", packed)

    def begin_step(self, microbatches):
        if self.replicas > 1 and len(microbatches) == self.total_micro:
            microbatches = replica_share(microbatches, self.replica, self.replicas)
        assert len(microbatches) == self.n_micro
        self._packed = [pack_inputs(mb) for mb in microbatches]
        self.env.run(self.p_begin_clean if (self.async_optimizer and self._grads_clean) else self.p_begin)
        self._grads_clean = False

    def run_task(self, i):
        """Queues task i of this rank's list (step() runs them all in order; a test that emulates several ranks in one
        process interleaves the lists of its Trainers itself)."""
        program, k = self.tasks[i]
        if self.played:
            self.env.execute(f"{self.rank} io.link.rank")
        if k is not None:
            self._feed(self._packed[k])
        self.env.run(program)

    def check_and_read_losses(self):
        """The one wait of the step: kernel status and losses, before anything is applied to the weights."""
        e = self.env
        e.run(self.p_status)
        code = int(e.pop_number())
        if code >= 256:
            raise RuntimeError("the previous optimizer step met non-finite gradients (those elements were skipped): lower the loss scale")
        if code != 0:
            raise RuntimeError(f"a tensor-core kernel gave up a bounded wait (status {code}); the optimizer step was not applied")
        self.losses = []
        if self.last:
            e.change(0)
            # with replicas "loss_all" holds sums over the replicas by now (sync_replicas)
            self.losses = [float(v) / self.replicas for v in e.read("loss_all")]

    def apply_optimizer(self, tied_peer=None):
        """Adam on every parameter of the stage.  With tied_peer (a rank) the tied table's gradient is first exchanged
        with that rank, on the transfer stream, beside the Adam launches of the layers."""
        self.step_no += 1
        # gradients were summed over micro-batches and carry the loss scale: Adam divides both out
        gs = 1.0 / (self.loss_scale * self.total_micro)
        args = f"{self.lr} {self.step_no} {gs}"
        if self.async_optimizer:
            if tied_peer is None:
                self.env.execute(f"0 op.accumulate {args} optimizer_async")
            else:
                self.env.execute(f"0 op.accumulate {tied_peer} {args} optimizer_async_tied")
            self._grads_clean = True
        elif tied_peer is not None and self.early_exchange:
            # the exchange was started from the task list (X): wait for it, add, update
            self.env.execute(f"0 op.accumulate {args} optimizer_layers sync_tied_finish {args} optimizer_main")
        elif tied_peer is None:
            self.env.execute(f"0 op.accumulate {args} optimizer_step")
        else:
            self.env.execute(f"0 op.accumulate {tied_peer} sync_tied_start {args} optimizer_layers sync_tied_finish {args} optimizer_main")
        return float(np.mean(self.losses)) if self.losses else None

    def step(self, microbatches, after_task=None):
        """One optimizer step over the micro-batches; returns the mean loss (last stage) or None.  after_task(i), if
        given, is called when task i has been queued (a measurement hook: e.g. to record an event on the stream)."""
        self.begin_step(microbatches)
        for i in range(len(self.tasks)):
            self.run_task(i)
            if after_task is not None:
                after_task(i)
        if self.replicas > 1:
            self.env.execute("sync_replicas")
        self.check_and_read_losses()
        peer = None
        if self.world > 1 and (self.first or self.last):
            peer = self.world - 1 if self.first else 0
        return self.apply_optimizer(peer)

    def score(self, microbatches):
        """Forward only (prefill scoring): runs every micro-batch through the stages and, on the rank that holds the
        head, returns a list of (token_nll [batch, tokens] float32, mean NLL) per micro-batch -- token_nll[b, t] is the
        NLL of ids[b, t+1] at position t, 0 where that pair is not counted.  Other ranks return an empty list."""
        e = self.env
        if self.p_score is None:
            self.p_score = [e.build(f"slot_{k} stage_score") for k in range(self.n_slots)]
        out = []
        for k, mb in enumerate(microbatches):
            self._feed(pack_inputs(mb))
            e.run(self.p_score[k % self.n_slots])
            if self.last:
                e.change(0)
                nll = e.read("token_nll").copy()        # synchronises the compute stream
                out.append((nll, host.last_loss()))
        return out

    def save(self, prefix):
        """Checkpoint of this stage: fp32 master weights in the reference's per-tensor raw files plus the Adam moments
        (the words save_model writes them); the step count goes to <prefix>step.<rank>.txt."""
        if self.replica != 0:          # the replicas hold the same weights and moments: the first one writes them
            self.sync()
            return
        self.env.execute(f'op.sync "{prefix}" save_model op.sync')
        with open(f"{prefix}step.{self.rank}.txt", "w") as f:
            f.write(str(self.step_no))

    def load(self, prefix):
        self.env.execute(f'op.sync "{prefix}" load_model op.sync')
        with open(f"{prefix}step.{self.rank}.txt") as f:
            self.step_no = int(f.read().strip())

    def sync(self):
        self.env.run(self.p_sync)

    def drain(self):
        """Makes the compute stream wait for what is queued on the transfer stream (an asynchronous optimizer step), so
        that an event recorded on the compute stream afterwards covers it.  Does not block the host."""
        self.env.execute("op.stream.join")

    def close(self):
        # the training switches live in the process-wide computing context: hand them back at their defaults
        self.env.execute("op.sync 0 op.accumulate 1 op.loss_scale 1 op.verbose")
        if self.overlap:
            self.env.execute("io.link.close")
        for p in self._programs + (self.p_score or []):
            self.env.free_program(p)
        self.env.close()


def gemm_flops_per_microbatch(hidden, vocab, n_layers, tokens_total, with_head=True):
    """FLOPs of every GEMM launch of one micro-batch's forward + backward (2 m n k each; the
    backward has two GEMMs per forward GEMM)."""
    per_layer_fwd = 2 * tokens_total * 12 * hidden * hidden
    head_fwd = 2 * tokens_total * hidden * vocab
    return int(3 * n_layers * per_layer_fwd) + (3 * head_fwd if with_head else 0)
