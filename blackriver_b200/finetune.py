"""Fine-tune driver over the C++ host side: builds a BLOOM-shaped model (or one pipeline stage of
it) with the generated words scripts and runs training steps made of micro-batches.

It plays the role of the reference's driver (blackriver/train_bloom.cpp: BloomInput feeding ids
and masks, BloomAttentions running the words) with one rank per GPU: rank r owns a contiguous
block of layers, the first rank also the embedding, the last rank the final LayerNorm, the tied
LM head and the loss.  Each step runs every micro-batch forward through the pipeline, then every
micro-batch backward (activations of all micro-batches in flight are kept in per-micro-batch
slots), sums the two copies of the tied-table gradient, and applies Adam.
Everything that computes is a word executed by the words machine on device tensors.
"""
import numpy as np

from . import host, words

LM_HEAD_COST_IN_LAYERS = 5.9      # measured step time of final LayerNorm + 250880-way head + loss, in 7b1 decoder layers (5.1 by FLOPs)


def partition_layers(n_layers, world, head_cost=LM_HEAD_COST_IN_LAYERS):
    """Contiguous layer counts per stage.  The last stage also carries the final LayerNorm, the LM
    head and the loss, worth `head_cost` layers, so it gets correspondingly fewer layers -- none at
    all when the head alone already fills a stage's share (7b1 on 8 GPUs).  Picks the split whose
    most loaded stage is lightest; every stage but the last keeps at least one layer."""
    if world == 1:
        return [n_layers]
    best = None
    for last in range(0, n_layers - (world - 1) + 1):
        rest = n_layers - last
        heaviest = max(-(-rest // (world - 1)), last + head_cost)
        if best is None or heaviest <= best[0] + 1e-9:      # ties: more layers next to the head, fewer elsewhere
            best = (heaviest, last)
    last = best[1]
    rest = n_layers - last
    counts = [rest // (world - 1) + (1 if i < rest % (world - 1) else 0) for i in range(world - 1)]
    return counts + [last]


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


class Trainer:
    def __init__(self, hidden, heads, vocab, n_layers, batch, tokens, n_micro, rank=0, world=1, dtype="half", seed=0,
                 loss_scale=1024.0, lr=1e-4, logits_rows=None, init_std=0.02, verbose=False, head_cost=LM_HEAD_COST_IN_LAYERS):
        self.rank, self.world, self.n_micro = rank, world, n_micro
        self.batch, self.tokens = batch, tokens
        self.loss_scale, self.lr = float(loss_scale), float(lr)
        self.counts = partition_layers(n_layers, world, head_cost)
        self.first, self.last = rank == 0, rank == world - 1
        my_layers = self.counts[rank]
        self.n_slots = n_micro if world > 1 else 1
        self.env = host.Env(my_layers + 1)
        text = words.fused_words(
            hidden=hidden, heads=heads, vocab=vocab, n_layers=my_layers, batch=batch, tokens=tokens, dtype=dtype,
            first_stage=self.first, last_stage=self.last, logits_rows=logits_rows, init_std=init_std, seed=seed,
            layer_offset=sum(self.counts[:rank]), n_slots=self.n_slots,
            prev_rank=None if self.first else rank - 1, next_rank=None if self.last else rank + 1)
        self.env.execute(text)
        self.env.execute("build_model init_model zero_grads")
        self.env.execute(f"{self.loss_scale} op.loss_scale {1 if verbose else 0} op.verbose")
        e = self.env
        # compiled once, run many times
        self.p_fwd = [e.build(f"slot_{k if self.n_slots > 1 else 0} stage_forward") for k in range(self.n_slots)]
        self.p_bwd = [e.build(f"slot_{k if self.n_slots > 1 else 0} stage_backward") for k in range(self.n_slots)]
        self.p_begin = e.build("zero_grads 1 op.accumulate")
        self.p_sync = e.build("op.sync")
        self.p_score = None          # built on first use
        self.step_no = 0
        self.losses = []

    def _feed(self, mb):
        ids, mask, lens = mb
        e = self.env
        e.change(0)
        e.write("ids_", ids)
        e.write("mask_", mask)
        e.write("lens_", lens)

    def step(self, microbatches):
        """One optimizer step over the micro-batches; returns the mean loss (last stage) or None."""
        e = self.env
        assert len(microbatches) == self.n_micro
        e.run(self.p_begin)
        self.losses = []
        if self.world == 1:
            for mb in microbatches:
                self._feed(mb)
                e.run(self.p_fwd[0])
                e.run(self.p_bwd[0])
                self.losses.append(host.last_loss())
        else:
            for k, mb in enumerate(microbatches):
                self._feed(mb)
                e.run(self.p_fwd[k])
            for k, mb in enumerate(microbatches):
                self._feed(mb)
                e.run(self.p_bwd[k])
                if self.last:
                    self.losses.append(host.last_loss())
            if self.first or self.last:
                peer = self.world - 1 if self.first else 0
                e.execute(f"{peer} sync_tied_grads")
        self.step_no += 1
        # gradients were summed over micro-batches and carry the loss scale: Adam divides both out
        gs = 1.0 / (self.loss_scale * self.n_micro)
        e.execute(f"0 op.accumulate {self.lr} {self.step_no} {gs} optimizer_step")
        return float(np.mean(self.losses)) if self.losses else None

    def score(self, microbatches):
        """Forward only (prefill scoring): runs every micro-batch through the stages and, on the rank that holds the
        head, returns a list of (token_nll [batch, tokens] float32, mean NLL) per micro-batch -- token_nll[b, t] is the
        NLL of ids[b, t+1] at position t, 0 where that pair is not counted.  Other ranks return an empty list."""
        e = self.env
        if self.p_score is None:
            self.p_score = [e.build(f"slot_{k} stage_score") for k in range(self.n_slots)]
        out = []
        for k, mb in enumerate(microbatches):
            self._feed(mb)
            e.run(self.p_score[k % self.n_slots])
            if self.last:
                e.change(0)
                nll = e.read("token_nll").copy()        # synchronises the compute stream
                out.append((nll, host.last_loss()))
        return out

    def sync(self):
        self.env.run(self.p_sync)

    def close(self):
        # the training switches live in the process-wide computing context: hand them back at their defaults
        self.env.execute("0 op.accumulate 1 op.loss_scale 1 op.verbose")
        for p in self.p_fwd + self.p_bwd + [self.p_begin, self.p_sync] + (self.p_score or []):
            self.env.free_program(p)
        self.env.close()


def gemm_flops_per_microbatch(hidden, vocab, n_layers, tokens_total, with_head=True):
    """FLOPs of every GEMM launch of one micro-batch's forward + backward (2 m n k each; the
    backward has two GEMMs per forward GEMM)."""
    per_layer_fwd = 2 * tokens_total * 12 * hidden * hidden
    head_fwd = 2 * tokens_total * hidden * vocab
    return 3 * n_layers * per_layer_fwd + (3 * head_fwd if with_head else 0)
