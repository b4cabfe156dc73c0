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

LM_HEAD_COST_IN_LAYERS = 4.9      # forward FLOPs of the 250880-way head relative to one 7b1 decoder layer


def partition_layers(n_layers, world, head_cost=LM_HEAD_COST_IN_LAYERS):
    """Contiguous layer counts per stage.  The last stage also carries the LM head + loss, worth
    `head_cost` layers, so it gets correspondingly fewer layers -- none at all when the head alone
    already fills a stage's share (7b1 on 8 GPUs)."""
    if world == 1:
        return [n_layers]
    target = (n_layers + head_cost) / world
    last = max(0, min(n_layers - (world - 1), int(round(target - head_cost))))
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


def plan_stages(n_layers, world, interleave=1, head_cost=LM_HEAD_COST_IN_LAYERS):
    """Assignment of contiguous layer chunks ("virtual stages") to ranks.

    Returns (chunks_per_rank, wrap_partner): chunks_per_rank[r] is the ordered list of rank r's chunks,
    each a dict with n_layers, layer_offset (global index of its first layer), first / last (holds the
    embedding / the head), and how its input and output travel: "in" / "out" are None, ("rank", peer)
    for a neighbour hand-off on the compute stream, or ("wrap",) for the asynchronous wrap link.
    With interleave v > 1 the stages are visited in v rounds over a ring of ranks (breadth-first
    schedule); when the last rank cannot be given at least v layers next to the head it leaves the ring
    and keeps the head only.  wrap_partner is the rank that closes the ring (None without interleaving)."""
    v = max(1, int(interleave))
    if world == 1:
        return [[dict(n_layers=n_layers, layer_offset=0, first=True, last=True, **{"in": None, "out": None})]], None
    if v == 1:
        counts = partition_layers(n_layers, world, head_cost)
        out, off = [], 0
        for r, c in enumerate(counts):
            out.append([dict(n_layers=c, layer_offset=off, first=r == 0, last=r == world - 1,
                             **{"in": None if r == 0 else ("rank", r - 1), "out": None if r == world - 1 else ("rank", r + 1)})])
            off += c
        return out, None
    target = (n_layers + head_cost) / world
    r_last = max(0, int(round(target - head_cost)))
    head_only = r_last < v
    ring = world - 1 if head_only else world
    assert ring >= 2, "interleaving needs at least two ranks with layers"
    if head_only:
        r_last = 0
    rest = n_layers - r_last
    ring_ranks = ring if head_only else world - 1          # ranks that share `rest`
    totals = [rest // ring_ranks + (1 if i < rest % ring_ranks else 0) for i in range(ring_ranks)]
    if not head_only:
        totals.append(r_last)
    assert min(totals) >= v, "too few layers per rank for this interleave factor"
    per_chunk = [[t // v + (1 if c < t % v else 0) for c in range(v)] for t in totals]
    seq = [(c, r) for c in range(v) for r in range(ring)]       # visiting order of the virtual stages
    chunks = [[] for _ in range(world)]
    off = 0
    for i, (c, r) in enumerate(seq):
        n = per_chunk[r][c]
        is_last_vstage = (i == len(seq) - 1) and not head_only
        src = None if i == 0 else (("wrap",) if r == 0 else ("rank", r - 1))
        if i + 1 < len(seq):
            dst = ("wrap",) if seq[i + 1][1] == 0 else ("rank", seq[i + 1][1])
        else:
            dst = ("rank", world - 1) if head_only else None
        chunks[r].append(dict(n_layers=n, layer_offset=off, first=i == 0, last=is_last_vstage, **{"in": src, "out": dst}))
        off += n
    if head_only:
        chunks[world - 1].append(dict(n_layers=0, layer_offset=off, first=False, last=True, **{"in": ("rank", world - 2), "out": None}))
    return chunks, ring - 1


class Trainer:
    def __init__(self, hidden, heads, vocab, n_layers, batch, tokens, n_micro, rank=0, world=1, dtype="half", seed=0,
                 loss_scale=1024.0, lr=1e-4, logits_rows=None, init_std=0.02, verbose=False, interleave=1):
        self.rank, self.world, self.n_micro = rank, world, n_micro
        self.batch, self.tokens = batch, tokens
        self.loss_scale, self.lr = float(loss_scale), float(lr)
        plan, self.wrap_partner = plan_stages(n_layers, world, interleave)
        self.plan = plan
        self.counts = [sum(c["n_layers"] for c in chunks) for chunks in plan]
        self.chunks = plan[rank]
        self.n_slots = n_micro if world > 1 else 1
        if self.wrap_partner is not None:
            host.collective_boot_wrap(self.wrap_partner)          # collective: every rank calls it
        self.env = e = host.Env(sum(c["n_layers"] + 1 for c in self.chunks))
        base = 0
        for ci, c in enumerate(self.chunks):
            c["base"], c["sfx"] = base, (f"_c{ci}" if len(self.chunks) > 1 else "")
            kind_in, kind_out = c["in"], c["out"]
            e.execute(words.fused_words(
                hidden=hidden, heads=heads, vocab=vocab, n_layers=c["n_layers"], batch=batch, tokens=tokens, dtype=dtype,
                first_stage=c["first"], last_stage=c["last"], logits_rows=logits_rows, init_std=init_std, seed=seed,
                layer_offset=c["layer_offset"], n_slots=self.n_slots,
                prev_rank=kind_in[1] if kind_in and kind_in[0] == "rank" else None,
                next_rank=kind_out[1] if kind_out and kind_out[0] == "rank" else None,
                in_wrap=bool(kind_in and kind_in[0] == "wrap"), out_wrap=bool(kind_out and kind_out[0] == "wrap"),
                hash_base=base, word_suffix=c["sfx"]))
            e.execute(f"build_model{c['sfx']} init_model{c['sfx']} zero_grads{c['sfx']}")
            base += c["n_layers"] + 1
        e.execute(f"{self.loss_scale} op.loss_scale {1 if verbose else 0} op.verbose")
        # compiled once, run many times
        for c in self.chunks:
            sfx = c["sfx"]
            slots = range(self.n_slots)
            c["fwd"] = [e.build(f"slot_{k}{sfx} stage_forward{sfx}") for k in slots]
            c["bwd"] = [e.build(f"slot_{k}{sfx} stage_backward{sfx}") for k in slots]
        self.p_begin = e.build(" ".join(f"zero_grads{c['sfx']}" for c in self.chunks) + " 1 op.accumulate")
        self.p_sync = e.build("op.sync")
        self.first = any(c["first"] for c in self.chunks)
        self.last = any(c["last"] for c in self.chunks)
        self.step_no = 0
        self.losses = []

    def _feed(self, chunk, mb):
        ids, mask, lens = mb
        e = self.env
        e.change(chunk["base"])
        e.write("ids_", ids)
        e.write("mask_", mask)
        e.write("lens_", lens)

    def step(self, microbatches):
        """One optimizer step over the micro-batches; returns the mean loss (on the rank that holds the
        head) or None.  Order: every chunk forward over all micro-batches, chunk by chunk, then the
        chunks in reverse order backward over all micro-batches."""
        e = self.env
        assert len(microbatches) == self.n_micro
        e.run(self.p_begin)
        self.losses = []
        if self.world == 1:
            c = self.chunks[0]
            for mb in microbatches:
                self._feed(c, mb)
                e.run(c["fwd"][0])
                e.run(c["bwd"][0])
                self.losses.append(host.last_loss())
        else:
            for c in self.chunks:
                for k, mb in enumerate(microbatches):
                    self._feed(c, mb)
                    e.run(c["fwd"][k])
            for c in reversed(self.chunks):
                for k, mb in enumerate(microbatches):
                    self._feed(c, mb)
                    e.run(c["bwd"][k])
                    if c["last"]:
                        self.losses.append(host.last_loss())
            if self.first != self.last:          # the two holders of the tied table sum their gradients
                holder = self.chunks[0] if self.first else self.chunks[-1]
                head_rank = next(r for r, ch in enumerate(self.plan) if any(c["last"] for c in ch))
                peer = head_rank if self.first else 0
                e.execute(f"{peer} sync_tied_grads{holder['sfx']}")
        self.step_no += 1
        # gradients were summed over micro-batches and carry the loss scale: Adam divides both out
        gs = 1.0 / (self.loss_scale * self.n_micro)
        e.execute("0 op.accumulate " + " ".join(f"{self.lr} {self.step_no} {gs} optimizer_step{c['sfx']}" for c in self.chunks))
        return float(np.mean(self.losses)) if self.losses else None

    def sync(self):
        self.env.run(self.p_sync)

    def close(self):
        for c in self.chunks:
            for p in c["fwd"] + c["bwd"]:
                self.env.free_program(p)
        self.env.free_program(self.p_begin)
        self.env.free_program(self.p_sync)
        self.env.close()


def gemm_flops_per_microbatch(hidden, vocab, n_layers, tokens_total, with_head=True):
    """FLOPs of every GEMM launch of one micro-batch's forward + backward (2 m n k each; the
    backward has two GEMMs per forward GEMM)."""
    per_layer_fwd = 2 * tokens_total * 12 * hidden * hidden
    head_fwd = 2 * tokens_total * hidden * vocab
    return 3 * n_layers * per_layer_fwd + (3 * head_fwd if with_head else 0)
