"""Discrete-event model of the pipeline schedules, for reasoning about them without GPUs.

A schedule is one ordered list of operations per rank -- what the rank's compute stream executes:
    ("work", cost)                  compute
    ("send", peer) / ("recv", peer) a stage hand-off; matched in order per (sender, receiver) pair
Two link models:
    rendezvous   a send completes only when the receiver has reached the matching recv (what
                 ncclSend / ncclRecv of a 16.8 MB activation do), so sender and receiver leave together
    buffered     a send never waits (one-sided write into a per-micro-batch receive window); the
                 receiver waits for the data
`simulate` reports whether every rank finishes (a False is a deadlock of the schedule under that link
model) and the makespan.  Costs are in units of one decoder layer's forward; a layer's backward costs
two, the head (final LayerNorm + LM head + loss) `head_cost` layers for forward + backward together.

The model reproduces the measured scaling of the all-forward-then-all-backward schedule (0.84 on 4
GPUs, 0.58-0.64 on 8) and is how candidate schedules are compared before they are built."""
from . import finetune

FWD, BWD = 1.0, 2.0      # cost of one layer, forward / backward


def stage_costs(counts, head_cost):
    """(forward, backward) cost per micro-batch of every stage; the head splits 1 : 2 like a layer."""
    out = []
    for r, c in enumerate(counts):
        extra = head_cost if r == len(counts) - 1 else 0.0
        out.append((c * FWD + extra * FWD, c * BWD + extra * BWD))
    return out


def gpipe_programs(counts, n_micro, head_cost=finetune.LM_HEAD_COST_IN_LAYERS):
    """Every micro-batch forward through all stages, then every micro-batch backward (finetune.Trainer.step)."""
    world = len(counts)
    costs = stage_costs(counts, head_cost)
    progs = []
    for r in range(world):
        ops = []
        for _ in range(n_micro):
            if r > 0:
                ops.append(("recv", r - 1))
            ops.append(("work", costs[r][0]))
            if r < world - 1:
                ops.append(("send", r + 1))
        for _ in range(n_micro):
            if r < world - 1:
                ops.append(("recv", r + 1))
            ops.append(("work", costs[r][1]))
            if r > 0:
                ops.append(("send", r - 1))
        progs.append(ops)
    return progs


def one_f_one_b_programs(counts, n_micro, head_cost=finetune.LM_HEAD_COST_IN_LAYERS):
    """Warm-up forwards, then alternating one forward / one backward, then the remaining backwards."""
    world = len(counts)
    costs = stage_costs(counts, head_cost)
    progs = []
    for r in range(world):
        warm = min(world - 1 - r, n_micro)
        ops = []

        def fwd():
            if r > 0:
                ops.append(("recv", r - 1))
            ops.append(("work", costs[r][0]))
            if r < world - 1:
                ops.append(("send", r + 1))

        def bwd():
            if r < world - 1:
                ops.append(("recv", r + 1))
            ops.append(("work", costs[r][1]))
            if r > 0:
                ops.append(("send", r - 1))

        for _ in range(warm):
            fwd()
        for _ in range(n_micro - warm):
            fwd()
            bwd()
        for _ in range(warm):
            bwd()
        progs.append(ops)
    return progs


def simulate(programs, link="rendezvous"):
    """Runs the per-rank programs; returns (finished, makespan, per-rank busy time)."""
    assert link in ("rendezvous", "buffered")
    world = len(programs)
    pc = [0] * world
    clock = [0.0] * world
    busy = [0.0] * world
    mailbox = {}      # (src, dst) -> arrival times of sent, not yet received messages (buffered links)
    progressed = True
    while progressed:
        progressed = False
        for r in range(world):
            while pc[r] < len(programs[r]):
                op = programs[r][pc[r]]
                if op[0] == "work":
                    clock[r] += op[1]
                    busy[r] += op[1]
                elif op[0] == "send":
                    dst = op[1]
                    if link == "buffered":
                        mailbox.setdefault((r, dst), []).append(clock[r])
                    else:
                        nxt = programs[dst][pc[dst]] if pc[dst] < len(programs[dst]) else None
                        if nxt != ("recv", r):
                            break      # the receiver is not there yet
                        t = max(clock[r], clock[dst])
                        clock[r] = clock[dst] = t
                        pc[dst] += 1
                elif op[0] == "recv":
                    if link == "rendezvous":
                        break          # completed by the sender's branch above
                    box = mailbox.get((op[1], r))
                    if not box:
                        break
                    clock[r] = max(clock[r], box.pop(0))
                pc[r] += 1
                progressed = True
    finished = all(pc[r] == len(programs[r]) for r in range(world))
    return finished, max(clock), busy


def efficiency(counts, n_micro, programs, link="rendezvous", head_cost=finetune.LM_HEAD_COST_IN_LAYERS):
    """Scaling efficiency the schedule would reach: one GPU's time for the same work / (ranks x makespan)."""
    ok, span, _ = simulate(programs, link)
    if not ok:
        return None
    single = n_micro * (sum(counts) + head_cost) * (FWD + BWD)
    return single / (len(counts) * span)


def greedy_estimate(layer_counts, n_micro, head_cost=finetune.LM_HEAD_COST_IN_LAYERS, tail_layers=0, tail_replicas=1,
                    split_backward=False, return_order=False):
    """Upper estimate for schedules that need buffered links: greedy list scheduling of the tasks F(stage, mb), B(stage, mb)
    and, with split_backward, W(stage, mb) -- the weight gradients, which nothing downstream waits for and which therefore
    fill idle time (priority: B, then F, then W).  The stages are the entries of layer_counts, one rank each, followed
    by a tail stage of `tail_layers` layers + the head, replicated on `tail_replicas` ranks that take the micro-batches in
    turn.  Costs: forward, input-gradient and weight-gradient pass of a layer one unit each (the backward of the other
    schedules is the last two together).  Returns the scaling efficiency, and with return_order also the order in which
    every rank starts its tasks: a static schedule that `replay` can execute."""
    stages = [float(c) for c in layer_counts] + [float(tail_layers) + head_cost]
    n_stage = len(stages)
    n_body = len(layer_counts)
    world = n_body + tail_replicas
    kinds = 3 if split_backward else 2

    def rank_of(s, m):
        return s if s < n_body else n_body + m % tail_replicas

    def cost(s, kind):
        return stages[s] if (split_backward or kind == 0) else 2.0 * stages[s]

    ready = [[] for _ in range(world)]
    clock = [0.0] * world
    order = [[] for _ in range(world)]      # (kind, stage, micro-batch) in the order each rank starts them
    for m in range(n_micro):
        ready[rank_of(0, m)].append(((1, m, 0), 0.0, 0, m, 0))
    left = kinds * n_stage * n_micro
    while left:
        best = None
        for r in range(world):
            if not ready[r]:
                continue
            avail = [x for x in ready[r] if x[1] <= clock[r] + 1e-12]
            cand, start = (min(avail), clock[r]) if avail else (min(ready[r], key=lambda x: (x[1], x[0])), None)
            if start is None:
                start = cand[1]
            if best is None or start < best[0]:
                best = (start, r, cand)
        start, r, cand = best
        ready[r].remove(cand)
        _, _, s, m, kind = cand
        end = start + cost(s, kind)
        clock[r] = end
        order[r].append(("FBW"[kind], s, m))
        left -= 1
        if kind == 0:
            if s + 1 < n_stage:
                ready[rank_of(s + 1, m)].append(((1, m, s + 1), end, s + 1, m, 0))
            else:
                ready[rank_of(s, m)].append(((0, m, s), end, s, m, 1))
        elif kind == 1:
            if split_backward:
                ready[rank_of(s, m)].append(((2, m, s), end, s, m, 2))
            if s > 0:
                ready[rank_of(s - 1, m)].append(((0, m, s - 1), end, s - 1, m, 1))
    single = n_micro * (sum(layer_counts) + tail_layers + head_cost) * 3.0
    if return_order:
        return single / (world * max(clock)), order
    return single / (world * max(clock))


def replay(order, layer_counts, n_micro, head_cost=finetune.LM_HEAD_COST_IN_LAYERS, tail_layers=0, tail_replicas=1,
           split_backward=False):
    """Executes a static schedule -- per rank the list of ("F" | "B" | "W", stage, micro-batch) in issue order, as
    greedy_estimate(..., return_order=True) produces it -- with buffered links: a task starts when the rank has finished
    the task before it and its inputs have arrived.  Returns (finished, efficiency, what has to be kept): the largest
    number of micro-batches whose activations a rank holds at once (forward done, backward not yet) and the largest
    number of deferred weight-gradient passes (backward done, W not yet), per rank."""
    stages = [float(c) for c in layer_counts] + [float(tail_layers) + head_cost]
    n_stage, n_body = len(stages), len(layer_counts)
    world = n_body + tail_replicas
    done = {}
    pc = [0] * world
    clock = [0.0] * world
    live_act = [0] * world
    live_w = [0] * world
    peak_act = [0] * world
    peak_w = [0] * world

    def needs(kind, s, m):
        if kind == "F":
            return [("F", s - 1, m)] if s > 0 else []
        if kind == "B":
            return [("F", s, m)] + ([("B", s + 1, m)] if s + 1 < n_stage else [])
        return [("B", s, m)]

    progressed = True
    while progressed:
        progressed = False
        for r in range(world):
            while pc[r] < len(order[r]):
                kind, s, m = order[r][pc[r]]
                deps = needs(kind, s, m)
                if any(d not in done for d in deps):
                    break
                start = max([clock[r]] + [done[d] for d in deps])
                c = stages[s] if (split_backward or kind == "F") else 2.0 * stages[s]
                clock[r] = done[(kind, s, m)] = start + c
                if kind == "F":
                    live_act[r] += 1
                elif kind == "B":
                    if split_backward:
                        live_w[r] += 1
                    else:
                        live_act[r] -= 1
                else:
                    live_w[r] -= 1
                    live_act[r] -= 1      # the layer inputs are needed until the weight gradients have been taken
                peak_act[r] = max(peak_act[r], live_act[r])
                peak_w[r] = max(peak_w[r], live_w[r])
                pc[r] += 1
                progressed = True
    finished = all(pc[r] == len(order[r]) for r in range(world))
    single = n_micro * (sum(layer_counts) + tail_layers + head_cost) * 3.0
    return finished, (single / (world * max(clock)) if finished else None), {"activations": peak_act, "deferred": peak_w}


def report(n_layers=30, n_micro=16, head_cost=finetune.LM_HEAD_COST_IN_LAYERS):
    rows = []
    for world in (2, 4, 8):
        counts = finetune.partition_layers(n_layers, world, head_cost)
        for name, build in (("all-forward-all-backward", gpipe_programs), ("one-forward-one-backward", one_f_one_b_programs)):
            for link in ("rendezvous", "buffered"):
                rows.append((world, counts, name, link, efficiency(counts, n_micro, build(counts, n_micro, head_cost), link, head_cost)))
    return rows


if __name__ == "__main__":
    for world, counts, name, link, eff in report():
        print(f"{world} GPUs {counts}  {name:26s} {link:10s}  " + ("deadlock" if eff is None else f"{eff:.3f}"))
    print("greedy estimates, buffered links, 16 micro-batches:")
    for label, kw in (("4 GPUs [9,9,9]+head", dict(layer_counts=[9, 9, 9], tail_layers=3)),
                      ("8 GPUs [5,5,4,4,4,4,4]+head", dict(layer_counts=[5, 5, 4, 4, 4, 4, 4])),
                      ("8 GPUs [5,5,5,4,4,4] + (3 layers + head) x 2 ranks", dict(layer_counts=[5, 5, 5, 4, 4, 4], tail_layers=3, tail_replicas=2))):
        a = greedy_estimate(n_micro=16, **kw)
        b = greedy_estimate(n_micro=16, split_backward=True, **kw)
        print(f"  {label:52s} backward whole {a:.3f}   weight gradients deferred {b:.3f}")
