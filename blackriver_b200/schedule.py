"""Static task order of the overlapped pipeline.

The reference runs its stages strictly one after the other: every layer's forward, then the loss and one backward
(blackriver/train_bloom.cpp:211-241), with blocking hand-offs (bloomz-7b/train.words:250-258).  Here a training step is
cut, per rank and micro-batch k, into three tasks

    F(k)  forward of the stage                      needs F(k) of the previous rank
    B(k)  input gradients of the stage               needs F(k) here and B(k) of the next rank
    W(k)  weight gradients (column sums + dy^T x)    needs B(k) here; nothing waits for it but the optimizer

and every rank executes a fixed list of them.  Hand-offs are one-sided and buffered (PipeLinks), so any list that
respects the data dependencies is safe; the list decides how much of the fill and drain of the pipeline is spent idle.
`build` produces the lists with a greedy event simulation (a rank that becomes free takes, in this order of
preference, a ready B, a ready F, a pending W); `check` replays lists against the dependencies and reports a deadlock
or a memory-slot conflict before anything is queued on a GPU.

Slots: a rank keeps the saved activations of at most `n_slots` micro-batches, micro-batch k using slot k % n_slots, so
F(k) may only start once W(k - n_slots) has finished on that rank.
"""
from dataclasses import dataclass

# Costs of one decoder layer's three tasks and of the LM head + loss (milliseconds per micro-batch of 2048 tokens on a
# B200, from the measured task durations of the 7b1-shaped step on two stages; only their ratios matter): forward GEMMs + attention forward; input-gradient GEMMs +
# attention backward + LayerNorm / GELU backward; weight-gradient GEMMs + column sums.  The head's forward part
# (logits GEMM + log-softmax) is counted with its B task because it runs there.
LAYER_COST = (0.786, 0.924, 0.685)
HEAD_COST = (0.5, 6.2, 3.6)


@dataclass(frozen=True)
class Task:
    kind: str      # "F", "B" or "W"
    k: int         # micro-batch


def stage_costs(counts, layer_cost=LAYER_COST, head_cost=HEAD_COST):
    """(F, B, W) cost of one micro-batch on every rank; the last rank carries the head."""
    out = []
    for r, n in enumerate(counts):
        f, b, w = (n * c for c in layer_cost)
        if r == len(counts) - 1:
            f, b, w = f + head_cost[0], b + head_cost[1], w + head_cost[2]
        out.append((max(f, 1e-3), max(b, 1e-3), max(w, 1e-3)))
    return out


def _deps(world, n_slots, r, t):
    """Tasks (rank, Task) that must have finished before task t may start on rank r."""
    d = []
    if t.kind == "F":
        if r > 0:
            d.append((r - 1, Task("F", t.k)))
        if t.k >= n_slots:
            d.append((r, Task("W", t.k - n_slots)))
    elif t.kind == "B":
        d.append((r, Task("F", t.k)))
        if r < world - 1:
            d.append((r + 1, Task("B", t.k)))
    else:
        d.append((r, Task("B", t.k)))
    return d


def build(world, n_micro, costs, n_slots=None, link_latency=0.02, patience=0.25):
    """Greedy list schedule.  costs[r] = (F, B, W) durations of one micro-batch on rank r.
    `patience`: a rank about to start a W although a B or F becomes ready within patience x (cost of W) waits for that
    task instead.  Returns (orders, makespan): orders[r] is rank r's task list, makespan the simulated step time."""
    n_slots = n_micro if n_slots is None else max(1, min(n_slots, n_micro))
    done = {}                                   # (rank, Task) -> finish time
    orders = [[] for _ in range(world)]
    free_at = [0.0] * world
    nxt = [{"F": 0, "B": 0, "W": 0} for _ in range(world)]
    total = 3 * n_micro
    dur = {"F": 0, "B": 1, "W": 2}

    def ready_time(r, t):
        """Time at which every dependency has finished (None while one of them is not scheduled yet)."""
        when = 0.0
        for (dr, dt) in _deps(world, n_slots, r, t):
            f = done.get((dr, dt))
            if f is None:
                return None
            when = max(when, f + (link_latency if dr != r else 0.0))
        return when

    while any(len(o) < total for o in orders):
        # Decisions are taken in the order of simulated time: the rank whose next start comes first decides next, so
        # everything that finishes before that moment is already known.
        best = None
        for r in range(world):
            if len(orders[r]) == total:
                continue
            cands = []
            for pref, kind in enumerate(("B", "F", "W")):
                k = nxt[r][kind]
                if k >= n_micro:
                    continue
                when = ready_time(r, Task(kind, k))
                if when is not None:
                    cands.append((when, pref, kind, k))
            if not cands:
                continue
            now = free_at[r]
            startable = [c for c in cands if c[0] <= now + 1e-12]
            if startable:
                _, pref, kind, k = min(startable, key=lambda c: c[1])
                start = now
                if kind == "W":
                    # a weight-gradient pass cannot be interrupted: leave a gap rather than make a task that feeds
                    # another rank wait for most of it
                    soon = [c for c in cands if c[1] < 2 and c[0] < now + patience * costs[r][2]]
                    if soon:
                        start, pref, kind, k = min(soon, key=lambda c: (c[0], c[1]))
            else:
                start, pref, kind, k = min(cands, key=lambda c: (c[0], c[1]))
            if best is None or (start, r) < best[:2]:
                best = (start, r, kind, k)
        if best is None:
            raise RuntimeError("schedule.build: no task can start (dependency cycle)")
        start, r, kind, k = best
        t = Task(kind, k)
        done[(r, t)] = start + costs[r][dur[kind]]
        free_at[r] = done[(r, t)]
        orders[r].append(t)
        nxt[r][kind] += 1
    return orders, max(free_at)


def gpipe(world, n_micro):
    """All forwards, then backward and weight gradients micro-batch by micro-batch: the plain schedule."""
    one = [Task("F", k) for k in range(n_micro)]
    for k in range(n_micro):
        one += [Task("B", k), Task("W", k)]
    return [list(one) for _ in range(world)]


def check(orders, n_micro, n_slots, costs=None, link_latency=0.02):
    """Replays the per-rank lists against the dependencies.  Raises ValueError on an incomplete list, a task before its
    dependency on the same rank, or a deadlock across ranks.  Returns the simulated step time when costs are given
    (every rank executes its list in order, starting each task as soon as its dependencies have finished), else None."""
    world = len(orders)
    n_slots = max(1, min(n_slots, n_micro))
    want = {Task(kind, k) for kind in "FBW" for k in range(n_micro)}
    for r, o in enumerate(orders):
        if len(o) != len(want) or set(o) != want:
            raise ValueError(f"rank {r}: the list is not a permutation of F, B, W over {n_micro} micro-batches")
    pos = [0] * world
    done = {}
    free_at = [0.0] * world
    dur = {"F": 0, "B": 1, "W": 2}
    while any(pos[r] < len(orders[r]) for r in range(world)):
        moved = False
        for r in range(world):
            while pos[r] < len(orders[r]):
                t = orders[r][pos[r]]
                when = 0.0
                ok = True
                for (dr, dt) in _deps(world, n_slots, r, t):
                    f = done.get((dr, dt))
                    if f is None:
                        ok = False
                        break
                    when = max(when, f + (link_latency if dr != r else 0.0))
                if not ok:
                    break
                start = max(when, free_at[r])
                free_at[r] = start + (costs[r][dur[t.kind]] if costs else 1.0)
                done[(r, t)] = free_at[r]
                pos[r] += 1
                moved = True
        if not moved:
            stuck = {r: orders[r][pos[r]] for r in range(world) if pos[r] < len(orders[r])}
            raise ValueError(f"deadlock: every rank waits for a task that never runs: {stuck}")
    return max(free_at) if costs else None


# ---- consecutive steps -------------------------------------------------------------------------------------------------
# A rank starts the next step as soon as its own list and its own optimizer step are done; there is no barrier between
# steps.  A later rank therefore spends the time in which it would wait for the next step's first micro-batch on the
# weight-gradient tasks it still has left over, so in the steady state the pipeline's fill costs nothing as long as every
# rank has at least that much deferred work, and the step time tends to the largest per-rank work instead of work + fill.
# The one coupling between the two ends is the tied table: the first rank's update of it needs the last rank's LM-head
# gradient.  The last rank therefore takes the head's part of its deferred weight-gradient tasks first ("H"), starts the
# exchange ("X") and only then works off the layers' parts ("W").
ADAM_LAYER_COST = 1.0        # ms per decoder layer per step (28 bytes per parameter at HBM speed)
ADAM_TABLE_COST = 3.0        # the 250880 x 4096 table
TIED_EXCHANGE_COST = 3.0     # 2 GB each way over NVLink


def expand_last_rank(order):
    """The last rank's list with every W(k) cut into H(k) (LM-head weight gradient) and W(k) (its layers): pairs stay
    together up to the last B; what is left after it runs heads first, then the exchange marker X, then the layers."""
    last_b = max((i for i, t in enumerate(order) if t.kind == "B"), default=-1)
    out = []
    for t in order[:last_b + 1]:
        if t.kind == "W":
            out.append(Task("H", t.k))
        out.append(t)
    tail = [t for t in order[last_b + 1:]]
    out += [Task("H", t.k) for t in tail if t.kind == "W"]
    out.append(Task("X", -1))
    out += tail
    return out


def steady_period(orders, costs, n_micro, n_slots, head_w=None, layers=None, link_latency=0.02, steps=3):
    """Step time in the steady state: `steps` consecutive steps are replayed, every rank running its list in order and
    then its optimizer step (layers' Adam; the holders of the tied table exchange its gradient once both have it and
    update it last), and the time between the ends of the last two steps is returned.
    head_w = the LM-head part of the last rank's W cost; layers[r] = decoder layers on rank r (for Adam's cost)."""
    world = len(orders)
    n_slots = max(1, min(n_slots, n_micro))
    head_w = HEAD_COST[2] if head_w is None else head_w
    layers = layers or [0.0] * world
    lists = [list(o) for o in orders]
    if world > 1:
        lists[-1] = expand_last_rank(orders[-1])
    dur = {"F": 0, "B": 1, "W": 2}

    def cost(r, t):
        if t.kind == "X":
            return 0.0
        if t.kind == "H":
            return min(head_w, costs[r][2])
        c = costs[r][dur[t.kind]]
        if t.kind == "W" and world > 1 and r == world - 1:
            c = max(c - head_w, 0.0)
        return c

    free_at = [0.0] * world
    ends = []
    for _ in range(steps):
        pos = [0] * world
        done = {}
        table_ready = [None, None]          # first rank: after its last B; last rank: at X
        while any(pos[r] < len(lists[r]) for r in range(world)):
            moved = False
            for r in range(world):
                while pos[r] < len(lists[r]):
                    t = lists[r][pos[r]]
                    when = 0.0
                    ok = True
                    deps = [] if t.kind in "HX" else _deps(world, n_slots, r, t)
                    if t.kind == "H":
                        deps = [(r, Task("B", t.k))]
                    for (dr, dt) in deps:
                        f = done.get((dr, dt))
                        if f is None:
                            ok = False
                            break
                        when = max(when, f + (link_latency if dr != r else 0.0))
                    if not ok:
                        break
                    start = max(when, free_at[r])
                    free_at[r] = start + cost(r, t)
                    done[(r, t)] = free_at[r]
                    if t.kind == "X":
                        table_ready[1] = free_at[r]
                    if r == 0 and t.kind == "B" and t.k == n_micro - 1:
                        pass
                    pos[r] += 1
                    moved = True
            if not moved:
                raise ValueError("deadlock in the replay of consecutive steps")
        last_b0 = max(done[(0, Task("B", k))] for k in range(n_micro))
        table_ready[0] = last_b0
        if world > 1:
            exchanged = max(table_ready[0], table_ready[1]) + TIED_EXCHANGE_COST
        for r in range(world):
            t_end = free_at[r] + ADAM_LAYER_COST * layers[r]
            if world > 1 and (r == 0 or r == world - 1):
                t_end = max(t_end, exchanged) + ADAM_TABLE_COST
            elif world == 1:
                t_end += ADAM_TABLE_COST
            free_at[r] = t_end
        ends.append(max(free_at))
    return ends[-1] - ends[-2] if steps > 1 else ends[-1]


def efficiency(makespan, costs, n_micro):
    """Simulated step time of one rank doing all the work, divided by (ranks x the pipeline's step time)."""
    return n_micro * sum(sum(c) for c in costs) / (len(costs) * makespan)


def n_slots_for(world, n_micro, layers_per_rank, bytes_per_layer_slot, budget_bytes=56 << 30):
    """Micro-batches whose saved activations (and kept gradients) fit the activation budget of the fullest rank."""
    if world == 1:
        return 1
    per_slot = max(1, max(layers_per_rank)) * bytes_per_layer_slot
    return int(max(2, min(n_micro, budget_bytes // max(per_slot, 1))))


def choose_partition(n_layers, world, n_micro, n_slots=None, layer_cost=LAYER_COST, head_cost=HEAD_COST):
    """Contiguous layer counts per rank (the last rank also carries final LayerNorm + LM head + loss and may hold no
    layer at all) with the shortest simulated step.  Candidates: every number of layers next to the head up to an even
    share, the other layers spread as evenly as whole layers allow, the fuller stages anywhere among the ranks."""
    if world == 1:
        return [n_layers]
    from itertools import combinations
    best = None
    for last in range(0, n_layers // world + 2):
        rest = n_layers - last
        if rest < world - 1:
            continue
        lo, extra = divmod(rest, world - 1)
        for where in combinations(range(world - 1), extra):
            counts = [lo + (1 if i in where else 0) for i in range(world - 1)] + [last]
            costs = stage_costs(counts, layer_cost, head_cost)
            _, span = build(world, n_micro, costs, n_slots)
            key = (round(span, 6), [-c for c in counts])          # ties: the fuller stages first
            if best is None or key < best[0]:
                best = (key, counts)
    return best[1]


# ---- stages cut at half-layer boundaries -----------------------------------------------------------------------------
# A decoder layer is two units: "A" = input LayerNorm, QKV projection, attention, dense projection + residual;
# "M" = post-attention LayerNorm, h -> 4h + GELU, 4h -> h + residual.  The tensor between them (the residual stream after
# attention) has the same shape as a layer's output, so a stage boundary may fall there too, which lets 30 layers be
# spread over 7 ranks in pieces of 4.3 layers instead of 5 and 4.  Costs (F, B, W) in the unit of LAYER_COST, from the
# same measured profile: A carries a third of the layer's GEMM FLOPs plus the attention kernels, M two thirds.
UNIT_COST = {"A": (0.327, 0.439, 0.250), "M": (0.459, 0.485, 0.435)}
# What the two holders of the tied 250880 x 4096 table carry besides their layers, per micro-batch: the embedding gather +
# LayerNorm and their backward (first rank only), and a sixteenth of the table's Adam update and gradient exchange
TABLE_COST = (0.04, 0.08, 0.45)


def unit_kind(u):
    return "A" if u % 2 == 0 else "M"


def stage_costs_units(bounds, unit_cost=None, head_cost=HEAD_COST):
    """bounds = [u_0 = 0, u_1, ..., u_world = 2 * layers]: rank r owns units [u_r, u_r+1).  (F, B, W) per micro-batch and rank."""
    unit_cost = unit_cost or UNIT_COST
    out = []
    world = len(bounds) - 1
    for r in range(world):
        f = b = w = 0.0
        for u in range(bounds[r], bounds[r + 1]):
            c = unit_cost[unit_kind(u)]
            f, b, w = f + c[0], b + c[1], w + c[2]
        if r == world - 1:
            f, b, w = f + head_cost[0], b + head_cost[1], w + head_cost[2]
        if world > 1 and (r == 0 or r == world - 1):
            f, b, w = f + TABLE_COST[0] * (r == 0), b + TABLE_COST[1] * (r == 0), w + TABLE_COST[2]
        out.append((max(f, 1e-3), max(b, 1e-3), max(w, 1e-3)))
    return out


def choose_partition_units(n_layers, world, n_micro, n_slots=None, unit_cost=None, head_cost=HEAD_COST, whole_layers=False,
                           steady=False):
    """Stage boundaries in units (2 per layer) with the shortest simulated step.  Candidates come from an exact search
    (dynamic programme over contiguous splits) for the split that minimises the largest of
    n_micro x (work of the stage) + alpha x (forward time of everything before it), for several alpha: the second term
    is the time a stage has to wait for its first micro-batch, which later stages cannot get back.  Every rank but the
    last owns at least one unit; the last may own none (head only).  whole_layers=True allows boundaries between layers only."""
    unit_cost = unit_cost or UNIT_COST
    n_units = 2 * n_layers
    if world == 1:
        return [0, n_units]
    step = 2 if whole_layers else 1
    cost = [sum(unit_cost[unit_kind(u)]) for u in range(n_units)]
    fwd = [unit_cost[unit_kind(u)][0] for u in range(n_units)]
    pre_c = [0.0]
    pre_f = [0.0]
    for u in range(n_units):
        pre_c.append(pre_c[-1] + cost[u])
        pre_f.append(pre_f[-1] + fwd[u])
    head = sum(head_cost)
    points = list(range(0, n_units + 1, step))
    best = None
    seen = set()
    for alpha in (0.0, 0.5, 1.0, 1.5, 2.0, 3.0):
        def stage(a, b, is_last):
            return n_micro * (pre_c[b] - pre_c[a] + (head if is_last else 0.0)) + alpha * pre_f[a]
        INF = float("inf")
        # dp[r][i]: best (smallest) largest-stage value when the first r ranks own units [0, points[i])
        dp = [[INF] * len(points) for _ in range(world + 1)]
        arg = [[-1] * len(points) for _ in range(world + 1)]
        dp[0][0] = 0.0
        for r in range(1, world + 1):
            last = r == world
            for i in range(len(points)):
                if last and points[i] != n_units:
                    continue
                for k in range(len(points)):
                    if k > i or dp[r - 1][k] == INF:
                        continue
                    if not last and k == i:
                        continue                      # every rank but the last owns something
                    v = max(dp[r - 1][k], stage(points[k], points[i], last))
                    if v < dp[r][i]:
                        dp[r][i], arg[r][i] = v, k
        i = len(points) - 1
        if dp[world][i] == INF:
            continue
        bounds = [n_units]
        for r in range(world, 0, -1):
            i = arg[r][i]
            bounds.append(points[i])
        bounds.reverse()
        if tuple(bounds) in seen:
            continue
        seen.add(tuple(bounds))
        costs = stage_costs_units(bounds, unit_cost, head_cost)
        orders, span = build(world, n_micro, costs, n_slots)
        if steady:
            span = steady_period(orders, costs, n_micro, n_slots if n_slots else n_micro, head_w=head_cost[2],
                                 layers=[(bounds[r + 1] - bounds[r]) / 2 for r in range(world)])
        if best is None or span < best[0] - 1e-9:
            best = (span, bounds)
    if best is None:
        raise ValueError("more ranks than units to give them")
    return best[1]
