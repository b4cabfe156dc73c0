"""Static task order of the overlapped pipeline (CPU): the greedy lists respect every dependency and slot limit,
broken lists are caught before anything would be queued on a GPU, and the simulated fill / drain behaves as the
arithmetic says."""
import pytest

from blackriver_b200 import schedule as S
from blackriver_b200.finetune import partition_layers


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("n_micro,n_slots", [(16, 16), (16, 8), (16, 3), (4, 4), (5, 2), (1, 1)])
def test_greedy_lists_are_valid(world, n_micro, n_slots):
    counts = partition_layers(30, world)
    costs = S.stage_costs(counts)
    orders, span = S.build(world, n_micro, costs, n_slots)
    assert len(orders) == world
    replayed = S.check(orders, n_micro, n_slots, costs)
    assert abs(replayed - span) <= 1e-6 * span
    for o in orders:                                   # per kind the micro-batches go in order on every rank
        for kind in "FBW":
            ks = [t.k for t in o if t.kind == kind]
            assert ks == sorted(ks) == list(range(n_micro))
    assert 0 < S.efficiency(span, costs, n_micro) <= 1.0


def test_greedy_beats_the_plain_order_on_the_benchmark_shapes():
    for world, floor in ((2, 0.93), (4, 0.88), (8, 0.75)):
        counts = partition_layers(30, world)
        costs = S.stage_costs(counts)
        _, span = S.build(world, 16, costs, 16)
        plain = S.check(S.gpipe(world, 16), 16, 16, costs)
        assert span < plain
        assert S.efficiency(span, costs, 16) >= floor, (world, S.efficiency(span, costs, 16))


def test_single_rank_needs_no_idle_time():
    costs = S.stage_costs([30])
    orders, span = S.build(1, 4, costs, 4)
    assert abs(span - 4 * sum(costs[0])) < 1e-9
    assert S.check(orders, 4, 4, costs) == pytest.approx(span)


def test_check_rejects_broken_lists():
    costs = S.stage_costs([2, 2])
    orders, _ = S.build(2, 4, costs, 4)
    bad = [list(o) for o in orders]
    bad[1].pop()
    with pytest.raises(ValueError, match="permutation"):
        S.check(bad, 4, 4)
    # rank 0 wants the gradient of micro-batch 0 before it has sent micro-batch 0 forward: nobody can move
    bad = [list(o) for o in orders]
    i_f, i_b = bad[0].index(S.Task("F", 0)), bad[0].index(S.Task("B", 0))
    bad[0][i_f], bad[0][i_b] = bad[0][i_b], bad[0][i_f]
    with pytest.raises(ValueError, match="deadlock"):
        S.check(bad, 4, 4)
    # a list made for 4 slots does not fit 2: a forward would overwrite activations whose weight gradients are pending
    orders4, _ = S.build(2, 8, costs, 8)
    with pytest.raises(ValueError, match="deadlock"):
        S.check(orders4, 8, 2)


def test_slot_count_follows_the_activation_budget():
    act = 2 * 1024 * 4096 * 2
    assert S.n_slots_for(1, 16, [30], 23 * act) == 1
    assert S.n_slots_for(8, 16, [5, 5, 4, 4, 4, 4, 4, 0], 23 * act) == 16
    assert 2 <= S.n_slots_for(2, 16, [18, 12], 23 * act) < 16
    assert S.n_slots_for(2, 16, [18, 12], 23 * act, budget_bytes=1) == 2


def test_last_rank_takes_head_gradients_first_and_marks_the_exchange():
    """The last rank's list with every W cut into the LM-head part H and the layers' part W: H(k) comes before W(k) and
    after B(k), the exchange marker X comes after the last H and after the last B, and what follows X is only layers'
    weight gradients (work that nothing but this rank's own optimizer waits for)."""
    for world, n_micro, slots in ((2, 4, 4), (4, 16, 16), (8, 16, 16), (3, 6, 3)):
        costs = S.stage_costs_units(S.choose_partition_units(12, world, n_micro, slots))
        orders, _ = S.build(world, n_micro, costs, slots)
        ex = S.expand_last_rank(orders[-1])
        kinds = [t.kind for t in ex]
        assert kinds.count("X") == 1 and kinds.count("H") == n_micro and kinds.count("W") == n_micro
        x = kinds.index("X")
        assert all(k == "W" for k in kinds[x + 1:])
        pos = {(t.kind, t.k): i for i, t in enumerate(ex)}
        for k in range(n_micro):
            assert pos[("B", k)] < pos[("H", k)] < pos[("W", k)]
            assert pos[("H", k)] < x and pos[("B", k)] < x
        # without the cut the list is the original one
        assert [t for t in ex if t.kind in "FBW"] == list(orders[-1])


def test_steady_state_period():
    """Consecutive steps without a barrier: the step time in the steady state is at least the largest per-rank work
    plus that rank's optimizer, never more than an isolated step plus the slowest optimizer, and the partition chosen
    for it is no worse, by that measure, than the one chosen for an isolated step."""
    for world, slots in ((2, 8), (4, 16), (8, 16)):
        n_micro = 16
        res = {}
        for steady in (False, True):
            b = S.choose_partition_units(30, world, n_micro, slots, steady=steady)
            costs = S.stage_costs_units(b)
            layers = [(b[r + 1] - b[r]) / 2 for r in range(world)]
            orders, span = S.build(world, n_micro, costs, slots)
            period = S.steady_period(orders, costs, n_micro, slots, layers=layers)
            work = max(n_micro * sum(c) + S.ADAM_LAYER_COST * l for c, l in zip(costs, layers))
            assert work - 1e-6 <= period <= span + S.ADAM_LAYER_COST * max(layers) + S.ADAM_TABLE_COST + S.TIED_EXCHANGE_COST + 1e-6
            res[steady] = period
        assert res[True] <= res[False] + 1e-6
    # one rank: the period is the work of the step plus the optimizer
    costs = S.stage_costs_units([0, 60])
    orders, span = S.build(1, 4, costs, 1)
    assert abs(S.steady_period(orders, costs, 4, 1, layers=[30]) - (span + 30 * S.ADAM_LAYER_COST + S.ADAM_TABLE_COST)) < 1e-6
