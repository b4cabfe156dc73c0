"""The schedule the Trainer runs, checked on the discrete-event model: it must finish under rendezvous sends (a
send that waits for its receiver, which is how large NCCL point-to-point transfers behave), and the model must
stay close to the measured scaling so that it can be trusted when schedules are compared."""
from blackriver_b200 import finetune, pipeline_sim as ps


def test_trainer_schedule_finishes_under_rendezvous_sends():
    for world in (2, 3, 4, 8):
        for n_micro in (1, 2, 16):
            counts = finetune.partition_layers(30, world)
            ok, span, busy = ps.simulate(ps.gpipe_programs(counts, n_micro), "rendezvous")
            assert ok, (world, n_micro)
            assert span >= max(busy) > 0


def test_model_matches_measured_scaling():
    # measured on B200s: 0.85 on 4 GPUs ([9,9,9,3]); 0.64 on 8 GPUs ([5,5,4,4,4,4,4,0])
    e4 = ps.efficiency([9, 9, 9, 3], 16, ps.gpipe_programs([9, 9, 9, 3], 16))
    c8 = [5, 5, 4, 4, 4, 4, 4, 0]
    e8 = ps.efficiency(c8, 16, ps.gpipe_programs(c8, 16))
    assert 0.78 <= e4 <= 0.90 and 0.55 <= e8 <= 0.68
    # a link that buffers does not change this schedule's makespan: its sends never wait long
    assert abs(ps.efficiency(c8, 16, ps.gpipe_programs(c8, 16), "buffered") - e8) < 1e-9


def test_one_forward_one_backward_needs_buffered_links():
    counts = finetune.partition_layers(30, 4)
    progs = ps.one_f_one_b_programs(counts, 16)
    assert ps.simulate(progs, "rendezvous")[0] is False      # two neighbours each waiting to send to the other
    assert ps.simulate(progs, "buffered")[0] is True


def test_greedy_estimates():
    # without deferring anything the greedy order is no better than the Trainer's schedule ...
    whole = ps.greedy_estimate([5, 5, 4, 4, 4, 4, 4], 16)
    c8 = [5, 5, 4, 4, 4, 4, 4, 0]
    assert abs(whole - ps.efficiency(c8, 16, ps.gpipe_programs(c8, 16))) < 0.02
    # ... deferring the weight gradients into the idle time and sharing the head between two ranks is what closes the gap
    split = ps.greedy_estimate([5, 5, 4, 4, 4, 4, 4], 16, split_backward=True)
    shared = ps.greedy_estimate([5, 5, 5, 4, 4, 4], 16, tail_layers=3, tail_replicas=2, split_backward=True)
    assert whole < split < shared and shared >= 0.85
    assert ps.greedy_estimate([9, 9, 9], 16, tail_layers=3, split_backward=True) >= 0.93


def test_static_schedule_replays_to_the_same_makespan():
    kw = dict(layer_counts=[5, 5, 5, 4, 4, 4], n_micro=16, tail_layers=3, tail_replicas=2, split_backward=True)
    eff, order = ps.greedy_estimate(return_order=True, **kw)
    assert sum(len(o) for o in order) == 3 * 7 * 16                      # every task of every stage and micro-batch, once
    ok, eff2, keep = ps.replay(order, **kw)
    assert ok and abs(eff - eff2) < 1e-9
    assert max(keep["activations"]) <= 16 and max(keep["deferred"]) <= 16
    # a schedule with a task before its producer does not finish
    bad = [list(o) for o in order]
    i = next(j for j, t in enumerate(bad[0]) if t[0] == "B")
    bad[0][0], bad[0][i] = bad[0][i], bad[0][0]
    assert ps.replay(bad, **kw)[0] is False
