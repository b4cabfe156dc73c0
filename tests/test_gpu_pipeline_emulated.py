"""The overlapped pipeline on ONE GPU: the stages of a 2-, 3- and 4-rank pipeline live in one process, each with its
own words machine and stage script, and exchange activations and gradients through the one-sided links in loop-back
mode (the process keeps one link block per played rank, chained like real neighbours).  The test queues every rank's task list
interleaved in an order that respects the dependencies (what the ranks' GPUs would do concurrently), so the split
input-gradient / weight-gradient passes, the per-slot kept gradients, the link windows, arrival and release counters
and the static schedule are all exercised without a second GPU.  Losses and updated weights must equal those of the
same model trained as one stage, within the fp16 tolerances of the multi-GPU test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = dict(hidden=128, heads=2, vocab=512, n_layers=4, batch=2, tokens=64)


@pytest.fixture(scope="module")
def host():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from blackriver_b200 import host as _host
    try:
        _host.context_boot(0, None, 256 << 20)
        _host.collective_boot_local(0, 1)
        owned = True
    except _host.HostError:
        owned = False
    yield _host
    if owned:
        _host.context_shutdown()


def global_order(orders, n_micro, n_slots):
    """A sequential interleaving of the ranks' lists in which every task comes after its dependencies."""
    from blackriver_b200 import schedule as S
    world = len(orders)
    pos = [0] * world
    done = set()
    out = []
    while any(pos[r] < len(orders[r]) for r in range(world)):
        moved = False
        for r in range(world):
            if pos[r] < len(orders[r]):
                t = orders[r][pos[r]]
                if all(d in done for d in S._deps(world, n_slots, r, t)):
                    done.add((r, t))
                    out.append((r, pos[r]))
                    pos[r] += 1
                    moved = True
        assert moved
    return out


def train_single(host, mbs, n_micro, steps):
    from blackriver_b200 import finetune
    tr = finetune.Trainer(CFG["hidden"], CFG["heads"], CFG["vocab"], CFG["n_layers"], CFG["batch"], CFG["tokens"], n_micro,
                          rank=0, world=1, seed=9, lr=1e-3, init_std=0.05)
    losses = [tr.step(mbs) for _ in range(steps)]
    tr.sync()
    tr.env.change(1); w = tr.env.read("_flat.master").copy()
    tr.env.change(0); table = tr.env.read("word_embeddings.weight.master").copy()
    tr.close()
    return losses, w, table


@pytest.mark.parametrize("world,head_cost,n_micro,n_slots,split,async_opt",
                         [(2, 0.5, 4, 4, True, False), (3, 2.5, 6, 3, True, False), (4, 0.5, 5, 2, True, False),
                          (3, 0.2, 4, 4, True, False), (2, 0.5, 4, 2, False, False), (3, 2.5, 6, 3, True, True), (4, 0.5, 5, 2, True, True)])
def test_emulated_ranks_match_single_stage(host, world, head_cost, n_micro, n_slots, split, async_opt):
    from blackriver_b200 import finetune
    mbs = finetune.make_microbatches(n_micro, CFG["batch"], CFG["tokens"], CFG["vocab"], 20, seed=5)
    ref_losses, ref_w, ref_table = train_single(host, mbs, n_micro, steps=2)

    trs = [finetune.Trainer(CFG["hidden"], CFG["heads"], CFG["vocab"], CFG["n_layers"], CFG["batch"], CFG["tokens"], n_micro,
                            rank=r, world=world, seed=9, lr=1e-3, init_std=0.05, head_cost=head_cost, n_slots=n_slots,
                            play_all_ranks=True, split_layers=split, async_optimizer=async_opt)
           for r in range(world)]
    try:
        assert all(t.overlap and t.n_slots == n_slots for t in trs)
        if head_cost > 2:
            assert trs[0].counts[-1] == 0            # a head-only last stage
        if not split:
            assert all(c == int(c) for c in trs[0].counts)
        if world == 3 and head_cost < 0.3:
            assert any(c != int(c) for c in trs[0].counts)      # 4 layers over 3 ranks: some layer is shared by two ranks
        from blackriver_b200 import schedule as S
        orders, _ = S.build(world, n_micro, trs[0].stage_costs, n_slots)
        assert [list(o) for o in orders] == [list(t.order) for t in trs]      # every rank derives the same lists
        seq = global_order([t.order for t in trs], n_micro, n_slots)
        losses = []
        for _ in range(2):
            for t in trs:
                t.begin_step(mbs)
            for r, i in seq:
                trs[r].run_task(i)
            for t in trs:
                t.check_and_read_losses()
            # the two holders of the tied table sum their gradients (NCCL in a real job)
            e0, e1 = trs[0].env, trs[-1].env
            e0.change(0); e1.change(0)
            g = e0.read("word_embeddings.weight_g").astype(np.float32) + e1.read("word_embeddings.weight_g").astype(np.float32)
            e0.write("word_embeddings.weight_g", g); e1.write("word_embeddings.weight_g", g)
            out = [t.apply_optimizer() for t in trs]
            losses.append(out[-1])
        for t in trs:
            t.sync()
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) <= 1e-3 * abs(b)
        trs[0].env.change(1); w = trs[0].env.read("_flat.master")
        trs[0].env.change(0); table0 = trs[0].env.read("word_embeddings.weight.master")
        trs[-1].env.change(0); table1 = trs[-1].env.read("word_embeddings.weight.master")
        # two Adam steps of size lr = 1e-3: a weight whose tiny gradient rounds differently in fp16 may move the other
        # way, so the bound is a few update steps relative to the largest weight
        assert np.abs(w - ref_w).max() / np.abs(ref_w).max() <= 1e-2
        assert np.abs(table0 - ref_table).max() / np.abs(ref_table).max() <= 1e-2
        assert np.array_equal(table0, table1)
    finally:
        for t in trs:
            t.close()


def test_link_counters_and_windows(host):
    """Loop-back links through the words: a tensor sent to the 'next rank' appears in this rank's side-0 window after
    io.link.wait, twice in a row on the same slot (the second send has to see the release of the first)."""
    env = host.Env(1)
    try:
        env.execute('4096 2 io.link.open')
        env.execute('0 1 8 128 2 "half" io.link.window "win" !  8 128 2 "cuda" "half" op.create "src" !')
        for value in (1.5, -2.25):
            env.execute(f'"src" @ {value} op.fill  "src" @ 1 1 io.link.send  0 1 io.link.wait  1 io.link.fence')
            env.execute('8 128 2 "cuda" "half" op.create "copy" !  "copy" @ "win" @ op.copy  0 1 io.link.release  op.sync')
            assert np.all(env.read("copy") == np.float16(value))
        env.execute("io.link.close")
    finally:
        env.close()
