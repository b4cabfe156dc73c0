"""Multi-rank path: host logic under gloo on CPU (world size 2 and 3), and -- when at least two GPUs
are visible -- the real NCCL pipeline against a single-GPU run of the same model."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "pipeline_worker.py")


def launch(world, backend, out_path, port, head_cost=0.5, overlap=True, replicas=1, async_opt=False, early_exchange=False):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), WORKER, backend, out_path]
    env = dict(os.environ, OMP_NUM_THREADS="2", BR_TEST_HEAD_COST=str(head_cost), BR_TEST_OVERLAP="1" if overlap else "0",
               BR_TEST_REPLICAS=str(replicas), BR_TEST_ASYNC_OPT="1" if async_opt else "0",
               BR_TEST_EARLY_EXCHANGE="1" if early_exchange else "0")
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.load(open(out_path))


@pytest.mark.parametrize("world,head_cost", [(2, 0.5), (3, 0.5), (3, 2.5)])
def test_stage_logic_on_cpu_ranks(tmp_path, world, head_cost):
    res = launch(world, "gloo", str(tmp_path / "out.json"), 29510 + world + int(head_cost), head_cost)
    assert res["ok"] and sum(res["counts"]) == 4 and len(res["counts"]) == world
    assert (res["counts"][-1] == 0) == (head_cost > 2)


def test_partition_balances_head():
    from blackriver_b200.finetune import partition_layers
    expect = {1: [30], 2: [17, 13], 4: [9, 9, 8, 4], 8: [5, 5, 4, 4, 4, 4, 4, 0]}
    for world in (1, 2, 4, 8):
        c = partition_layers(30, world)
        assert c == expect[world]
        assert sum(c) == 30 and min(c[:-1] or [1]) >= 1 and c[-1] >= 0
    assert partition_layers(4, 3, 2.5) == [2, 2, 0]        # a head heavier than a stage's share stands alone
    assert partition_layers(4, 2, 0.5) == [2, 2] and partition_layers(4, 3, 0.5)[-1] >= 1


def check_against_single(res):
    for a, b in zip(res["pipe_losses"], res["ref_losses"]):
        assert abs(a - b) <= 1e-3 * abs(b)
    # two Adam steps of size lr = 1e-3: a weight whose tiny gradient rounds differently in fp16 may move the
    # other way, so the bound is a few update steps relative to the largest weight
    assert res["w_err"] <= 1e-2 and res["table_err"] <= 1e-2
    assert res["tables_agree"]          # both holders of the tied table applied the same summed gradient
    if res["replicas"] == 1:
        # the forward-only scoring pass over the same stages (initial weights): per-token NLL and its mean
        assert res["scored"] == 2 and res["score_err"] <= 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("overlap", [True, False])
def test_two_stage_pipeline_matches_single_gpu(tmp_path, overlap):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = launch(2, "nccl", str(tmp_path / "out.json"), 29531 + int(overlap), overlap=overlap)
    assert res["overlap"] == overlap
    check_against_single(res)


@pytest.mark.gpu
@pytest.mark.parametrize("overlap", [True, False])
def test_pipeline_with_head_only_last_stage(tmp_path, overlap):
    import torch
    if torch.cuda.device_count() < 3:
        pytest.skip("needs three GPUs")
    res = launch(3, "nccl", str(tmp_path / "out.json"), 29535 + int(overlap), head_cost=2.5, overlap=overlap)
    assert res["counts"] == [2, 2, 0] and res["overlap"] == overlap
    check_against_single(res)


def test_replica_layout_and_shares():
    from blackriver_b200.finetune import replica_layout, replica_share
    # 8 ranks as 2 replicas of 4 stages: stages of one pipeline are neighbouring ranks
    assert [replica_layout(r, 8, 2, 16)[:2] for r in range(8)] == [(0, 0), (0, 1), (0, 2), (0, 3), (1, 0), (1, 1), (1, 2), (1, 3)]
    assert replica_layout(5, 8, 2, 16) == (1, 1, 4, 8) and replica_layout(3, 4, 4, 16) == (3, 0, 1, 4)
    with pytest.raises(ValueError):
        replica_layout(0, 6, 4, 16)
    with pytest.raises(ValueError):
        replica_layout(0, 4, 2, 5)
    mbs = list(range(16))
    shares = [replica_share(mbs, r, 4) for r in range(4)]
    assert sorted(sum(shares, [])) == mbs and all(len(x) == 4 for x in shares) and shares[1] == [1, 5, 9, 13]


@pytest.mark.gpu
def test_two_stage_pipeline_with_the_optimizer_on_the_transfer_stream(tmp_path):
    """Adam and the tied-table exchange queued on the transfer stream beside the next step's first forward."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = launch(2, "nccl", str(tmp_path / "out.json"), 29545, async_opt=True)
    assert res["overlap"]
    check_against_single(res)


@pytest.mark.gpu
def test_two_stage_pipeline_with_the_early_table_exchange(tmp_path):
    """The last rank takes the LM-head weight gradients first and starts the exchange of the tied table's gradient from
    its task list, before the layers' weight gradients."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = launch(2, "nccl", str(tmp_path / "out.json"), 29547, early_exchange=True)
    assert res["overlap"] and res["early_exchange"]
    check_against_single(res)


@pytest.mark.gpu
def test_two_replicas_match_single_gpu(tmp_path):
    """Two data-parallel replicas of the whole model (2 GPUs): each takes half of the micro-batches, gradients are summed
    by io.nccl.allreduce; losses and weights must match the single-GPU step over all micro-batches."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = launch(2, "nccl", str(tmp_path / "out.json"), 29541, replicas=2)
    assert res["replicas"] == 2 and res["replicas_agree"] and res["counts"] == [4.0]
    check_against_single(res)


@pytest.mark.gpu
def test_two_replicas_of_a_two_stage_pipeline(tmp_path):
    import torch
    if torch.cuda.device_count() < 4:
        pytest.skip("needs four GPUs")
    res = launch(4, "nccl", str(tmp_path / "out.json"), 29543, replicas=2)
    assert res["replicas"] == 2 and res["replicas_agree"] and len(res["counts"]) == 2 and res["overlap"]
    check_against_single(res)
