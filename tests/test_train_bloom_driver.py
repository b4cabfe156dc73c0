"""The compiled driver (blackriver_b200/lib/train_bloom) over a generated stage script."""
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
EXE = os.path.join(ROOT, "blackriver_b200", "lib", "train_bloom")
CFG = dict(hidden=128, heads=2, vocab=512, n_layers=3, batch=2, tokens=64, n_micro=3)


def emit(tmp_path, rank=0, world=1):
    from blackriver_b200 import emit_stage
    text, mine = emit_stage.stage_script(CFG["hidden"], CFG["heads"], CFG["vocab"], CFG["n_layers"], CFG["batch"], CFG["tokens"],
                                         CFG["n_micro"], rank, world, seed=9, init_std=0.05)
    path = str(tmp_path / f"stage{rank}.words")
    open(path, "w").write(text)
    return path, mine


def test_usage_and_emit(tmp_path):
    r = subprocess.run([EXE, "--help"], capture_output=True, text=True)
    assert r.returncode == 2 and "usage: train_bloom" in r.stderr
    from blackriver_b200 import emit_stage, host
    out = str(tmp_path / "s.words")
    assert emit_stage.main(["--out", out, "--hidden", "128", "--heads", "2", "--vocab", "512", "--layers", "3", "--batch", "2",
                            "--tokens", "64", "--micro", "3", "--rank", "1", "--world", "2", "--head-cost", "0.5"]) == 0
    env = host.Env(4)
    env.execute(open(out).read())                      # the emitted stage compiles in the words machine
    prog = env.build("slot_2 stage_forward slot_2 stage_backward")
    env.free_program(prog)
    env.close()


def test_fails_loudly_without_a_gpu(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    path, mine = emit(tmp_path)
    r = subprocess.run([EXE, "--script", path, "--layers", str(mine), "--batch", "2", "--tokens", "64", "--vocab", "512"],
                       capture_output=True, text=True, env=dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK="0"))
    assert r.returncode == 1 and "train_bloom rank 0" in r.stderr      # no CPU path: the driver stops with the CUDA error


@pytest.mark.gpu
def test_driver_matches_trainer(tmp_path):
    """Same stage script, same seeds, same token ids: the compiled driver and the Python Trainer run the same words
    in the same order, so their losses agree to the last printed digit."""
    from blackriver_b200 import finetune
    from blackriver_b200 import host
    mbs = finetune.make_microbatches(CFG["n_micro"], CFG["batch"], CFG["tokens"], CFG["vocab"], 20, seed=5)
    prefix = str(tmp_path / "data")
    np.stack([m[0] for m in mbs]).astype(np.int32).tofile(prefix + ".ids.bin")
    np.stack([m[1] for m in mbs]).astype(np.int32).tofile(prefix + ".mask.bin")
    np.stack([m[2] for m in mbs]).astype(np.int32).tofile(prefix + ".lens.bin")
    path, mine = emit(tmp_path)
    r = subprocess.run([EXE, "--script", path, "--layers", str(mine), "--batch", str(CFG["batch"]), "--tokens", str(CFG["tokens"]),
                        "--micro", str(CFG["n_micro"]), "--vocab", str(CFG["vocab"]), "--steps", "2", "--lr", "0.001",
                        "--data", prefix],
                       capture_output=True, text=True, timeout=300, env=dict(os.environ, RANK="0", WORLD_SIZE="1", LOCAL_RANK="0"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    got = [float(x) for x in re.findall(r"loss ([0-9.]+)", r.stdout)]
    assert len(got) == 2

    try:
        host.context_boot(0, None, 256 << 20)
        host.collective_boot_local(0, 1)
        owned = True
    except host.HostError:
        owned = False          # another test module of this process booted it already
    tr = finetune.Trainer(CFG["hidden"], CFG["heads"], CFG["vocab"], CFG["n_layers"], CFG["batch"], CFG["tokens"], CFG["n_micro"],
                          rank=0, world=1, seed=9, lr=1e-3, init_std=0.05)
    want = [tr.step(mbs) for _ in range(2)]
    tr.sync()
    tr.close()
    if owned:
        host.context_shutdown()
    for a, b in zip(got, want):
        assert abs(a - b) <= 2e-6 * abs(b) + 1e-6
    assert want[1] < want[0]      # and it trains
