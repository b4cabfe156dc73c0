"""Worker for the pipeline tests: run under torchrun with WORLD_SIZE ranks.

backend nccl (GPU): trains a small model for two steps as a WORLD_SIZE-stage pipeline (overlapped schedule with
one-sided hand-offs, or -- BR_TEST_OVERLAP=0 -- the plain order over NCCL send / receive), then rank 0 trains the same
model on one GPU and compares losses and updated weights.
With BR_TEST_REPLICAS = R the ranks form R data-parallel replicas of a WORLD_SIZE / R-stage pipeline.
backend gloo (CPU): checks the host-side logic only -- stage partition, identical micro-batches and identical task
lists on every rank, stage scripts of both kinds compile in the words machine."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from blackriver_b200 import finetune, host, words  # noqa: E402

CFG = dict(hidden=128, heads=2, vocab=512, n_layers=4, batch=2, tokens=64, n_micro=4)


def main():
    backend = sys.argv[1]
    out_path = sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    mbs = finetune.make_microbatches(CFG["n_micro"], CFG["batch"], CFG["tokens"], CFG["vocab"], 20, seed=5)
    head_cost = float(os.environ.get("BR_TEST_HEAD_COST", "0.5"))
    counts = finetune.partition_layers(CFG["n_layers"], world, head_cost=head_cost)
    if backend == "gloo":
        dist.init_process_group("gloo")
        gathered = [None] * world
        digest = [int(np.sum([m[0].astype(np.int64).sum() for m in mbs])), counts]
        dist.all_gather_object(gathered, digest)
        assert all(g == gathered[0] for g in gathered), "ranks disagree on inputs or partition"
        assert sum(counts) == CFG["n_layers"] and all(c >= 1 for c in counts[:-1]) and counts[-1] >= 0
        first, last = rank == 0, rank == world - 1
        from blackriver_b200 import schedule
        costs = schedule.stage_costs(counts)
        orders, _ = schedule.build(world, CFG["n_micro"], costs, CFG["n_micro"])
        schedule.check(orders, CFG["n_micro"], CFG["n_micro"])
        lists = [None] * world
        dist.all_gather_object(lists, [[(t.kind, t.k) for t in o] for o in orders])
        assert all(x == lists[0] for x in lists), "ranks disagree on the task lists"
        for overlap in (False, True):
            env = host.Env(counts[rank] + 1)
            env.execute(words.fused_words(hidden=CFG["hidden"], heads=CFG["heads"], vocab=CFG["vocab"], n_layers=counts[rank],
                                          batch=CFG["batch"], tokens=CFG["tokens"], first_stage=first, last_stage=last,
                                          n_slots=CFG["n_micro"], n_micro=CFG["n_micro"], prev_rank=None if first else rank - 1,
                                          next_rank=None if last else rank + 1, layer_offset=sum(counts[:rank]), overlap=overlap,
                                          async_optimizer=True))
            text = ('slot_1 stage_f slot_1 "loss@1" stage_b slot_1 stage_w' if overlap else
                    'slot_1 stage_forward slot_1 stage_backward slot_1 "loss@1" stage_backward_async')
            prog = env.build(text + " sync_replicas 1e-3 1 1.0 optimizer_async 0 1e-3 1 1.0 optimizer_async_tied")     # links every word of the stage
            env.free_program(prog)
            env.close()
        dist.barrier()
        if rank == 0:
            json.dump({"ok": True, "counts": counts}, open(out_path, "w"))
        dist.destroy_process_group()
        return

    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    host.context_boot(local, torch.cuda.current_stream().cuda_stream, 128 << 20)
    box = [host.collective_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    host.collective_boot(rank, world, box[0])
    replicas = int(os.environ.get("BR_TEST_REPLICAS", "1"))
    host.collective_split(replicas)
    stages = world // replicas
    tr = finetune.Trainer(CFG["hidden"], CFG["heads"], CFG["vocab"], CFG["n_layers"], CFG["batch"], CFG["tokens"], CFG["n_micro"],
                          rank=rank, world=world, seed=9, lr=1e-3, init_std=0.05, head_cost=head_cost,
                          overlap=os.environ.get("BR_TEST_OVERLAP", "1") != "0", replicas=replicas,
                          async_optimizer=os.environ.get("BR_TEST_ASYNC_OPT", "0") == "1",
                          early_exchange=os.environ.get("BR_TEST_EARLY_EXCHANGE", "0") == "1")
    # forward-only scoring through the same stages (the prefill path) with the initial weights: per-token NLL from the
    # rank that holds the head
    scored = tr.score(mbs[:2]) if replicas == 1 else []
    tr.sync()
    losses = [tr.step(mbs) for _ in range(2)]
    tr.sync()
    w_first = None
    if tr.counts[tr.rank] >= 1:
        tr.env.change(1)
        w_first = tr.env.read("_flat.master").copy()          # first layer of this stage
    tr.env.change(0)
    table = tr.env.read("word_embeddings.weight.master").copy() if (tr.first or tr.last) else None
    box = [[(nll.tolist(), mean) for nll, mean in scored]]
    dist.broadcast_object_list(box, src=stages - 1)
    pipe_scores = box[0]
    box = [losses]
    dist.broadcast_object_list(box, src=stages - 1)           # the head's rank of the first replica
    pipe_losses = box[0]
    tables = [None] * world
    dist.all_gather_object(tables, None if table is None else float(np.abs(table).sum()))
    # the replicas of a stage must hold the same weights bit for bit: they applied the same summed gradient
    digests = [None] * world
    dist.all_gather_object(digests, None if w_first is None else float(np.abs(w_first.astype(np.float64)).sum()))
    replicas_agree = all(digests[r] == digests[r % stages] for r in range(world))
    tables = tables[:stages]
    tr.close()
    if rank == 0:
        single = finetune.Trainer(CFG["hidden"], CFG["heads"], CFG["vocab"], CFG["n_layers"], CFG["batch"], CFG["tokens"],
                                  CFG["n_micro"], rank=0, world=1, seed=9, lr=1e-3, init_std=0.05)
        ref_scores = single.score(mbs[:2])
        ref_losses = [single.step(mbs) for _ in range(2)]
        single.sync()
        score_err = 0.0
        for (nll, mean), (rn, rm) in zip(pipe_scores, ref_scores):
            score_err = max(score_err, float(np.abs(np.asarray(nll, np.float32) - rn).max()), abs(mean - rm))
        single.env.change(1)
        ref_w = single.env.read("_flat.master").copy()
        single.env.change(0)
        ref_table = single.env.read("word_embeddings.weight.master").copy()
        single.close()
        res = {
            "pipe_losses": pipe_losses, "ref_losses": ref_losses,
            "w_err": float(np.abs(w_first - ref_w).max() / np.abs(ref_w).max()),
            "table_err": float(np.abs(table - ref_table).max() / np.abs(ref_table).max()),
            "tables_agree": abs(tables[0] - tables[-1]) <= 1e-6 * abs(tables[0]),
            "scored": len(pipe_scores), "score_err": score_err, "early_exchange": os.environ.get("BR_TEST_EARLY_EXCHANGE", "0") == "1",
            "counts": tr.counts, "overlap": tr.overlap, "n_slots": tr.n_slots, "replicas": replicas, "replicas_agree": replicas_agree,
        }
        json.dump(res, open(out_path, "w"))
    dist.barrier()
    host.collective_shutdown()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
