"""Writes the words script of one pipeline stage and prints the train_bloom command that runs it.

    python -m blackriver_b200.emit_stage --rank 0 --world 1 --out stage0.words \\
        --hidden 4096 --heads 32 --vocab 250880 --layers 30 --batch 2 --tokens 1024 --micro 16

One script per rank (the stage's layer block, its neighbours and its share of embedding / head are
fixed in the script); the compiled driver blackriver_b200/lib/train_bloom executes it."""
import argparse
import os
import sys

from . import finetune, words


def stage_script(hidden, heads, vocab, n_layers, batch, tokens, n_micro, rank, world, dtype="half", seed=0, init_std=0.02,
                 logits_rows=None, head_cost=finetune.LM_HEAD_COST_IN_LAYERS):
    """(script text, layers of this stage) for rank `rank` of `world` contiguous stages."""
    counts = finetune.partition_layers(n_layers, world, head_cost)
    first, last = rank == 0, rank == world - 1
    text = words.fused_words(
        hidden=hidden, heads=heads, vocab=vocab, n_layers=counts[rank], batch=batch, tokens=tokens, dtype=dtype,
        first_stage=first, last_stage=last, logits_rows=logits_rows, init_std=init_std, seed=seed,
        layer_offset=sum(counts[:rank]), n_slots=n_micro if world > 1 else 1, n_micro=n_micro,
        prev_rank=None if first else rank - 1, next_rank=None if last else rank + 1)
    return text, counts[rank]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", required=True)
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--vocab", type=int, default=250880)
    ap.add_argument("--layers", type=int, default=30, help="decoder layers of the whole model")
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--micro", type=int, default=16)
    ap.add_argument("--dtype", default="half", choices=["half", "float"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--init-std", type=float, default=0.02)
    ap.add_argument("--head-cost", type=float, default=finetune.LM_HEAD_COST_IN_LAYERS)
    a = ap.parse_args(argv)
    text, mine = stage_script(a.hidden, a.heads, a.vocab, a.layers, a.batch, a.tokens, a.micro, a.rank, a.world, a.dtype,
                              a.seed, a.init_std, a.batch * a.tokens, a.head_cost)
    with open(a.out, "w") as f:
        f.write(text)
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "train_bloom")
    print(f"RANK={a.rank} WORLD_SIZE={a.world} LOCAL_RANK={a.rank} {exe} --script {a.out} --layers {mine} "
          f"--batch {a.batch} --tokens {a.tokens} --micro {a.micro} --vocab {a.vocab}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
