#!/usr/bin/env python
"""Benchmark of the B200-native BLOOM decoder hot path.

Default workload (`--workload finetune`): one BLOOM-7b1-architecture fine-tune step with random
initialisation -- 30 layers, hidden 4096, 32 heads x 128, MLP 16384, vocabulary 250880 with tied
embedding, embedding LayerNorm, ALiBi; fp16 weights/activations, fp32 master weights and Adam;
16 micro-batches of batch 2 x seq 1024 (32768 tokens per step) with right padding, valid lengths
uniform in [512, 1024], seed 3; gradient accumulation over the micro-batches, then one optimizer
step.  It runs through the reference-facing interface: the generated words scripts executed by the
words machine on device tensors.  With N > 1 GPUs (torchrun) the 30 layers are split into N
contiguous pipeline stages (embedding on the first rank, final LayerNorm + LM head + loss on the
last) and the same 16 micro-batches flow through NCCL send/recv, so total work is fixed
("scaling": "strong").  `value` is tokens/s; `e2e` times the same step including the host->device
copy of every micro-batch's ids/mask/lengths and the device->host read of every loss (both are
part of the step as the interface defines it).  `roofline` describes the dominant kernel of the
step, the tcgen05 GEMM: FLOPs of all GEMM launches of one step / their summed CUDA-event time /
measured bf16 tensor peak.  `kernels` adds the HBM-bound operator microbench (`--workload ops`:
fp16, 8192 tokens, LayerNorm / GELU / log-softmax+NLL) in GB/s against the measured HBM peak.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload finetune|ops|c3|prefill]
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOKENS = 8192
HIDDEN = 4096
HIDDEN4 = 16384
VOCAB = 250880
MASK_FRAC = 0.1
SEED = 1
WORKLOAD = ("operator microbench, fp16 storage / fp32 accumulate, 8192 tokens: LayerNorm fwd+bwd [8192,4096]; "
            "bloom-GELU fwd+bwd [8192,4096] and [8192,16384]; log-softmax+NLL fwd+gradient [8192,250880], "
            "10% rows ignored; seed 1")


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ts, line in self.samples:
            if ts < t0 or ts > t1 + 0.1:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def make_host_inputs(torch, rank, dev):
    """Seeded synthetic inputs of the microbench shapes, kept in pinned host memory (the caller's
    copy).  The random draws are made by the device generator and copied out once, because
    drawing two billion normals on the host takes minutes; the timed regions never draw."""
    g = torch.Generator(device=dev).manual_seed(SEED + 1000 * rank)

    def pinned(t):
        out = torch.empty(t.shape, dtype=t.dtype).pin_memory()
        out.copy_(t)
        return out
    h = {}
    for s in range(2):
        h[f"x{s}"] = pinned(torch.randn(TOKENS, HIDDEN, generator=g, device=dev).half())
        h[f"dy{s}"] = pinned(torch.randn(TOKENS, HIDDEN, generator=g, device=dev).half())
        h[f"x4_{s}"] = pinned(torch.randn(TOKENS, HIDDEN4, generator=g, device=dev).half())
        h[f"dy4_{s}"] = pinned(torch.randn(TOKENS, HIDDEN4, generator=g, device=dev).half())
    h["gamma"] = pinned((1.0 + 0.1 * torch.randn(HIDDEN, generator=g, device=dev)).half())
    h["beta"] = pinned((0.1 * torch.randn(HIDDEN, generator=g, device=dev)).half())
    logits = torch.empty((TOKENS, VOCAB), dtype=torch.float16).pin_memory()
    for r0 in range(0, TOKENS, 1024):   # logits ~ N(0, sigma=2), drawn in row chunks
        logits[r0:r0 + 1024].copy_((torch.randn(1024, VOCAB, generator=g, device=dev) * 2.0).half())
    h["logits"] = logits
    target = torch.randint(0, VOCAB, (TOKENS,), generator=g, device=dev, dtype=torch.int32)
    target[torch.rand(TOKENS, generator=g, device=dev) < MASK_FRAC] = -100
    h["target"] = pinned(target)
    torch.cuda.synchronize()
    return h


def run_ops(args, emit=True):
    import torch
    import torch.distributed as dist
    from blackriver_b200 import ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    peak, peak_kind = load_peaks()

    host = make_host_inputs(torch, rank, dev)
    d = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
    torch.cuda.synchronize()
    n_valid = int((host["target"] >= 0).sum())
    grad_scale = 1.0 / max(n_valid, 1)

    # outputs / scratch, allocated once (the C ABI itself never allocates)
    o = {}
    for s in range(2):
        o[f"y{s}"] = torch.empty_like(d[f"x{s}"])
        o[f"dx{s}"] = torch.empty_like(d[f"x{s}"])
        o[f"g{s}"] = torch.empty_like(d[f"x{s}"])
        o[f"dg{s}"] = torch.empty_like(d[f"x{s}"])
        o[f"g4_{s}"] = torch.empty_like(d[f"x4_{s}"])
        o[f"dg4_{s}"] = torch.empty_like(d[f"x4_{s}"])
        o[f"var{s}"] = torch.empty(TOKENS, dtype=torch.float32, device=dev)
    o["dgamma"] = torch.empty_like(d["gamma"])
    o["dbeta"] = torch.empty_like(d["beta"])
    o["dlogits"] = torch.empty_like(d["logits"])
    o["row_loss"] = torch.empty(TOKENS, dtype=torch.float32, device=dev)
    o["loss"] = torch.empty(1, dtype=torch.float32, device=dev)
    from blackriver_b200 import brk
    ws_bytes = brk.lib().brk_layernorm_bwd_workspace_bytes(TOKENS, HIDDEN)
    o["ws"] = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
    rows_host = torch.empty(TOKENS, dtype=torch.float32).pin_memory()

    # fill both LayerNorm sets once so that backward has a valid (y, var) of the other set
    for s in range(2):
        _, _, var = ops.layernorm(d[f"x{s}"], d["gamma"], d["beta"], 1e-5, out=o[f"y{s}"])
        o[f"var{s}"].copy_(var)
    torch.cuda.synchronize()

    KERNELS = ("ln_fwd", "gelu16k_fwd", "ln_bwd", "gelu16k_bwd", "gelu4k_fwd", "gelu4k_bwd", "nll_fwd_bwd")
    LAUNCHES_PER_STEP = 1 + 1 + 2 + 1 + 1 + 1 + 1 + 1  # ln_bwd is two launches; + the loss sum

    # one launcher per kernel family; a / b = the buffer set read by forward / by backward ops
    def k_ln_fwd(a, b):
        brk.call("brk_layernorm_fwd", d[f"x{a}"].data_ptr(), d["gamma"].data_ptr(), d["beta"].data_ptr(),
                 o[f"y{a}"].data_ptr(), 0, o[f"var{a}"].data_ptr(), TOKENS, HIDDEN, 1e-5, brk.F16, ops.stream())

    def k_ln_bwd(a, b):
        ops.layernorm_backward(d[f"dy{b}"], d["gamma"], d["beta"], o[f"var{b}"], o[f"y{b}"], 1e-5, dgamma=o["dgamma"],
                               dbeta=o["dbeta"], dx=o[f"dx{b}"], workspace=o["ws"])

    launchers = {
        "ln_fwd": k_ln_fwd,
        "gelu16k_fwd": lambda a, b: ops.gelu(d[f"x4_{a}"], out=o[f"g4_{a}"]),
        "ln_bwd": k_ln_bwd,
        "gelu16k_bwd": lambda a, b: ops.gelu_backward(d[f"dy4_{b}"], d[f"x4_{b}"], out=o[f"dg4_{b}"]),
        "gelu4k_fwd": lambda a, b: ops.gelu(d[f"x{a}"], out=o[f"g{a}"]),
        "gelu4k_bwd": lambda a, b: ops.gelu_backward(d[f"dy{b}"], d[f"x{b}"], out=o[f"dg{b}"]),
        "nll_fwd_bwd": lambda a, b: ops.logsoftmax_nll_backward(d["logits"], d["target"], grad_scale, row_loss=o["row_loss"],
                                                                dlogits=o["dlogits"]),
    }

    def step(i, ev=None):
        a, b = i % 2, (i + 1) % 2   # set read by forward ops / by backward ops (last touched a step ago)
        if ev is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            ev.append(("start", e))
        for k in KERNELS:
            launchers[k](a, b)
            if ev is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                ev.append((k, e))
        ops.sum_f32(o["row_loss"], out=o["loss"])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    t_wall0 = time.time()
    ev = []
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(args.warmup + i, ev)
    e1.record()
    barrier()
    t_wall1 = time.time()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    loss_val = float(o["loss"].item()) * grad_scale

    per_kernel = {k: [] for k in KERNELS}
    for j in range(1, len(ev)):
        k, e = ev[j]
        if k != "start":
            per_kernel[k].append(ev[j - 1][1].elapsed_time(e))

    # ---- per kernel: runs of back-to-back launches of one kernel between two events ------------
    # (the intervals above also contain the event records between unlike kernels; here consecutive launches
    # alternate between the two buffer sets, 134 MB and more apart, so no launch finds its data in L2)
    batched = {}
    for k in KERNELS:
        reps = 6 if k == "nll_fwd_bwd" else 24
        for i in range(2):
            launchers[k](i % 2, (i + 1) % 2)
        b0 = torch.cuda.Event(enable_timing=True)
        b1 = torch.cuda.Event(enable_timing=True)
        b0.record()
        for i in range(reps):
            launchers[k](i % 2, (i + 1) % 2)
        b1.record()
        b1.synchronize()
        batched[k] = b0.elapsed_time(b1) / reps
    batched_launches = sum((6 if k == "nll_fwd_bwd" else 24) + 2 for k in KERNELS) + 26      # ln_bwd is two launches

    # ---- end to end: host buffers in, losses out, copies inside the timed region -------------
    h2d_keys = ["x0", "dy0", "x4_0", "dy4_0", "gamma", "beta", "logits", "target"]
    h2d_bytes = sum(host[k].numel() * host[k].element_size() for k in h2d_keys)
    d2h_bytes = loss_host.numel() * 4 + rows_host.numel() * 4

    def e2e_step(i):
        for k in h2d_keys:
            d[k].copy_(host[k], non_blocking=True)
        # one set only: the caller hands over one batch; LayerNorm backward consumes this step's y
        brk.call("brk_layernorm_fwd", d["x0"].data_ptr(), d["gamma"].data_ptr(), d["beta"].data_ptr(),
                 o["y0"].data_ptr(), 0, o["var0"].data_ptr(), TOKENS, HIDDEN, 1e-5, brk.F16, ops.stream())
        ops.gelu(d["x4_0"], out=o["g4_0"])
        ops.layernorm_backward(d["dy0"], d["gamma"], d["beta"], o["var0"], o["y0"], 1e-5, dgamma=o["dgamma"],
                               dbeta=o["dbeta"], dx=o["dx0"], workspace=o["ws"])
        ops.gelu_backward(d["dy4_0"], d["x4_0"], out=o["dg4_0"])
        ops.gelu(d["x0"], out=o["g0"])
        ops.gelu_backward(d["dy0"], d["x0"], out=o["dg0"])
        ops.logsoftmax_nll_backward(d["logits"], d["target"], grad_scale, row_loss=o["row_loss"], dlogits=o["dlogits"])
        ops.sum_f32(o["row_loss"], out=o["loss"])
        loss_host.copy_(o["loss"], non_blocking=True)
        rows_host.copy_(o["row_loss"], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step(0)
    barrier()
    f0 = torch.cuda.Event(enable_timing=True)
    f1 = torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)

    # ---- max over ranks --------------------------------------------------------------------------
    if world > 1:
        t = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e = float(t[0]), float(t[1])

    ms_per_step = ms_total / args.steps
    value = world * TOKENS / (ms_per_step * 1e-3)
    e2e_value = world * TOKENS / (ms_e2e / e2e_steps * 1e-3)

    out = None
    if rank == 0:
        es = 2
        masked = TOKENS - n_valid
        alg = {
            "ln_fwd": 2 * TOKENS * HIDDEN * es + 2 * HIDDEN * es + 4 * TOKENS,
            "ln_bwd": 3 * TOKENS * HIDDEN * es + 4 * TOKENS + 2 * HIDDEN * es * 2,
            "gelu4k_fwd": 2 * TOKENS * HIDDEN * es, "gelu4k_bwd": 3 * TOKENS * HIDDEN * es,
            "gelu16k_fwd": 2 * TOKENS * HIDDEN4 * es, "gelu16k_bwd": 3 * TOKENS * HIDDEN4 * es,
            # ignored rows are never read; their gradient row is written as zeros
            "nll_fwd_bwd": (2 * n_valid + masked) * VOCAB * es + 8 * TOKENS,
        }
        kern = {}
        for k in KERNELS:
            ms = batched[k]      # average launch duration over a run of launches of this kernel
            gbs = alg[k] / (ms * 1e-3) / 1e9
            kern[k] = {"ms": round(ms, 4), "ms_between_events_in_step": round(statistics.mean(per_kernel[k]), 4),
                       "algorithmic_bytes": alg[k], "gbs": round(gbs, 1), "frac_of_" + peak_kind + "_hbm": round(gbs / peak, 3)}
        dom = "nll_fwd_bwd"
        roofline = {"kernel": dom, "bound": "hbm", "achieved": kern[dom]["gbs"], "peak": peak, "unit": "GB/s",
                    "frac": round(kern[dom]["gbs"] / peak, 3), "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)"
                    if peak_kind == "measured" else "fallback 6650 GB/s", "traffic": load_traffic()}
        cpu = cpu_baseline()
        out = {
            "metric": "tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens_per_gpu": TOKENS,
                       "l2": "inputs larger than L2: two rotating LN/GELU buffer sets and an 8 GB logits sweep per step "
                             "separate every re-use"},
            "clocks": clocks, "gpu_launches": LAUNCHES_PER_STEP * args.steps,
            "gpu_launches_per_kernel_runs": batched_launches,
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps},
            "roofline": roofline, "kernels": kern, "cpu_baseline": cpu, "loss": round(loss_val, 5),
        }
        if emit:
            emit_line(out)
    if world > 1 and emit:
        dist.destroy_process_group()
    result = out if rank == 0 else None
    del d, o, host
    torch.cuda.empty_cache()
    return result



# ------------------------------------------------------------------------------------------
# fine-tune workload (the default)
# ------------------------------------------------------------------------------------------
FT = dict(hidden=4096, heads=32, vocab=VOCAB, n_layers=30, batch=2, tokens=1024, n_micro=16, min_len=512, seed=3)
FT_WORKLOAD = ("BLOOM-7b1-architecture fine-tune step, random init: 30 layers, hidden 4096, 32 heads x 128, MLP 16384, vocab 250880 "
               "tied, embedding LayerNorm, ALiBi; fp16 weights/activations, fp32 master weights + Adam; 16 micro-batches of "
               "batch 2 x seq 1024 (32768 tokens/step), right padding with lengths U[512,1024], seed 3; contiguous pipeline "
               "stages over the GPUs")


# The other single-step configurations of the same model: one micro-batch of batch 4 x seq 512 on one GPU, and the
# forward-only long-context prefill (8 sequences of 2048 tokens, no padding, per-token NLL), one sequence per micro-batch.
C3 = dict(hidden=4096, heads=32, vocab=VOCAB, n_layers=30, batch=4, tokens=512, n_micro=1, min_len=256, seed=2)
C3_WORKLOAD = ("BLOOM-7b1-architecture fine-tune step, random init, on one GPU: batch 4 x seq 512 (2048 tokens/step), right padding "
               "with lengths U[256,512], seed 2; fp16 weights/activations, fp32 master weights + Adam")
PREFILL = dict(hidden=4096, heads=32, vocab=VOCAB, n_layers=30, batch=1, tokens=2048, n_micro=8, min_len=2048, seed=4)
PREFILL_WORKLOAD = ("BLOOM-7b1-architecture forward-only long-context prefill, fp16: batch 8 x seq 2048 (16384 tokens/pass), no "
                    "padding, ALiBi causal, per-token NLL against the shifted inputs over the 250880-way head, seed 4; one "
                    "sequence per micro-batch through contiguous pipeline stages")


def load_tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured sustained (MEASURED_PEAKS.json bf16_tflops_sustained)"
    return 1400.0, "fallback 1.4 PFLOP/s sustained"


def run_finetune(args):
    import torch
    import torch.distributed as dist
    from blackriver_b200 import finetune, host

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    cfg = dict(C3 if args.workload == "c3" else FT)
    workload_text = C3_WORKLOAD if args.workload == "c3" else FT_WORKLOAD
    if args.layers:
        cfg["n_layers"] = args.layers
    if args.micro:
        cfg["n_micro"] = args.micro

    # the HBM-bound operator microbench first (its buffers are released before the model is built)
    ops_line = None
    if not args.skip_ops and world == 1 and args.workload == "finetune":
        ops_args = argparse.Namespace(steps=50, warmup=3)
        ops_line = run_ops(ops_args, emit=False)

    # the library computes on torch's current stream so that torch events bracket its work.  That has to be a stream of
    # its own: the legacy default stream has handle 0, which the library reads as "create your own stream", and events
    # on the default stream would not wait for that one.
    compute_stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(compute_stream)
    host.context_boot(local, compute_stream.cuda_stream, 512 << 20)
    if world > 1:
        box = [host.collective_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        host.collective_boot(rank, world, box[0])
        host.collective_split(args.replicas)
    else:
        host.collective_boot_local(0, 1)

    tr = finetune.Trainer(cfg["hidden"], cfg["heads"], cfg["vocab"], cfg["n_layers"], cfg["batch"], cfg["tokens"], cfg["n_micro"],
                          rank=rank, world=world, seed=cfg["seed"], logits_rows=cfg["batch"] * cfg["tokens"],
                          overlap=not args.no_overlap, replicas=args.replicas if world > 1 else 1,
                          async_optimizer=args.async_optimizer, early_exchange=args.early_exchange)
    mbs = finetune.make_microbatches(cfg["n_micro"], cfg["batch"], cfg["tokens"], cfg["vocab"], cfg["min_len"], cfg["seed"])
    tokens_per_step = cfg["n_micro"] * cfg["batch"] * cfg["tokens"]
    valid_per_step = int(sum(int(m[2].sum()) for m in mbs))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    loss = None
    for _ in range(args.warmup):
        loss = tr.step(mbs)
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    t0w = time.time()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    trace = []
    for _ in range(args.steps):
        loss = tr.step(mbs)
        trace.append(loss)
    tr.drain()          # the last optimizer step may still be running on the transfer stream: the end event waits for it
    e1.record()
    barrier()
    t1w = time.time()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop(t0w, t1w) if rank == 0 else None

    # ---- end to end: every micro-batch's ids / mask / lengths go host -> device and every loss comes
    # back device -> host inside the step; here the step result is also read after each step --------
    e2e_steps = max(1, min(args.steps, 3))
    barrier()
    f0 = torch.cuda.Event(enable_timing=True)
    f1 = torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(e2e_steps):
        loss = tr.step(mbs)
        tr.sync()
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)

    # ---- one instrumented step: device time per kernel family (CUDA events around every library call)
    host.profile_start()
    tr.step(mbs)
    prof = host.profile_stop()
    barrier()

    # ---- optional: when every task of one step ended on each rank's device (events behind the tasks), next to the
    # schedule simulation's plan for the same lists
    timeline = None
    if args.timeline:
        barrier()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(tr.tasks) + 2)]
        evs[0].record()
        tr.step(mbs, after_task=lambda i: evs[i + 1].record())
        tr.drain()
        evs[-1].record()
        torch.cuda.synchronize()
        names = [(t.kind, t.k) for t in tr.order] if tr.order else [("F" if i % 2 == 0 else "BW", i // 2) for i in range(len(tr.tasks))]
        mine = [[k, n, round(evs[0].elapsed_time(evs[i + 1]), 3)] for i, (k, n) in enumerate(names)]
        mine.append(["opt", -1, round(evs[0].elapsed_time(evs[-1]), 3)])
        timeline = [mine]
        if world > 1:
            gathered_tl = [None] * world
            dist.all_gather_object(gathered_tl, mine)
            timeline = gathered_tl
        barrier()

    # device time of every rank's kernels in the instrumented step (each interval carries ~3 us of event overhead): the
    # rank with the largest sum paces the pipeline, the gap to the step time is what it spent waiting
    busy = [round(sum(v["ms"] for v in prof.values()), 1)]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, busy[0])
        busy = gathered
        t = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e = float(t[0]), float(t[1])
        box = [loss, trace]
        dist.broadcast_object_list(box, src=tr.world - 1)        # the head's rank (of the first replica)
        loss, trace = box

    if tr.world == 1:
        schedule_name = "forward + backward per micro-batch"
    elif tr.overlap:
        schedule_name = ("static forward / input-gradient / weight-gradient task lists per rank (greedy, simulated efficiency %.2f), "
                         "one-sided hand-offs on transfer streams" % tr.simulated_efficiency)
    else:
        schedule_name = "all forwards then all backwards, NCCL send / receive on the compute stream"
    if rank == 0:
        ms_per_step = ms_total / args.steps
        value = tokens_per_step / (ms_per_step * 1e-3)
        e2e_value = tokens_per_step / (ms_e2e / e2e_steps * 1e-3)
        # every forward and input-gradient task copies its micro-batch's ids / mask / lengths host -> device; before the
        # optimizer the losses and the two kernel status words are read back
        h2d = sum(finetune.pack_inputs(mbs[k]).nbytes for _, k in tr.tasks if k is not None)
        d2h = cfg["n_micro"] * 4 + 8
        peak_tf, peak_src = load_tensor_peak()
        # rank 0's GEMM work in whole-layer equivalents (a stage may end between a layer's attention and MLP halves)
        flops = cfg["n_micro"] * finetune.gemm_flops_per_microbatch(cfg["hidden"], cfg["vocab"], tr.gemm_layers, cfg["batch"] * cfg["tokens"],
                                                                  with_head=(tr.world == 1)) // tr.replicas
        gemm_ms = prof.get("gemm_f16", {}).get("ms", 0.0)
        achieved = flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        fam = {k: {"ms": round(v["ms"], 3), "calls": v["calls"]} for k, v in sorted(prof.items(), key=lambda kv: -kv[1]["ms"])}
        launches = sum(v["calls"] for v in prof.values())
        out = {
            "metric": "tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 storage, f32 accumulate, f32 master weights",
            "data": "synthetic",
            "config": {"workload": workload_text, "layers": cfg["n_layers"], "micro_batches": cfg["n_micro"],
                       "tokens_per_step": tokens_per_step, "valid_tokens_per_step": valid_per_step,
                       "parallelism": ("pp%d" % world) if tr.replicas == 1 else ("dp%d x pp%d, gradients all-reduced over replicas" % (tr.replicas, tr.world)), "stage_layers": tr.counts, "schedule": schedule_name, "slots": tr.n_slots,
                       "l2": "inputs larger than L2: per step every kernel streams >= 14 GB of weights and activations between re-uses"},
            "clocks": clocks, "gpu_launches": launches * args.steps,
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps},
            "roofline": {"kernel": "gemm_tc_kernel (tcgen05/TMEM, all GEMM launches of rank 0's stage in one step)",
                         "bound": "tensor", "achieved": None if achieved is None else round(achieved, 1), "peak": peak_tf,
                         "unit": "TFLOP/s", "frac": None if achieved is None else round(achieved / peak_tf, 3),
                         "peak_source": peak_src, "traffic": None,
                         "traffic_note": "the family mixes shapes; the h->4h launch (2048 x 16384 x 4096) moves 152.5 MB read + "
                                         "47.8 MB written per launch in DRAM against 151.0 + 67.1 MB algorithmic "
                                         "(profiles/gemm_f16_pair_2048x16384x4096.md)",
                         "flops_per_step": flops, "ms_per_step": round(gemm_ms, 3)},
            "step_profile_ms": fam, "rank_kernel_ms": busy, "timeline_ms": timeline,
            "in_step_hbm_kernels": in_step_hbm(prof, cfg) if world == 1 else None,
            "kernels": None if ops_line is None else ops_line.get("kernels"),
            "ops_microbench": None if ops_line is None else {"value": ops_line["value"], "unit": "tokens/s",
                                                             "roofline": ops_line["roofline"]},
            "cpu_baseline": cpu_baseline_finetune() if world == 1 else None, "loss": None if loss is None else round(loss, 4),
            # mean loss of every timed step (they follow the warm-up steps): equal across GPU counts for equal --warmup / --steps
            "loss_trace": [None if v is None else round(v, 4) for v in trace],
        }
        emit_line(out)
    tr.close()
    if world > 1:
        host.collective_shutdown()
        dist.destroy_process_group()


def run_prefill(args):
    """Forward-only scoring of 8 x 2048 tokens: one pass = every sequence through all stages and the head, per-token NLL
    read back on the rank that holds the head."""
    import torch
    import torch.distributed as dist
    from blackriver_b200 import finetune, host

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = dict(PREFILL)
    if args.layers:
        cfg["n_layers"] = args.layers
    compute_stream = torch.cuda.Stream(device=dev)          # torch events and the library's work share this stream
    torch.cuda.set_stream(compute_stream)
    host.context_boot(local, compute_stream.cuda_stream, 512 << 20)
    if world > 1:
        box = [host.collective_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        host.collective_boot(rank, world, box[0])
    else:
        host.collective_boot_local(0, 1)
    tr = finetune.Trainer(cfg["hidden"], cfg["heads"], cfg["vocab"], cfg["n_layers"], cfg["batch"], cfg["tokens"], cfg["n_micro"],
                          rank=rank, world=world, seed=cfg["seed"], logits_rows=cfg["batch"] * cfg["tokens"],
                          overlap=not args.no_overlap, n_slots=4)
    mbs = finetune.make_microbatches(cfg["n_micro"], cfg["batch"], cfg["tokens"], cfg["vocab"], cfg["min_len"], cfg["seed"])
    tokens_per_pass = cfg["n_micro"] * cfg["batch"] * cfg["tokens"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out = None
    for _ in range(args.warmup):
        out = tr.score(mbs)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    t0w = time.time()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = tr.score(mbs)
    tr.sync()
    e1.record()
    barrier()
    t1w = time.time()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop(t0w, t1w) if rank == 0 else None
    host.profile_start()
    tr.score(mbs)
    prof = host.profile_stop()
    barrier()
    mean_nll = float(sum(m for _, m in out) / len(out)) if out else None
    if world > 1:
        t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t[0])
        box = [mean_nll]
        dist.broadcast_object_list(box, src=world - 1)
        mean_nll = box[0]
    if rank == 0:
        ms = ms_total / args.steps
        value = tokens_per_pass / (ms * 1e-3)
        peak_tf, peak_src = load_tensor_peak()
        n, H, V = cfg["batch"] * cfg["tokens"], cfg["hidden"], cfg["vocab"]
        flops = cfg["n_micro"] * (tr.gemm_layers * 2 * n * 12 * H * H + (2 * n * H * V if world == 1 else 0))
        gemm_ms = prof.get("gemm_f16", {}).get("ms", 0.0)
        achieved = flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        # the scoring pass reads every micro-batch's per-token NLL back, so the timed region already is the end-to-end one
        h2d = sum(finetune.pack_inputs(m).nbytes for m in mbs)
        d2h = tokens_per_pass * 4
        emit_line({
            "metric": "tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
            "config": {"workload": PREFILL_WORKLOAD, "layers": cfg["n_layers"], "micro_batches": cfg["n_micro"],
                       "tokens_per_step": tokens_per_pass, "parallelism": "pp%d" % world, "stage_layers": tr.counts,
                       "l2": "inputs larger than L2: every pass streams the stage's weights (>= 1.7 GB per GPU) between re-uses"},
            "clocks": clocks, "gpu_launches": sum(v["calls"] for v in prof.values()) * args.steps,
            "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "roofline": {"kernel": "gemm_tc_pair_kernel (forward GEMMs of rank 0's stage in one pass)", "bound": "tensor",
                         "achieved": None if achieved is None else round(achieved, 1), "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": None if achieved is None else round(achieved / peak_tf, 3), "peak_source": peak_src, "traffic": None},
            "step_profile_ms": {k: {"ms": round(v["ms"], 3), "calls": v["calls"]} for k, v in sorted(prof.items(), key=lambda kv: -kv[1]["ms"])},
            "cpu_baseline": None, "mean_nll": None if mean_nll is None else round(mean_nll, 4),
        })
    tr.close()
    if world > 1:
        host.collective_shutdown()
        dist.destroy_process_group()


def in_step_hbm(prof, cfg):
    """The HBM-bound kernels as the step launches them (2048 rows per launch, inputs mostly still in L2 from the kernel
    before): interval between the event records around each launch (about 3 us of event overhead included), algorithmic
    bytes per launch and the rate against the measured HBM copy peak."""
    n, H, es = cfg["batch"] * cfg["tokens"], cfg["hidden"], 2
    peak, _ = load_peaks()
    per_call = {
        "layernorm_fwd": 2 * n * H * es + 2 * H * es + 4 * n,
        "layernorm_bwd": 4 * n * H * es + 4 * n + 4 * H * es,      # dy, y and the residual in, dx out (the layers' launches)
        "gelu_bwd": 3 * n * 4 * H * es,
        "add": 3 * n * H * es,
        # four bias gradients per layer: dy of 4h->h, h->4h, dense and QKV, read once each
        "colsum": (1 + 4 + 1 + 3) * n * H * es / 4,
    }
    out = {}
    for k, b in per_call.items():
        if k in prof and prof[k]["calls"]:
            us = prof[k]["ms"] / prof[k]["calls"] * 1e3
            gbs = b / (us * 1e-6) / 1e9
            out[k] = {"us_per_launch": round(us, 2), "algorithmic_bytes": int(b), "gbs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / peak, 3)}
    return out


FT_CPU_LAYER_TOKENS = 32


def cpu_finetune_parts(np, orc, layer_tokens, rng):
    """Inputs of the CPU sample: one 7b1-shaped decoder layer on `layer_tokens` tokens and the LM head."""
    H, heads = FT["hidden"], FT["heads"]
    p = {}
    for name in orc.LAYER_PARAMS:
        if name.endswith("layernorm.weight"):
            p[name] = np.ones(H, np.float32)
        elif name.endswith(".bias"):
            k = {"query_key_value": 3, "dense_h_to_4h": 4}.get(name.split(".")[0], 1)
            p[name] = np.zeros(k * H, np.float32)
        else:
            o, i = {"query_key_value.weight": (3, 1), "dense.weight": (1, 1), "dense_h_to_4h.weight": (4, 1),
                    "dense_4h_to_h.weight": (1, 4)}[name]
            p[name] = rng.standard_normal((o * H, i * H), dtype=np.float32) * np.float32(0.02)
    x = rng.standard_normal((1, layer_tokens, H), dtype=np.float32)
    mask = np.ones((1, layer_tokens), np.int32)
    return p, x, orc.alibi(heads, layer_tokens), orc.build_xmask(mask), heads


def cpu_layer_seconds(orc, parts):
    p, x, al, xm, heads = parts
    t0 = time.perf_counter()
    out, saved = orc.layer_forward(x, p, al, xm, heads)
    orc.layer_backward(x, p, saved, heads)
    return time.perf_counter() - t0


def cpu_head_seconds_per_token(np, orc, rng, tokens=2):
    H, V = FT["hidden"], FT["vocab"]
    block = rng.standard_normal((1024, H), dtype=np.float32) * np.float32(0.02)
    w = np.tile(block, (V // 1024 + 1, 1))[:V]                 # cheap to build; the arithmetic does not care
    x = rng.standard_normal((1, tokens + 1, H), dtype=np.float32)
    ids = rng.integers(0, V, (1, tokens + 1)).astype(np.int32)
    mask = np.ones((1, tokens + 1), np.int32)
    wg = np.zeros_like(w)
    t0 = time.perf_counter()
    orc.loss_backward(x, ids, mask, w, w_g=wg)
    return (time.perf_counter() - t0) / tokens


def cpu_baseline_finetune():
    import numpy as np
    from oracle import oracle as orc
    orc.use_all_cores()
    rng = np.random.default_rng(FT["seed"])
    parts = cpu_finetune_parts(np, orc, FT_CPU_LAYER_TOKENS, rng)
    t_layer = min(cpu_layer_seconds(orc, parts) for _ in range(2))
    t_head = cpu_head_seconds_per_token(np, orc, rng)
    per_token = FT["n_layers"] * t_layer / FT_CPU_LAYER_TOKENS + t_head
    return {"value": round(1.0 / per_token, 4), "unit": "tokens/s", "cores": orc.num_threads(), "kind": "port",
            "sample": f"fp32 CPU oracle (OpenMP): one 7b1-shaped decoder layer fwd+bwd on {FT_CPU_LAYER_TOKENS} tokens "
                      f"({t_layer:.2f} s) and LM head + loss fwd+bwd on 2 tokens ({t_head:.2f} s/token); "
                      "extrapolated to 30 layers + head per token, no optimizer"}


def time_gemm_shapes(torch, ops, brk, dev):
    """Every GEMM shape of one 7b1 layer and of the LM head for one micro-batch of 2048 tokens, in isolation: CUDA events
    around single launches, L2 flushed before each, median of 5; both epilogues of the CTA-pair kernel."""
    g = torch.Generator(device=dev).manual_seed(0)
    N, H = 2048, 4096
    shapes = {  # name: (m, n, k, trans_a, trans_b, accumulate)
        "fwd_qkv": (N, 3 * H, H, 0, 1, 0), "fwd_dense": (N, H, H, 0, 1, 0), "fwd_h4h": (N, 4 * H, H, 0, 1, 0), "fwd_4hh": (N, H, 4 * H, 0, 1, 0),
        "dx_qkv": (N, H, 3 * H, 0, 0, 0), "dx_dense": (N, H, H, 0, 0, 0), "dx_h4h": (N, H, 4 * H, 0, 0, 0), "dx_4hh": (N, 4 * H, H, 0, 0, 0),
        "dw_qkv": (3 * H, H, N, 1, 0, 1), "dw_dense": (H, H, N, 1, 0, 1), "dw_h4h": (4 * H, H, N, 1, 0, 1), "dw_4hh": (H, 4 * H, N, 1, 0, 1),
        "head_fwd": (N, VOCAB, H, 0, 1, 0), "head_dx": (N, H, VOCAB, 0, 0, 0), "head_dw": (VOCAB, H, N, 1, 0, 1),
    }
    res = {}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for name, (m, n, k, ta, tb, acc) in shapes.items():
        a = torch.randn((k, m) if ta else (m, k), generator=g, device=dev).half()
        b = torch.randn((n, k) if tb else (k, n), generator=g, device=dev).half()
        c = torch.zeros(m, n, device=dev).half()
        for epi, nosplit, tag in ((0, 0, "tma"), (0, 1, "tma, no split-k"), (1, 1, "registers")):
            brk.lib().brk_gemm_f16_set_epilogue(epi)
            brk.lib().brk_gemm_f16_set_split_k(nosplit)
            ts = []
            for _ in range(6):
                flush.zero_()
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
                ops.gemm_f16(a, b, c, m, n, k, ta, tb, a.shape[1], b.shape[1], n, accumulate=bool(acc))
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            t = sorted(ts[1:])[2]
            res[f"{name}/{tag}"] = {"us": round(t * 1e3, 1), "tflops": round(2 * m * n * k / t / 1e9, 1)}
        del a, b, c
    brk.lib().brk_gemm_f16_set_epilogue(0)
    brk.lib().brk_gemm_f16_set_split_k(0)
    assert brk.lib().brk_gemm_f16_status() == 0
    return res


def time_hbm_shapes(torch, ops, brk, dev):
    """The HBM-bound kernels at the row count the fine-tune step launches them with (one micro-batch = 2048 rows) and at the
    microbench's 8192: CUDA events around single launches, median of 5, once with L2 flushed before each launch ("cold")
    and once with the inputs written just before ("warm": what the step sees after the producing GEMM).  LayerNorm in both
    kernel modes (0 = shared-memory ring, persistent CTAs; 1 = a warp per row from registers)."""
    g = torch.Generator(device=dev).manual_seed(0)
    H = 4096
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    peak, _ = load_peaks()
    res = {}

    def timed(fn, warm_src):
        out = {}
        for cond in ("cold", "warm"):
            ts = []
            for _ in range(6):
                if cond == "cold":
                    flush.zero_()
                else:
                    for t in warm_src:
                        t.add_(0)            # rewrites the inputs: they sit in L2 as after their producer
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            out[cond] = sorted(ts[1:])[2]
        return out

    def put(name, t, nbytes):
        res[name] = {c: {"us": round(v * 1e3, 2), "gbs": round(nbytes / v / 1e6, 1), "frac_of_measured_hbm": round(nbytes / v / 1e6 / peak, 3)}
                     for c, v in t.items()}

    for rows in (2048, 8192):
        x = torch.randn(rows, H, generator=g, device=dev).half()
        dy = torch.randn(rows, H, generator=g, device=dev).half()
        y = torch.empty_like(x)
        dx = torch.empty_like(x)
        gamma = torch.ones(H, device=dev).half()
        beta = torch.zeros(H, device=dev).half()
        dg, db = torch.empty_like(gamma), torch.empty_like(beta)
        ws = torch.empty(max(16, brk.lib().brk_layernorm_bwd_workspace_bytes(rows, H)), dtype=torch.uint8, device=dev)
        _, _, var = ops.layernorm(x, gamma, beta, out=y)
        for mode in (0, 1):
            brk.lib().brk_layernorm_set_mode(mode)
            put(f"layernorm_fwd/rows{rows}/mode{mode}", timed(lambda: ops.layernorm(x, gamma, beta, out=y), [x]), 2 * rows * H * 2)
            put(f"layernorm_bwd/rows{rows}/mode{mode}",
                timed(lambda: ops.layernorm_backward(dy, gamma, beta, var, y, dgamma=dg, dbeta=db, dx=dx, workspace=ws), [dy, y]),
                3 * rows * H * 2)
        brk.lib().brk_layernorm_set_mode(0)
        put(f"add/rows{rows}", timed(lambda: ops.add(x, dy, out=dx), [x, dy]), 3 * rows * H * 2)
        for cols in (H, 4 * H):
            m = torch.randn(rows, cols, generator=g, device=dev).half()
            out = torch.zeros(cols, device=dev).half()
            cws = torch.empty(brk.lib().brk_colsum_workspace_bytes(rows, cols), dtype=torch.uint8, device=dev)
            put(f"colsum/rows{rows}/cols{cols}",
                timed(lambda: brk.call("brk_colsum_ws", m.data_ptr(), out.data_ptr(), rows, cols, 1, 1, cws.data_ptr(), cws.numel(), ops.stream()), [m]),
                rows * cols * 2)
            del m
    return res


def time_attention_shapes(torch, ops, brk, dev):
    """Fused attention forward and backward (delta + dK/dV + dQ kernels) at several shapes, head dimension 128: CUDA events
    around 10 launches queued back to back.  FLOPs: causal half of 4 B h T^2 d forward, 2.5 x that backward."""
    res = {}
    d = 128
    for B, T, heads in ((2, 1024, 32), (1, 2048, 32), (4, 1024, 32), (8, 256, 32), (16, 128, 32), (2, 1024, 8)):
        H = heads * d
        qkv = torch.randn(B * T, 3 * H, device=dev).half()
        out = torch.empty(B * T, H, device=dev).half()
        lse = torch.empty(B, heads, T, device=dev)
        dout = torch.randn(B * T, H, device=dev).half()
        grads = torch.empty(B * T, 3 * H, device=dev).half()
        ws = torch.empty(brk.lib().brk_flash_attn_bwd_workspace_bytes(B, T, heads), dtype=torch.uint8, device=dev)
        base, gb = qkv.data_ptr(), grads.data_ptr()

        def fwd():
            brk.call("brk_flash_attn_fwd", base, base + 2 * H, base + 4 * H, 3 * H, out.data_ptr(), H, lse.data_ptr(), 0, 0, B, T, heads, d,
                     ops.stream())

        def bwd():
            brk.call("brk_flash_attn_bwd", base, base + 2 * H, base + 4 * H, 3 * H, out.data_ptr(), dout.data_ptr(), H, lse.data_ptr(),
                     gb, gb + 2 * H, gb + 4 * H, 3 * H, 0, 0, B, T, heads, d, ws.data_ptr(), ws.numel(), ops.stream())
        o = {"work_items": B * heads * ((T + 127) // 128)}
        flops = 4 * B * heads * T * T * d / 2
        for name, fn, mult in (("fwd", fwd, 1.0), ("bwd", bwd, 2.5)):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 100
            o[name + "_us"] = round(us, 1)
            o[name + "_tflops"] = round(mult * flops / us / 1e6, 1)
        res[f"batch{B}_tokens{T}_heads{heads}"] = o
    assert brk.lib().brk_flash_attn_status() == 0
    return res


def run_case(args):
    """A few launches of one kernel family on a small, larger-than-L2 case (for ncu captures), or a timing table."""
    import torch
    from blackriver_b200 import ops
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    if args.case in ("gemm_shapes", "attn_shapes", "hbm_shapes"):
        from blackriver_b200 import brk
        table = {"gemm_shapes": time_gemm_shapes, "attn_shapes": time_attention_shapes, "hbm_shapes": time_hbm_shapes}[args.case](torch, ops, brk, dev)
        emit_line({"case": args.case, "table": table})
        return
    g = torch.Generator(device=dev).manual_seed(SEED)
    rows = args.rows
    reps = 3
    if args.case == "nll":
        logits = (torch.randn(rows, VOCAB, generator=g, device=dev) * 2).half()
        target = torch.randint(0, VOCAB, (rows,), generator=g, device=dev, dtype=torch.int32)
        target[torch.rand(rows, generator=g, device=dev) < MASK_FRAC] = -100
        dl = torch.empty_like(logits)
        rl = torch.empty(rows, dtype=torch.float32, device=dev)
        for _ in range(reps):
            ops.logsoftmax_nll_backward(logits, target, 1.0 / rows, row_loss=rl, dlogits=dl)
        for _ in range(reps):
            ops.logsoftmax_nll(logits, target, row_loss=rl)
    elif args.case == "ln":
        rows = max(rows, TOKENS * 2)      # 2 x 134 MB per tensor: larger than L2
        x = torch.randn(rows, HIDDEN, generator=g, device=dev).half()
        dy = torch.randn(rows, HIDDEN, generator=g, device=dev).half()
        gamma = torch.ones(HIDDEN, device=dev).half()
        beta = torch.zeros(HIDDEN, device=dev).half()
        for _ in range(reps):
            y, _, var = ops.layernorm(x, gamma, beta)
        for _ in range(reps):
            ops.layernorm_backward(dy, gamma, beta, var, y)
    elif args.case == "gemm":
        m, n, k = 2048, 16384, 4096          # the h -> 4h projection of one micro-batch
        a = torch.randn(m, k, generator=g, device=dev).half()
        b = torch.randn(n, k, generator=g, device=dev).half()
        c = torch.empty(m, n, device=dev).half()
        for _ in range(reps * 2):
            ops.gemm_f16(a, b, c, m, n, k, 0, 1, k, k, n)
    elif args.case == "gemm_dx":
        # input gradient of the h -> 4h projection for one micro-batch: dX [2048, 4096] = dy [2048, 16384] x W [16384, 4096];
        # 128 pair tiles, each cut into 4 split-k items
        m, n, k = 2048, 4096, 16384
        a = torch.randn(m, k, generator=g, device=dev).half()
        b = torch.randn(k, n, generator=g, device=dev).half()
        c = torch.empty(m, n, device=dev).half()
        for _ in range(reps * 2):
            ops.gemm_f16(a, b, c, m, n, k, 0, 0, k, n, n)
    elif args.case == "gemm_dw":
        # weight gradient of the h -> 4h projection for one micro-batch: W_g [16384, 4096] += dy^T [16384, 2048] x [2048, 4096]
        m, n, k = 16384, 4096, 2048
        a = torch.randn(k, m, generator=g, device=dev).half()
        b = torch.randn(k, n, generator=g, device=dev).half()
        c = torch.zeros(m, n, device=dev).half()
        for _ in range(reps * 2):
            ops.gemm_f16(a, b, c, m, n, k, 1, 0, m, n, n, accumulate=True)
    elif args.case == "attn":
        from blackriver_b200 import brk
        B, T, heads, d = 2, 1024, 32, 128
        H = heads * d
        qkv = torch.randn(B * T, 3 * H, generator=g, device=dev).half()
        out = torch.empty(B * T, H, device=dev).half()
        lse = torch.empty(B, heads, T, device=dev)
        base = qkv.data_ptr()
        for _ in range(reps):
            brk.call("brk_flash_attn_fwd", base, base + 2 * H, base + 4 * H, 3 * H, out.data_ptr(), H, lse.data_ptr(), 0, 0,
                     B, T, heads, d, ops.stream())
        dout = torch.randn(B * T, H, generator=g, device=dev).half()
        grads = torch.empty(B * T, 3 * H, device=dev).half()
        ws = torch.empty(brk.lib().brk_flash_attn_bwd_workspace_bytes(B, T, heads), dtype=torch.uint8, device=dev)
        gb = grads.data_ptr()
        for _ in range(reps):
            brk.call("brk_flash_attn_bwd", base, base + 2 * H, base + 4 * H, 3 * H, out.data_ptr(), dout.data_ptr(), H, lse.data_ptr(),
                     gb, gb + 2 * H, gb + 4 * H, 3 * H, 0, 0, B, T, heads, d, ws.data_ptr(), ws.numel(), ops.stream())
    else:
        x = torch.randn(TOKENS, HIDDEN4, generator=g, device=dev).half()
        dy = torch.randn(TOKENS, HIDDEN4, generator=g, device=dev).half()
        out = torch.empty_like(x)
        for _ in range(reps):
            ops.gelu(x, out=out)
        for _ in range(reps):
            ops.gelu_backward(dy, x, out=out)
    torch.cuda.synchronize()
    emit_line({"case": args.case, "rows": rows, "launch_groups": 2, "reps": reps})


# dram__bytes_read.sum + dram__bytes_write.sum of one log-softmax+NLL+gradient launch at 8192 rows: the ncu capture of
# the 1024-row case (565.7 MB read + 458.0 MB written per launch, profiles/nll_fwd_bwd_f16_1024rows.md) scaled by rows
NLL_TRAFFIC_BYTES_PER_LAUNCH = int((565.7e6 + 458.0e6) * 8)


def load_traffic():
    """Per-launch DRAM traffic of the operator bench's dominant kernel, from its committed ncu summary."""
    return NLL_TRAFFIC_BYTES_PER_LAUNCH


# ------------------------------------------------------------------------------------------
# CPU legs (the only place the benchmark touches oracle/)
# ------------------------------------------------------------------------------------------
CPU_SAMPLE_TOKENS = 1024


def cpu_inputs(np, sample, rng):
    f32 = np.float32
    x = rng.standard_normal((sample, HIDDEN), dtype=f32)
    dy = rng.standard_normal((sample, HIDDEN), dtype=f32)
    x4 = rng.standard_normal((sample, HIDDEN4), dtype=f32)
    dy4 = rng.standard_normal((sample, HIDDEN4), dtype=f32)
    gamma = np.ones(HIDDEN, f32)
    beta = np.zeros(HIDDEN, f32)
    logits = rng.standard_normal((sample, VOCAB), dtype=f32) * f32(2)
    target = rng.integers(0, VOCAB, sample).astype(np.int32)
    target[rng.random(sample) < MASK_FRAC] = -100
    return x, dy, x4, dy4, gamma, beta, logits, target


def cpu_pass(orc, inputs):
    """One pass of the same operator list with the CPU oracle on the sampled tokens; seconds."""
    x, dy, x4, dy4, gamma, beta, logits, target = inputs
    t0 = time.perf_counter()
    y, _, var = orc.layernorm(x, gamma, beta)
    orc.gelu(x4)
    orc.layernorm_backward(dy, gamma, beta, var, y)
    orc.gelu_backward(dy4, x4)
    orc.gelu(x)
    orc.gelu_backward(dy, x)
    orc.logsoftmax_nll(logits, target, grad_scale=1.0 / len(target))
    return time.perf_counter() - t0


def cpu_baseline(steps=3):
    import numpy as np
    from oracle import oracle as orc
    rng = np.random.default_rng(SEED)
    inputs = cpu_inputs(np, CPU_SAMPLE_TOKENS, rng)
    cpu_pass(orc, inputs)
    t = min(cpu_pass(orc, inputs) for _ in range(steps))
    return {"value": round(CPU_SAMPLE_TOKENS / t, 1), "unit": "tokens/s", "cores": orc.num_threads(), "kind": "port",
            "sample": f"{CPU_SAMPLE_TOKENS} of the 8192 tokens per pass, same operator list and shapes, fp32 CPU oracle "
                      f"(OpenMP), best of {steps}"}


def run_reference(args):
    """Reference arm: the reference has no CPU implementation of this path (its cpu_tensor is storage
    only), so this times the fp32 CPU restatement of its operator semantics on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle as orc
    orc.use_all_cores()          # the launcher of a multi-rank run exports OMP_NUM_THREADS=1; the CPU arm uses every core
    if args.workload == "ops":
        rng = np.random.default_rng(SEED)
        inputs = cpu_inputs(np, CPU_SAMPLE_TOKENS, rng)
        for _ in range(max(1, min(args.warmup, 3))):
            cpu_pass(orc, inputs)
        ts = [cpu_pass(orc, inputs) for _ in range(args.steps)]
        t = sum(ts) / len(ts)
        value, workload, sample = CPU_SAMPLE_TOKENS / t, WORKLOAD, f"{CPU_SAMPLE_TOKENS} of the 8192 tokens per step"
    else:
        # each timed step = one 7b1-shaped decoder layer fwd+bwd on S tokens, S sized from --steps so that the
        # run ends within a few minutes; the LM head + loss cost per token is measured once before the timed steps
        rng = np.random.default_rng(FT["seed"])
        budget = 150.0 / (args.steps + max(1, min(args.warmup, 3)))
        layer_tokens = int(max(8, min(256, budget / 0.08)))
        parts = cpu_finetune_parts(np, orc, layer_tokens, rng)
        t_head = cpu_head_seconds_per_token(np, orc, rng)
        for _ in range(max(1, min(args.warmup, 3))):
            cpu_layer_seconds(orc, parts)
        ts = [cpu_layer_seconds(orc, parts) for _ in range(args.steps)]
        t = sum(ts) / len(ts)
        value = 1.0 / (FT["n_layers"] * t / layer_tokens + t_head)
        workload = FT_WORKLOAD
        sample = (f"per step one decoder layer fwd+bwd on {layer_tokens} tokens ({t:.2f} s); LM head + loss {t_head:.2f} s/token "
                  "measured once; tokens/s extrapolated to 30 layers + head, no optimizer")
    out = {
        "impl": "reference", "metric": "tokens/s", "value": round(value, 4), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(t * 1e3, 3), "higher_is_better": True,
        "scaling": "strong" if args.workload != "ops" else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "note": "the reference has no CPU implementation of these operators (its cpu_tensor "
                   "is storage only); this arm times the fp32 CPU restatement of its operator semantics on the host cores, "
                   "each step a bounded sample of the workload"},
        "cpu_baseline": {"value": round(value, 4), "unit": "tokens/s", "cores": orc.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit_line(out)


RESULT_OUT = None      # the process's original stdout; everything else written to fd 1 goes to stderr


def emit_line(obj):
    """The one JSON line of a run."""
    out = RESULT_OUT or sys.stdout
    out.write(json.dumps(obj) + "\n")
    out.flush()


def keep_stdout_clean():
    """Libraries (NCCL's version banner, for one) print to fd 1; the run's stdout must carry the JSON
    line only, so fd 1 is pointed at stderr and the result is written to a private copy of the old fd 1."""
    global RESULT_OUT
    sys.stdout.flush()
    RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def main():
    keep_stdout_clean()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="finetune", choices=["finetune", "ops", "c3", "prefill"],
                    help="finetune: the headline step (16 micro-batches of 2 x 1024); ops: the operator microbench; c3: one "
                         "micro-batch of 4 x 512 on one GPU; prefill: forward-only scoring of 8 x 2048 tokens")
    ap.add_argument("--layers", type=int, default=0, help="fine-tune workload with fewer layers (development aid)")
    ap.add_argument("--micro", type=int, default=0, help="fine-tune workload with fewer micro-batches (development aid)")
    ap.add_argument("--replicas", type=int, default=1,
                    help="fine-tune workload: data-parallel replicas of a (gpus / replicas)-stage pipeline; the default is one pipeline over all GPUs")
    ap.add_argument("--timeline", action="store_true",
                    help="fine-tune workload: also report when each task of one step ended on every rank (development aid)")
    ap.add_argument("--early-exchange", action="store_true",
                    help="fine-tune workload: the last rank takes the LM-head weight gradients first and starts the tied-table "
                         "exchange from its task list; stages chosen for the steady-state step time")
    ap.add_argument("--async-optimizer", action="store_true",
                    help="fine-tune workload: queue Adam on the transfer stream beside the next step's first forward instead of on the compute stream after the step")
    ap.add_argument("--no-overlap", action="store_true",
                    help="multi-GPU: the plain schedule (all forwards, all backwards, NCCL hand-offs) instead of the overlapped one")
    ap.add_argument("--skip-ops", action="store_true", help="do not run the operator microbench before the fine-tune step")
    ap.add_argument("--case", default=None, choices=["nll", "ln", "gelu", "gemm", "gemm_dx", "gemm_dw", "attn", "gemm_shapes", "attn_shapes", "hbm_shapes"],
                    help="profiling aid: run a few launches of one kernel family on a small case and exit")
    ap.add_argument("--rows", type=int, default=1024, help="rows of the --case run")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = 200 if args.workload == "ops" else 5
    if args.case:
        return run_case(args)
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "ops":
        run_ops(args)
    elif args.workload == "prefill":
        run_prefill(args)
    else:
        run_finetune(args)


if __name__ == "__main__":
    main()
