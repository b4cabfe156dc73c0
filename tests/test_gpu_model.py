"""Whole-model training step through the words machine (fused fp16 path) against the CPU oracle.

A small BLOOM-shaped model (2 layers, hidden 128 = 2 heads x 64, vocab 512, tied embedding,
embedding LayerNorm, ALiBi, right padding) is built by the generated scripts, initialised on the
device with the seeded generator, and run forward + backward.  The oracle repeats the same
computation in fp32 from the device's fp16 initial weights.  Tolerances: loss 1e-3 relative,
gradients 2e-2 (max|err|/max|ref|); the optimizer kernel is checked separately on identical inputs."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def relerr(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


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
        owned = False          # another test module of this process booted it already
    yield _host
    if owned:
        _host.context_shutdown()


def oracle_model(p_main, layers, ids, mask, heads, eps=1e-5):
    B, T = ids.shape
    table = p_main["word_embeddings.weight"]
    x = orc.embedding_gather(table, ids)
    e, _, evar = orc.layernorm(x, p_main["word_embeddings_layernorm.weight"], p_main["word_embeddings_layernorm.bias"], eps)
    al = orc.alibi(heads, T); xm = orc.build_xmask(mask)
    h, saved = e, []
    for p in layers:
        h, s = orc.layer_forward(h, p, al, xm, heads, eps)
        saved.append(s)
    xf, _, fvar = orc.layernorm(h, p_main["ln_f.weight"], p_main["ln_f.bias"], eps)
    loss, xf_g, table_g = orc.loss_backward(xf, ids, mask, table)
    dg_f, db_f, dh = orc.layernorm_backward(xf_g, p_main["ln_f.weight"], p_main["ln_f.bias"], fvar, xf, eps)
    grads = []
    for p, s in zip(reversed(layers), reversed(saved)):
        dh, g = orc.layer_backward(dh, p, s, heads, eps)
        grads.append(g)
    grads.reverse()
    dg_e, db_e, dx = orc.layernorm_backward(dh, p_main["word_embeddings_layernorm.weight"], p_main["word_embeddings_layernorm.bias"], evar, e, eps)
    np.add.at(table_g, ids.reshape(-1), dx.reshape(-1, dx.shape[-1]))
    return loss, {"ln_f.weight": dg_f, "ln_f.bias": db_f, "word_embeddings_layernorm.weight": dg_e,
                  "word_embeddings_layernorm.bias": db_e, "word_embeddings.weight": table_g}, grads


def test_small_model_step(host):
    from blackriver_b200 import words
    H, heads, V, L, B, T = 128, 2, 512, 2, 2, 96
    lens = [96, 50]
    rng = np.random.default_rng(0)
    ids = rng.integers(0, V, (B, T)).astype(np.int32)
    mask = np.zeros((B, T), np.int32)
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    env = host.Env(L + 1)
    try:
        env.execute(words.fused_words(hidden=H, heads=heads, vocab=V, n_layers=L, batch=B, tokens=T, dtype="half",
                                      logits_rows=40, init_std=0.05, seed=3))
        env.execute("build_model init_model zero_grads")
        # give LayerNorms and biases non-trivial values so that their gradients are exercised
        for i in range(1, L + 1):
            env.change(i)
            for name in ("input_layernorm", "post_attention_layernorm"):
                env.write(name + ".weight", 1 + 0.1 * rng.standard_normal(H)); env.write(name + ".bias", 0.1 * rng.standard_normal(H))
            env.write("dense.bias", 0.05 * rng.standard_normal(H))
        env.change(0)
        env.write("ids_", ids); env.write("mask_", mask); env.write("lens_", np.array(lens, np.int32))
        main_names = ("word_embeddings.weight", "word_embeddings_layernorm.weight", "word_embeddings_layernorm.bias", "ln_f.weight", "ln_f.bias")
        p_main = {k: env.read(k).astype(np.float32) for k in main_names}
        layers = []
        for i in range(1, L + 1):
            env.change(i)
            layers.append({k: env.read(k).astype(np.float32) for k in orc.LAYER_PARAMS})
        env.change(0)
        assert abs(p_main["word_embeddings.weight"].std() - 0.05) < 0.005        # seeded device initialisation
        assert not np.array_equal(layers[0]["dense.weight"], layers[1]["dense.weight"])

        env.execute("model_forward model_backward op.sync")
        loss_ref, gmain_ref, glayers_ref = oracle_model(p_main, layers, ids, mask, heads)
        assert abs(host.last_loss() - loss_ref) <= 1e-3 * abs(loss_ref)
        for k in main_names:
            assert relerr(env.read(k + "_g"), gmain_ref[k]) <= 2e-2, k
        for i in range(1, L + 1):
            env.change(i)
            for k in orc.LAYER_PARAMS:
                assert relerr(env.read(k + "_g"), glayers_ref[i - 1][k + "_g"]) <= 2e-2, (i, k)
        env.change(0)

        # gradient accumulation over two identical micro-batches doubles every gradient
        g1 = env.read("ln_f.weight_g").astype(np.float32)
        env.change(1); w1 = env.read("dense_h_to_4h.weight_g").astype(np.float32); env.change(0)
        env.execute("1 op.accumulate model_forward model_backward op.sync 0 op.accumulate")
        assert relerr(env.read("ln_f.weight_g"), 2 * g1) <= 2e-2
        env.change(1); assert relerr(env.read("dense_h_to_4h.weight_g"), 2 * w1) <= 2e-2; env.change(0)

        # one optimizer step moves the weights and keeps the fp16 copy equal to the rounded master
        before = env.read("ln_f.weight.master").copy()
        env.execute("0.001 1 0.5 optimizer_step op.sync")
        after = env.read("ln_f.weight.master")
        assert np.abs(after - before).max() > 1e-4
        assert np.array_equal(env.read("ln_f.weight"), after.astype(np.float16))
        env.change(2)
        assert np.array_equal(env.read("_flat"), env.read("_flat.master").astype(np.float16))
    finally:
        env.close()


def read_params(env, L):
    main_names = ("word_embeddings.weight", "word_embeddings_layernorm.weight", "word_embeddings_layernorm.bias", "ln_f.weight", "ln_f.bias")
    env.change(0)
    p_main = {k: env.read(k).astype(np.float32) for k in main_names}
    layers = []
    for i in range(1, L + 1):
        env.change(i)
        layers.append({k: env.read(k).astype(np.float32) for k in orc.LAYER_PARAMS})
    env.change(0)
    return main_names, p_main, layers


def test_sixteen_microbatches_accumulate_like_the_oracle(host):
    """The benchmark's step sums the gradients of 16 different micro-batches in fp16 tensors at loss scale 1024 (the
    weight-gradient GEMM adds into them, LayerNorm and embedding gradients likewise).  Every accumulated gradient must
    stay within the fp16 bound of the fp32 oracle's sum, every per-micro-batch loss within 1e-3, and nothing may
    overflow."""
    from blackriver_b200 import finetune
    H, heads, V, L, B, T, M = 128, 2, 512, 2, 2, 96, 16
    scale = 1024.0
    mbs = finetune.make_microbatches(M, B, T, V, 30, seed=21)
    tr = finetune.Trainer(H, heads, V, L, B, T, n_micro=M, rank=0, world=1, seed=13, init_std=0.05, loss_scale=scale, logits_rows=80)
    try:
        env = tr.env
        main_names, p_main, layers = read_params(env, L)
        tr.begin_step(mbs)
        for i in range(len(tr.tasks)):
            tr.run_task(i)
        tr.check_and_read_losses()               # synchronises; the optimizer is NOT applied, the gradients stay
        sum_main = {k: 0.0 for k in main_names}
        sum_layers = [{k + "_g": 0.0 for k in orc.LAYER_PARAMS} for _ in range(L)]
        for j, (ids, mask, lens) in enumerate(mbs):
            loss_ref, gmain, glayers = oracle_model(p_main, layers, ids, mask, heads)
            assert abs(tr.losses[j] - loss_ref) <= 1e-3 * abs(loss_ref), j
            for k in main_names:
                sum_main[k] = sum_main[k] + gmain[k]
            for i in range(L):
                for k in sum_layers[i]:
                    sum_layers[i][k] = sum_layers[i][k] + glayers[i][k]
        env.change(0)
        for k in main_names:
            got = env.read(k + "_g").astype(np.float32)
            assert np.isfinite(got).all(), k
            assert relerr(got / scale, sum_main[k]) <= 2e-2, k
        for i in range(1, L + 1):
            env.change(i)
            for k in orc.LAYER_PARAMS:
                got = env.read(k + "_g").astype(np.float32)
                assert np.isfinite(got).all(), (i, k)
                assert relerr(got / scale, sum_layers[i - 1][k + "_g"]) <= 2e-2, (i, k)
        env.change(0)
    finally:
        tr.close()


def test_prefill_at_2048_tokens(host):
    """The long-context prefill shape: 2048 positions, head dimension 128, no padding, per-token NLL against the oracle."""
    from blackriver_b200 import finetune
    H, heads, V, L, B, T = 128, 1, 512, 1, 1, 2048
    rng = np.random.default_rng(6)
    ids = rng.integers(0, V, (B, T)).astype(np.int32)
    mask = np.ones((B, T), np.int32)
    mbs = [(ids, mask, np.array([T], np.int32))]
    tr = finetune.Trainer(H, heads, V, L, B, T, n_micro=1, rank=0, world=1, seed=17, init_std=0.05, logits_rows=512)
    try:
        env = tr.env
        main_names, p_main, layers = read_params(env, L)
        (nll, mean), = tr.score(mbs)
        x = orc.embedding_gather(p_main["word_embeddings.weight"], ids)
        h, _, _ = orc.layernorm(x, p_main["word_embeddings_layernorm.weight"], p_main["word_embeddings_layernorm.bias"], 1e-5)
        al = orc.alibi(heads, T); xm = orc.build_xmask(mask)
        for p in layers:
            h, _ = orc.layer_forward(h, p, al, xm, heads, 1e-5)
        xf, _, _ = orc.layernorm(h, p_main["ln_f.weight"], p_main["ln_f.bias"], 1e-5)
        tg, items = orc.loss_targets(ids, mask)
        assert items == T - 1
        logits = xf.reshape(B * T, H) @ p_main["word_embeddings.weight"].T
        total, row_loss, _ = orc.logsoftmax_nll(logits, tg.reshape(-1))
        assert nll.shape == (B, T) and nll[0, T - 1] == 0          # the last position has no target
        assert relerr(nll, row_loss.reshape(B, T)) <= 2e-2
        assert abs(mean - total / items) <= 1e-3 * abs(total / items)
    finally:
        tr.close()


def test_prefill_token_nll(host):
    """Forward-only scoring (the long-context prefill configuration at test size): per-token next-token NLL from the
    words path against the fp32 oracle; full-length and padded sequences; the logits band is smaller than the batch."""
    from blackriver_b200 import finetune
    H, heads, V, L, B, T = 128, 2, 512, 2, 2, 160
    rng = np.random.default_rng(4)
    mbs = []
    for lens in ([160, 160], [160, 71]):
        ids = rng.integers(0, V, (B, T)).astype(np.int32)
        mask = (np.arange(T)[None, :] < np.array(lens)[:, None]).astype(np.int32)
        ids[mask == 0] = 3
        mbs.append((ids, mask, np.array(lens, np.int32)))
    tr = finetune.Trainer(H, heads, V, L, B, T, n_micro=2, rank=0, world=1, seed=11, init_std=0.05, logits_rows=100)
    try:
        env = tr.env
        env.change(0)
        main_names = ("word_embeddings.weight", "word_embeddings_layernorm.weight", "word_embeddings_layernorm.bias", "ln_f.weight", "ln_f.bias")
        p_main = {k: env.read(k).astype(np.float32) for k in main_names}
        layers = []
        for i in range(1, L + 1):
            env.change(i)
            layers.append({k: env.read(k).astype(np.float32) for k in orc.LAYER_PARAMS})
        env.change(0)
        got = tr.score(mbs)
        assert len(got) == 2
        for (ids, mask, lens), (nll, mean) in zip(mbs, got):
            x = orc.embedding_gather(p_main["word_embeddings.weight"], ids)
            h, _, _ = orc.layernorm(x, p_main["word_embeddings_layernorm.weight"], p_main["word_embeddings_layernorm.bias"], 1e-5)
            al = orc.alibi(heads, T); xm = orc.build_xmask(mask)
            for p in layers:
                h, _ = orc.layer_forward(h, p, al, xm, heads, 1e-5)
            xf, _, _ = orc.layernorm(h, p_main["ln_f.weight"], p_main["ln_f.bias"], 1e-5)
            tg, items = orc.loss_targets(ids, mask)
            logits = xf.reshape(B * T, H) @ p_main["word_embeddings.weight"].T
            total, row_loss, _ = orc.logsoftmax_nll(logits, tg.reshape(-1))
            assert nll.shape == (B, T) and nll.dtype == np.float32
            assert np.array_equal(nll == 0, (tg < 0))                     # exactly the uncounted positions are zero
            assert relerr(nll, row_loss.reshape(B, T)) <= 2e-2
            assert abs(mean - total / items) <= 1e-3 * abs(total / items)
    finally:
        tr.close()


def test_adam_kernel_matches_oracle():
    from blackriver_b200 import brk, ops
    rng = np.random.default_rng(1)
    n = 100003
    w = rng.standard_normal(n).astype(np.float32); m = np.zeros(n, np.float32); v = np.zeros(n, np.float32)
    dw, dm, dv = (torch.from_numpy(x.copy()).cuda() for x in (w, m, v))
    w16 = torch.empty(n, dtype=torch.float16, device="cuda")
    for step in range(1, 4):
        g16 = (rng.standard_normal(n) * 64).astype(np.float16)
        orc.adam(w, m, v, g16.astype(np.float32), lr=1e-2, step=step, grad_scale=1 / 64)
        dg = torch.from_numpy(g16).cuda()
        brk.call("brk_adam_step", dw.data_ptr(), dm.data_ptr(), dv.data_ptr(), dg.data_ptr(), brk.F16, w16.data_ptr(), n, 1e-2, 0.9,
                 0.999, 1e-8, step, 1 / 64, ops.stream())
    torch.cuda.synchronize()
    np.testing.assert_allclose(dw.cpu().numpy(), w, rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(dv.cpu().numpy(), v, rtol=1e-5, atol=1e-9)
    assert np.array_equal(w16.cpu().numpy(), dw.cpu().numpy().astype(np.float16))


def test_init_normal_is_seeded_and_shape_independent():
    from blackriver_b200 import brk, ops
    a = torch.empty(100001, dtype=torch.float32, device="cuda")
    b = torch.empty(50000, dtype=torch.float32, device="cuda")
    brk.call("brk_init_normal", a.data_ptr(), a.numel(), 1.0, 0.5, 42, brk.F32, ops.stream())
    brk.call("brk_init_normal", b.data_ptr(), b.numel(), 1.0, 0.5, 42, brk.F32, ops.stream())
    x = a.cpu().numpy()
    assert np.array_equal(x[:50000], b.cpu().numpy())
    assert abs(x.mean() - 1.0) < 0.01 and abs(x.std() - 0.5) < 0.01
    brk.call("brk_init_normal", b.data_ptr(), b.numel(), 1.0, 0.5, 43, brk.F32, ops.stream())
    assert not np.array_equal(x[:50000], b.cpu().numpy())


def test_embedding_scatter_add():
    from blackriver_b200 import brk, ops
    rng = np.random.default_rng(2)
    V, H, n = 50, 64, 200
    ids = rng.integers(0, V, n).astype(np.int32)
    dx = rng.standard_normal((n, H)).astype(np.float32)
    ref = np.zeros((V, H), np.float32); np.add.at(ref, ids, dx)
    tg = torch.zeros((V, H), dtype=torch.float32, device="cuda")
    ddx, dids = torch.from_numpy(dx).cuda(), torch.from_numpy(ids).cuda()      # keep both alive across the call
    brk.call("brk_embedding_scatter_add", ddx.data_ptr(), dids.data_ptr(), tg.data_ptr(), n, H, V, brk.F32, ops.stream())
    np.testing.assert_allclose(tg.cpu().numpy(), ref, rtol=1e-5, atol=1e-5)


def test_checkpoint_resume_continues_the_same_run(host, tmp_path):
    """save_model / load_model: master weights in the reference's per-tensor raw fp32 files plus the Adam moments.
    Two steps, save, one more step -- against a differently initialised trainer that loads the checkpoint and takes
    the same third step: same loss, same weights."""
    from blackriver_b200 import finetune
    H, heads, V, L, B, T, M = 128, 2, 512, 2, 2, 64, 2
    mbs = finetune.make_microbatches(M, B, T, V, 20, seed=3)
    prefix = str(tmp_path) + "/ck_"
    a = finetune.Trainer(H, heads, V, L, B, T, n_micro=M, seed=31, init_std=0.05, lr=1e-3)
    try:
        a.step(mbs); a.step(mbs)
        a.save(prefix)
        loss_a = a.step(mbs)
        a.sync()
        a.env.change(2); wa = a.env.read("_flat.master").copy(); ma = a.env.read("_flat.m").copy()
        a.env.change(0); ta = a.env.read("word_embeddings.weight").copy()
    finally:
        a.close()
    # the files carry the reference's names and plain fp32 contents
    w = np.fromfile(prefix + "h1.dense_h_to_4h.weight.bin", np.float32)
    assert w.size == 4 * H * H and abs(w.std() - 0.05) < 0.01
    assert np.fromfile(prefix + "word_embeddings.weight.bin", np.float32).size == V * H
    b = finetune.Trainer(H, heads, V, L, B, T, n_micro=M, seed=77, init_std=0.02, lr=1e-3)
    try:
        b.load(prefix)
        assert b.step_no == 2
        loss_b = b.step(mbs)
        b.sync()
        b.env.change(2); wb = b.env.read("_flat.master").copy(); mb_ = b.env.read("_flat.m").copy()
        b.env.change(0); tb = b.env.read("word_embeddings.weight").copy()
    finally:
        b.close()
    # the two third steps repeat the same arithmetic on the same state; only the embedding gradient's atomic adds may
    # land in another order, which can move single table rows by a rounding step of fp16
    assert abs(loss_a - loss_b) <= 1e-4 * abs(loss_a)
    assert np.abs(wa - wb).max() <= 2.5e-3 and np.median(np.abs(wa - wb)) <= 1e-6      # at most one Adam step apart anywhere
    assert np.abs(ma - mb_).max() <= 1e-2 * np.abs(ma).max()
    assert np.abs(ta.astype(np.float32) - tb.astype(np.float32)).max() <= 2.5e-3


def test_async_optimizer_matches_the_blocking_one(host):
    """Adam queued on the transfer stream, with the next step's forward waiting layer by layer for the parameters it
    reads and the gradients cleared behind each update, must give the run of the optimizer on the compute stream."""
    from blackriver_b200 import finetune
    H, heads, V, L, B, T, M = 128, 2, 512, 3, 2, 64, 3
    mbs = finetune.make_microbatches(M, B, T, V, 20, seed=4)
    runs = []
    for flag in (False, True):
        tr = finetune.Trainer(H, heads, V, L, B, T, n_micro=M, seed=23, init_std=0.05, lr=1e-3, async_optimizer=flag)
        try:
            losses = [tr.step(mbs) for _ in range(4)]
            scored = tr.score(mbs[:1])[0][1]          # a forward right behind the last asynchronous update
            tr.sync()
            tr.env.change(3); w = tr.env.read("_flat.master").copy(); g = tr.env.read("_flat_g").copy()
            tr.env.change(0); t = tr.env.read("word_embeddings.weight.master").copy()
            runs.append((losses, scored, w, g, t))
        finally:
            tr.close()
    (la, sa, wa, ga, ta), (lb, sb, wb, gb, tb) = runs
    for a, b in zip(la, lb):
        assert abs(a - b) <= 1e-4 * abs(a)
    assert abs(sa - sb) <= 1e-4 * abs(sa)
    assert np.abs(wa - wb).max() <= 2.5e-3 and np.median(np.abs(wa - wb)) <= 1e-6
    assert np.abs(ta - tb).max() <= 2.5e-3
    assert not gb.any()                               # the asynchronous update leaves the gradients cleared


def test_adam_skips_non_finite_gradients():
    """An overflowed fp16 gradient (inf under the loss scale) must not poison the weight or the moments."""
    from blackriver_b200 import brk, ops
    n = 1001
    w = torch.ones(n, device="cuda"); m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    g = torch.full((n,), 0.5, dtype=torch.float16, device="cuda")
    g[7] = float("inf"); g[1000] = float("nan")
    w16 = torch.empty(n, dtype=torch.float16, device="cuda")
    assert brk.lib().brk_adam_status() == 0
    brk.call("brk_adam_step", w.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), brk.F16, w16.data_ptr(), n, 1e-2, 0.9, 0.999, 1e-8, 1, 1.0,
             ops.stream())
    torch.cuda.synchronize()
    assert brk.lib().brk_adam_status() == 1 and brk.lib().brk_adam_status() == 0      # reported once, then cleared
    wn = w.cpu().numpy()
    assert np.isfinite(wn).all() and wn[7] == 1.0 and wn[1000] == 1.0 and wn[0] < 1.0
    assert float(m[7]) == 0.0 and float(v[1000]) == 0.0
