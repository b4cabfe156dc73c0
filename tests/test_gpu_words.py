"""GPU parity through the reference-facing interface: the words machine runs the generated
model scripts (same words, tensor names and operator order as the reference's train.words) on
device tensors, and the results are compared with the CPU oracle.

Configuration of the main case: one BLOOM decoder layer forward + backward in fp32, hidden 1024,
16 heads x 64, MLP 4096, batch 2, seq 128, valid lengths uniform in [64,128], weights N(0,0.02),
biases 0, LayerNorm gamma 1 / beta 0, inputs and upstream gradient N(0,1), seed 0.
Tolerance: max |err| / max |ref| <= 1e-4 per tensor (fp32 kernels)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL32 = 1e-4


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


def make_layer(rng, hidden, trained_ln=False):
    p = {}
    for name in orc.LAYER_PARAMS:
        if name.endswith("layernorm.weight"):
            p[name] = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32) if trained_ln else np.ones(hidden, np.float32)
        elif name.endswith("layernorm.bias"):
            p[name] = (0.1 * rng.standard_normal(hidden)).astype(np.float32) if trained_ln else np.zeros(hidden, np.float32)
        elif name.endswith(".bias"):
            n = {"query_key_value": 3, "dense_h_to_4h": 4}.get(name.split(".")[0], 1) * hidden
            p[name] = (0.02 * rng.standard_normal(n)).astype(np.float32) if trained_ln else np.zeros(n, np.float32)
        else:
            o, i = {"query_key_value.weight": (3, 1), "dense.weight": (1, 1), "dense_h_to_4h.weight": (4, 1),
                    "dense_4h_to_h.weight": (1, 4)}[name]
            p[name] = (0.02 * rng.standard_normal((o * hidden, i * hidden))).astype(np.float32)
    return p


def run_layer_case(host, B, T, H, heads, lens, seed, trained_ln):
    from blackriver_b200 import words
    rng = np.random.default_rng(seed)
    p = make_layer(rng, H, trained_ln)
    x = rng.standard_normal((B, T, H)).astype(np.float32)
    dy = rng.standard_normal((B, T, H)).astype(np.float32)
    mask = np.zeros((B, T), np.int32)
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    al = orc.alibi(heads, T)
    xm = orc.build_xmask(mask)
    out_ref, saved = orc.layer_forward(x, p, al, xm, heads)
    dx_ref, g_ref = orc.layer_backward(dy, p, saved, heads)

    env = host.Env(2)
    try:
        env.execute(words.init_words(hidden=H, heads=heads, vocab=64, dtype="float", max_tokens=max(B * T, 64)))
        env.execute(words.train_words())
        env.execute('"cuda" $DEVICE ! create_layer_weight create_layer_grad zero_layer_grad')
        env.execute(f"{words.var_elements(B, T, H, heads, 64, 4)} create_var  {B} {T} create_dynamic")
        for k, v in p.items():
            env.write(k, v)
        env.write("xinput", x)
        env.write("yout_g", dy)
        env.write("alibi", al)
        env.write("xmask", xm)
        env.execute("layer_forward op.sync")
        assert relerr(env.read("xa"), out_ref) <= TOL32
        assert relerr(env.read("xll"), saved["xll"]) <= TOL32
        env.execute("layer_backward op.sync")
        assert relerr(env.read("xa"), dx_ref) <= TOL32
        for k in orc.LAYER_PARAMS:
            assert relerr(env.read(k + "_g"), g_ref[k + "_g"]) <= TOL32, k
    finally:
        env.close()


def test_decoder_layer_fp32_parity_config(host):
    rng = np.random.default_rng(0)
    lens = rng.integers(64, 129, 2).tolist()
    run_layer_case(host, B=2, T=128, H=1024, heads=16, lens=lens, seed=0, trained_ln=False)


def test_decoder_layer_small_trained_layernorm_and_short_rows(host):
    run_layer_case(host, B=3, T=20, H=64, heads=8, lens=(20, 1, 13), seed=1, trained_ln=True)


def test_decoder_layer_fp16_storage(host):
    """Same layer in fp16 storage (tensor-core GEMMs for the linear layers) against the fp32 oracle:
    <= 2e-2 on activations and gradients."""
    from blackriver_b200 import words
    B, T, H, heads = 2, 128, 1024, 16
    rng = np.random.default_rng(3)
    p = make_layer(rng, H, trained_ln=False)
    r16 = lambda a: a.astype(np.float16).astype(np.float32)
    p = {k: r16(v) for k, v in p.items()}
    x = r16(rng.standard_normal((B, T, H)).astype(np.float32))
    dy = r16(rng.standard_normal((B, T, H)).astype(np.float32))
    mask = np.zeros((B, T), np.int32); mask[0, :128] = 1; mask[1, :77] = 1
    al = orc.alibi(heads, T); xm = orc.build_xmask(mask)
    out_ref, saved = orc.layer_forward(x, p, al, xm, heads)
    dx_ref, g_ref = orc.layer_backward(dy, p, saved, heads)
    env = host.Env(1)
    try:
        env.execute(words.init_words(hidden=H, heads=heads, vocab=64, dtype="half", max_tokens=256))
        env.execute(words.train_words())
        env.execute('"cuda" $DEVICE ! create_layer_weight create_layer_grad')
        env.execute(f"{words.var_elements(B, T, H, heads, 64, 4)} create_var  {B} {T} create_dynamic")
        for k, v in p.items():
            env.write(k, v)
        env.write("xinput", x); env.write("yout_g", dy); env.write("alibi", al)
        env.write("xmask", np.maximum(xm, -60000.0))      # -FLT_MAX does not exist in fp16
        env.execute("layer_forward op.sync")
        assert relerr(env.read("xa"), out_ref) <= 2e-2
        env.execute("layer_backward op.sync")
        assert relerr(env.read("xa"), dx_ref) <= 2e-2
        for k in orc.LAYER_PARAMS:
            assert relerr(env.read(k + "_g"), g_ref[k + "_g"]) <= 2e-2, k
    finally:
        env.close()


def test_golden_block_through_words(host, golden_dir):
    """The fixture produced by the reference's PyTorch BloomBlock, replayed through the words."""
    import os
    from blackriver_b200 import words
    g = dict(np.load(os.path.join(golden_dir, "block_small.npz")))
    heads = int(g["heads"])
    B, T, H = g["x"].shape
    env = host.Env(1)
    try:
        env.execute(words.init_words(hidden=H, heads=heads, vocab=64, dtype="float", max_tokens=64))
        env.execute(words.train_words())
        env.execute('"cuda" $DEVICE ! create_layer_weight create_layer_grad')
        env.execute(f"{words.var_elements(B, T, H, heads, 64, 4)} create_var  {B} {T} create_dynamic")
        for k in orc.LAYER_PARAMS:
            env.write(k, g["p." + k])
        env.write("xinput", g["x"]); env.write("yout_g", g["dy"])
        env.write("alibi", orc.alibi(heads, T)); env.write("xmask", orc.build_xmask(g["mask"]))
        env.execute("layer_forward op.sync")
        assert relerr(env.read("xa"), g["out"]) <= TOL32
        env.execute("layer_backward op.sync")
        assert relerr(env.read("xa"), g["dx"]) <= TOL32
        for k in orc.LAYER_PARAMS:
            assert relerr(env.read(k + "_g"), g["g." + k]) <= TOL32, k
    finally:
        env.close()


def test_loss_backward_word(host):
    """ln_f + op.loss_backward + ln_f backward, the tail of the reference's train_0 word
    (bloomz-7b/train.words:305-318), against the oracle; ids/mask stay on the host as there."""
    from blackriver_b200 import words
    rng = np.random.default_rng(5)
    B, T, H, V = 2, 24, 64, 520
    x = rng.standard_normal((B, T, H)).astype(np.float32)
    w = (0.3 * rng.standard_normal((V, H))).astype(np.float32)
    ids = rng.integers(0, V, (B, T)).astype(np.int32)
    mask = np.zeros((B, T), np.int32); mask[0, :24] = 1; mask[1, :9] = 1
    gamma = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32); beta = (0.1 * rng.standard_normal(H)).astype(np.float32)
    xb_ref, _, var_ref = orc.layernorm(x, gamma, beta)
    wg0 = rng.standard_normal((V, H)).astype(np.float32)
    loss_ref, xg_ref, wg_ref = orc.loss_backward(xb_ref, ids, mask, w, w_g=wg0.copy())
    dg_ref, db_ref, dx_ref = orc.layernorm_backward(xg_ref, gamma, beta, var_ref, xb_ref)

    env = host.Env(1)
    try:
        env.execute(words.init_words(hidden=H, heads=4, vocab=V, dtype="float", max_tokens=64))
        env.execute(words.train_words())
        env.execute("create_main_weight create_main_grad zero_main_grad")
        # a logits band of 7 rows forces several bands per sequence
        env.execute(f"{words.var_elements(B, T, H, 4, V, 7)} create_var  {B} {T} create_dynamic")
        env.write("ln_f.weight", gamma); env.write("ln_f.bias", beta); env.write("lm_head.weight", w)
        env.write("lm_head.weight_g", wg0)
        env.write("xa", x); env.write("ids_", ids); env.write("mask_", mask)
        env.execute('"xa" @ "ln_mean" @ "post_ln_var" @ "ln_f.weight" @ "ln_f.bias" @ "xb" @ "LN_EPS" @ op.layernorm')
        env.execute('"xb" @ "ids_" @ "mask_" @ "lm_head.weight" @ "all_logits" @ "xa" @ "lm_head.weight_g" @ op.loss_backward')
        env.execute('"xa" @ "ln_f.weight" @ "ln_f.bias" @ "post_ln_var" @ "xb" @ "ln_f.weight_g" @ "ln_f.bias_g" @ "xc" @ "LN_EPS" @ op.layernorm_backward op.sync')
        assert abs(host.last_loss() - loss_ref) <= TOL32 * abs(loss_ref)
        assert relerr(env.read("xa"), xg_ref) <= TOL32
        assert relerr(env.read("lm_head.weight_g"), wg_ref) <= TOL32      # accumulated onto the previous value
        assert relerr(env.read("xc"), dx_ref) <= TOL32
        assert relerr(env.read("ln_f.weight_g"), dg_ref) <= TOL32 and relerr(env.read("ln_f.bias_g"), db_ref) <= TOL32
        # the same backward with the residual branch folded in: din = residual + input gradient
        env.execute('"xa" @ "ln_f.weight" @ "ln_f.bias" @ "post_ln_var" @ "xb" @ "ln_f.weight_g" @ "ln_f.bias_g" @ "xc" @ "xb" @ "LN_EPS" @ '
                    'op.layernorm_backward_residual op.sync')
        assert relerr(env.read("xc"), dx_ref + xb_ref) <= TOL32
        assert relerr(env.read("ln_f.weight_g"), dg_ref) <= TOL32
    finally:
        env.close()


def test_async_loss_word_matches_the_blocking_one(host):
    """op.loss_backward_async (no host round trip: the count of targets, the gradient factor and the mean loss stay on
    the device) against the oracle, with the weight gradient taken at once and deferred to op.loss_backward_w."""
    rng = np.random.default_rng(8)
    B, T, H, V = 2, 24, 64, 520
    x = (0.5 * rng.standard_normal((B, T, H))).astype(np.float32)
    w = (0.3 * rng.standard_normal((V, H))).astype(np.float32)
    ids = rng.integers(0, V, (B, T)).astype(np.int32)
    mask = np.zeros((B, T), np.int32); mask[0, :24] = 1; mask[1, :9] = 1
    wg0 = rng.standard_normal((V, H)).astype(np.float32)
    loss_ref, xg_ref, wg_ref = orc.loss_backward(x, ids, mask, w, w_g=wg0.copy())
    env = host.Env(1)
    try:
        env.execute(f'{B} {T} {H} 3 "cuda" "float" op.create "x" !  {B} {T} {H} 3 "cuda" "float" op.create "x_g" !')
        env.execute(f'{V} {H} 2 "cuda" "float" op.create "w" !  {V} {H} 2 "cuda" "float" op.create "w_g" !')
        env.execute(f'{B} {T} 2 "cuda" "int" op.create "ids" !  {B} {T} 2 "cuda" "int" op.create "mask" !  1 1 "cuda" "float" op.create "loss" !')
        env.execute(f'{B * T} {V} 2 "cuda" "float" op.create "band_all" !  7 {V} 2 "cuda" "float" op.create "band_7" !')
        env.write("x", x); env.write("w", w); env.write("ids", ids); env.write("mask", mask)
        for band, defer in (("band_7", 0), ("band_all", 0), ("band_all", 1)):
            env.write("w_g", wg0); env.write("loss", np.zeros(1, np.float32))
            env.execute(f'"x" @ "ids" @ "mask" @ "w" @ "{band}" @ "x_g" @ "w_g" @ "loss" @ {defer} op.loss_backward_async op.sync')
            assert abs(float(env.read("loss")[0]) - loss_ref) <= TOL32 * abs(loss_ref)
            assert relerr(env.read("x_g"), xg_ref) <= TOL32
            if defer:
                assert np.array_equal(env.read("w_g"), wg0)                    # untouched until the deferred pass
                env.execute(f'"{band}" @ "x" @ "w_g" @ op.loss_backward_w op.sync')
            assert relerr(env.read("w_g"), wg_ref) <= TOL32
        # all positions masked out: zero loss, zero gradients, nothing divided by zero
        env.write("mask", np.zeros((B, T), np.int32)); env.write("w_g", wg0)
        env.execute('"x" @ "ids" @ "mask" @ "w" @ "band_all" @ "x_g" @ "w_g" @ "loss" @ 0 op.loss_backward_async op.sync')
        assert float(env.read("loss")[0]) == 0.0 and not env.read("x_g").any() and np.array_equal(env.read("w_g"), wg0)
    finally:
        env.close()


def test_split_linear_backward_equals_the_whole(host):
    rng = np.random.default_rng(9)
    n, i, o = 48, 64, 96
    env = host.Env(1)
    try:
        for name, shape in (("dy", (n, o)), ("x", (n, i)), ("w", (o, i)), ("b", (o,)), ("xg1", (n, i)), ("xg2", (n, i)), ("wg1", (o, i)),
                            ("wg2", (o, i)), ("bg1", (o,)), ("bg2", (o,))):
            env.execute(" ".join(str(d) for d in shape) + f' {len(shape)} "cuda" "float" op.create "{name}" !')
        for name in ("dy", "x", "w", "b"):
            env.write(name, rng.standard_normal(env.tensor_info(name)["shape"]).astype(np.float32))
        env.execute('"dy" @ "x" @ "w" @ "b" @ "xg1" @ "wg1" @ "bg1" @ op.linear_backward')
        env.execute('"dy" @ "w" @ "xg2" @ op.linear_backward_x  "dy" @ "x" @ "wg2" @ "bg2" @ op.linear_backward_w  op.sync')
        for a, b in (("xg1", "xg2"), ("wg1", "wg2"), ("bg1", "bg2")):
            assert np.array_equal(env.read(a), env.read(b))
        xg_ref, wg_ref, bg_ref = orc.linear_backward(env.read("dy"), env.read("x"), env.read("w"))
        assert relerr(env.read("xg2"), xg_ref) <= TOL32 and relerr(env.read("wg2"), wg_ref) <= TOL32 and relerr(env.read("bg2"), bg_ref) <= TOL32
    finally:
        env.close()


def test_last_logits_on_the_device(host):
    """op.last_logits (blackriver/cuda_tensor.cpp:415-462): the row before the first padded position, and -- the
    reference's rule for a row without padding -- token 0; fp32 and fp16 tensors against the oracle."""
    rng = np.random.default_rng(10)
    B, T, H, V = 3, 16, 64, 200
    x = rng.standard_normal((B, T, H)).astype(np.float32)
    w = (0.2 * rng.standard_normal((V, H))).astype(np.float32)
    mask = np.zeros((B, T), np.int32); mask[0, :5] = 1; mask[1, :] = 1; mask[2, :1] = 1
    ref = orc.last_logits(x, mask, w)
    assert np.allclose(ref[1], x[1, 0] @ w.T, atol=1e-4)                     # a full row reads token 0, as the reference does
    assert np.allclose(ref[0], x[0, 4] @ w.T, atol=1e-4)
    env = host.Env(1)
    try:
        env.execute(f'{B} {T} 2 "cpu" "int" op.create "mask" !')
        env.write("mask", mask)
        for dt, tol in (("float", TOL32), ("half", 2e-2)):
            env.execute(f'{B} {T} {H} 3 "cuda" "{dt}" op.create "x" !  {V} {H} 2 "cuda" "{dt}" op.create "w" !  {B} {V} 2 "cuda" "{dt}" op.create "out" !')
            env.write("x", x); env.write("w", w)
            env.execute('"x" @ "mask" @ "w" @ "out" @ op.last_logits op.sync')
            xr, wr = env.read("x").astype(np.float32), env.read("w").astype(np.float32)
            assert relerr(env.read("out"), orc.last_logits(xr, mask, wr)) <= tol, dt
    finally:
        env.close()


def test_device_save_and_load_round_trip(host, tmp_path):
    """io.save / io.load of device tensors (blackriver/cuda_tensor.cpp:57-72): raw little-endian files; an fp16 tensor
    also accepts an fp32 file of the same element count, as the weight dumps are fp32."""
    rng = np.random.default_rng(11)
    a = rng.standard_normal((6, 40)).astype(np.float32)
    env = host.Env(1)
    try:
        env.execute('6 40 2 "cuda" "float" op.create "f" !  6 40 2 "cuda" "float" op.create "f2" !')
        env.execute('6 40 2 "cuda" "half" op.create "h" !  6 40 2 "cuda" "half" op.create "h2" !')
        env.write("f", a); env.write("h", a)
        pf, ph = str(tmp_path / "f.bin"), str(tmp_path / "h.bin")
        env.execute(f'"f" @ "{pf}" io.save  "h" @ "{ph}" io.save')
        assert np.array_equal(np.fromfile(pf, np.float32).reshape(6, 40), a)
        assert np.array_equal(np.fromfile(ph, np.float16).reshape(6, 40), a.astype(np.float16))
        env.execute(f'"f2" @ "{pf}" io.load  "h2" @ "{ph}" io.load op.sync')
        assert np.array_equal(env.read("f2"), a) and np.array_equal(env.read("h2"), a.astype(np.float16))
        env.execute(f'"h2" @ op.zero  "h2" @ "{pf}" io.load op.sync')              # fp32 file into an fp16 tensor
        assert np.array_equal(env.read("h2"), a.astype(np.float16))
    finally:
        env.close()
