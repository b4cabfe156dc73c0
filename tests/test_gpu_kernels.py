"""GPU parity tests: every CUDA kernel, called through the C ABI, against the CPU oracle on the
same seeded inputs.

Tolerances (from the task statement): fp32 kernels max |err| / max |ref| <= 1e-4; fp16 storage
<= 2e-2 on activations and gradients; integer / index / byte work bit-exact.  The error is
normalised by the largest reference magnitude because the tensors contain entries near zero.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TOL32 = 1e-4
TOL16 = 2e-2


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from blackriver_b200 import ops as _ops
    return _ops


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.detach().float().cpu().numpy() if t.dtype.is_floating_point else t.detach().cpu().numpy()


def relerr(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def h16(a):
    """Round to fp16 and back so oracle and kernel see identical inputs."""
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,hidden", [(256, 1024), (37, 4096), (5, 64), (3, 100), (1, 7), (9, 8192), (2, 16384)])
def test_layernorm_fwd_bwd_f32(ops, rows, hidden):
    rng = np.random.default_rng(rows * 7 + hidden)
    x = rng.standard_normal((rows, hidden)).astype(np.float32) * 1.5 + 0.3
    gamma = (1.0 + 0.2 * rng.standard_normal(hidden)).astype(np.float32)
    beta = (0.2 * rng.standard_normal(hidden)).astype(np.float32)
    dy = rng.standard_normal((rows, hidden)).astype(np.float32)
    y_ref, mean_ref, var_ref = orc.layernorm(x, gamma, beta, 1e-5)
    y, mean, var = ops.layernorm(dev(x), dev(gamma), dev(beta), 1e-5)
    assert relerr(host(y), y_ref) <= TOL32
    assert relerr(host(mean), mean_ref) <= TOL32
    assert relerr(host(var), var_ref) <= TOL32
    dg_ref, db_ref, dx_ref = orc.layernorm_backward(dy, gamma, beta, var_ref, y_ref, 1e-5)
    dg, db, dx = ops.layernorm_backward(dev(dy), dev(gamma), dev(beta), dev(var_ref), dev(y_ref), 1e-5)
    assert relerr(host(dx), dx_ref) <= TOL32
    assert relerr(host(dg), dg_ref) <= TOL32
    assert relerr(host(db), db_ref) <= TOL32


@pytest.mark.parametrize("rows,hidden", [(512, 4096), (33, 1024), (4, 72), (3, 50)])
def test_layernorm_fwd_bwd_f16(ops, rows, hidden):
    rng = np.random.default_rng(rows + hidden)
    x = h16(rng.standard_normal((rows, hidden)))
    gamma = h16(1.0 + 0.1 * rng.standard_normal(hidden))
    beta = h16(0.1 * rng.standard_normal(hidden))
    dy = h16(rng.standard_normal((rows, hidden)))
    y_ref, mean_ref, var_ref = orc.layernorm(x, gamma, beta, 1e-5)
    f16 = torch.float16
    y, mean, var = ops.layernorm(dev(x, f16), dev(gamma, f16), dev(beta, f16), 1e-5)
    assert relerr(host(y), y_ref) <= TOL16
    assert relerr(host(var), var_ref) <= 1e-3
    # backward consumes the fp16 LN output, as the operator interface prescribes
    y16 = host(y)
    dg_ref, db_ref, dx_ref = orc.layernorm_backward(dy, gamma, beta, var_ref, y16, 1e-5)
    dg, db, dx = ops.layernorm_backward(dev(dy, f16), dev(gamma, f16), dev(beta, f16), dev(var_ref), y, 1e-5)
    assert relerr(host(dx), dx_ref) <= TOL16
    assert relerr(host(dg), dg_ref) <= TOL16
    assert relerr(host(db), db_ref) <= TOL16


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("rows,hidden,dtype", [(6001, 4096, "f16"), (300, 2056, "f16"), (2500, 1024, "f32"), (151, 4096, "f32"),
                                                (297, 8192, "f16"), (1, 4096, "f16")])
def test_layernorm_ring_and_register_kernels(ops, mode, rows, hidden, dtype):
    """Rows of 2 KiB and more are prefetched through shared memory (mode 0) or held in registers only
    (mode 1); row counts that wrap the prefetch ring several times per CTA, odd counts, packet counts that
    are not a multiple of the warp size, in-place outputs."""
    from blackriver_b200 import brk
    rng = np.random.default_rng(rows + hidden)
    rnd = h16 if dtype == "f16" else (lambda a: np.asarray(a, np.float32))
    td = torch.float16 if dtype == "f16" else torch.float32
    tol = TOL16 if dtype == "f16" else TOL32
    x = rnd(rng.standard_normal((rows, hidden)) * 1.3 + 0.2)
    gamma = rnd(1.0 + 0.1 * rng.standard_normal(hidden))
    beta = rnd(0.1 * rng.standard_normal(hidden))
    dy = rnd(rng.standard_normal((rows, hidden)))
    y_ref, mean_ref, var_ref = orc.layernorm(x, gamma, beta, 1e-5)
    assert brk.raw("brk_layernorm_set_mode", mode) == 0
    try:
        xd = dev(x, td)
        y, mean, var = ops.layernorm(xd, dev(gamma, td), dev(beta, td), 1e-5, out=xd)      # in place
        assert relerr(host(y), y_ref) <= tol
        assert relerr(host(mean), mean_ref) <= 1e-3 and relerr(host(var), var_ref) <= 1e-3
        yin = host(y)
        dg_ref, db_ref, dx_ref = orc.layernorm_backward(dy, gamma, beta, var_ref, yin, 1e-5)
        dyd = dev(dy, td)
        dg, db, dx = ops.layernorm_backward(dyd, dev(gamma, td), dev(beta, td), dev(var_ref), y, 1e-5, dx=dyd)      # dx over dy
        assert relerr(host(dx), dx_ref) <= tol
        # column sums over thousands of rows, rounded to the tensor's type at the end
        assert relerr(host(dg), dg_ref) <= tol and relerr(host(db), db_ref) <= tol
    finally:
        brk.raw("brk_layernorm_set_mode", 0)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("rows,hidden,dtype", [(2048, 4096, "f16"), (301, 2056, "f16"), (37, 1024, "f32"), (9, 8192, "f16"), (5, 100, "f32")])
def test_layernorm_backward_with_residual(ops, mode, rows, hidden, dtype):
    """dx = residual + the LayerNorm's input gradient (the residual branch of the block folded into the kernel), in every
    kernel variant; also with the residual buffer as the output."""
    from blackriver_b200 import brk
    rng = np.random.default_rng(rows * 3 + hidden)
    rnd = h16 if dtype == "f16" else (lambda a: np.asarray(a, np.float32))
    td = torch.float16 if dtype == "f16" else torch.float32
    tol = TOL16 if dtype == "f16" else TOL32
    x = rnd(rng.standard_normal((rows, hidden)) * 1.3 + 0.2)
    gamma = rnd(1.0 + 0.1 * rng.standard_normal(hidden))
    beta = rnd(0.1 * rng.standard_normal(hidden))
    dy = rnd(rng.standard_normal((rows, hidden)))
    res = rnd(rng.standard_normal((rows, hidden)))
    y_ref, _, var_ref = orc.layernorm(x, gamma, beta, 1e-5)
    yin = rnd(y_ref)
    dg_ref, db_ref, dx_ref = orc.layernorm_backward(dy, gamma, beta, var_ref, yin, 1e-5)
    want = dx_ref.astype(np.float32) + res.astype(np.float32)
    assert brk.raw("brk_layernorm_set_mode", mode) == 0
    try:
        resd = dev(res, td)
        dg, db, dx = ops.layernorm_backward(dev(dy, td), dev(gamma, td), dev(beta, td), dev(var_ref), dev(yin, td), 1e-5, residual=resd)
        assert relerr(host(dx), want) <= tol
        assert relerr(host(dg), dg_ref) <= tol and relerr(host(db), db_ref) <= tol
        assert np.array_equal(host(resd), res)          # the residual itself is left alone
        _, _, dx2 = ops.layernorm_backward(dev(dy, td), dev(gamma, td), dev(beta, td), dev(var_ref), dev(yin, td), 1e-5, residual=resd, dx=resd)
        assert np.array_equal(host(dx2), host(dx))      # residual buffer as the output: same values
    finally:
        brk.raw("brk_layernorm_set_mode", 0)


def test_layernorm_unaligned_views_and_inplace(ops):
    rng = np.random.default_rng(5)
    rows, hidden = 6, 256
    buf = dev(rng.standard_normal(rows * hidden + 3).astype(np.float32))
    x = buf[3:].view(rows, hidden)          # 12-byte offset: the vector path must not be taken
    gamma = dev(np.ones(hidden, np.float32)); beta = dev(np.zeros(hidden, np.float32))
    y_ref, _, var_ref = orc.layernorm(host(x), host(gamma), host(beta))
    y, _, var = ops.layernorm(x, gamma, beta, out=x)   # in place
    assert relerr(host(y), y_ref) <= TOL32
    dy = dev(rng.standard_normal((rows, hidden)).astype(np.float32))
    dg_ref, db_ref, dx_ref = orc.layernorm_backward(host(dy), host(gamma), host(beta), var_ref, y_ref)
    dg, db, dx = ops.layernorm_backward(dy, gamma, beta, var, y, dx=dy)   # dx over dy
    assert relerr(host(dx), dx_ref) <= TOL32 and relerr(host(dg), dg_ref) <= TOL32


def test_layernorm_backward_accumulate(ops):
    rng = np.random.default_rng(6)
    rows, hidden = 64, 1024
    x = rng.standard_normal((rows, hidden)).astype(np.float32)
    gamma = np.ones(hidden, np.float32); beta = np.zeros(hidden, np.float32)
    dy = rng.standard_normal((rows, hidden)).astype(np.float32)
    y_ref, _, var_ref = orc.layernorm(x, gamma, beta)
    dg_ref, db_ref, _ = orc.layernorm_backward(dy, gamma, beta, var_ref, y_ref)
    dg = dev(np.full(hidden, 2.0, np.float32)); db = dev(np.full(hidden, -1.0, np.float32))
    ops.layernorm_backward(dev(dy), dev(gamma), dev(beta), dev(var_ref), dev(y_ref), dgamma=dg, dbeta=db, accumulate=True)
    assert relerr(host(dg), dg_ref + 2.0) <= TOL32 and relerr(host(db), db_ref - 1.0) <= TOL32


# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [256 * 4096, 1000003, 5, 1])
def test_gelu_f32(ops, n):
    rng = np.random.default_rng(n % 1000)
    x = (rng.standard_normal(n) * 3).astype(np.float32)
    dy = rng.standard_normal(n).astype(np.float32)
    assert relerr(host(ops.gelu(dev(x))), orc.gelu(x)) <= TOL32
    assert relerr(host(ops.gelu_backward(dev(dy), dev(x))), orc.gelu_backward(dy, x)) <= TOL32


def test_gelu_f16_and_inplace(ops):
    rng = np.random.default_rng(2)
    x = h16(rng.standard_normal(8 * 4096 + 5) * 2)
    dy = h16(rng.standard_normal(x.size))
    f16 = torch.float16
    assert relerr(host(ops.gelu(dev(x, f16))), orc.gelu(x)) <= TOL16
    xd = dev(x, f16)
    out = ops.gelu_backward(dev(dy, f16), xd, out=xd)   # x_g over x, as the layer_backward word does
    assert out.data_ptr() == xd.data_ptr()
    assert relerr(host(out), orc.gelu_backward(dy, x)) <= TOL16


def test_gelu_extremes(ops):
    x = np.array([0.0, -0.0, 1e-6, -1e-6, 10.0, -10.0, 50.0, -50.0, 1e4, -1e4], np.float32)
    y = host(ops.gelu(dev(x)))
    assert np.isfinite(y).all()
    np.testing.assert_allclose(y, orc.gelu(x), rtol=1e-5, atol=1e-6)
    g = host(ops.gelu_backward(dev(np.ones_like(x)), dev(x)))
    assert np.isfinite(g).all()
    np.testing.assert_allclose(g, orc.gelu_backward(np.ones_like(x), x), rtol=1e-4, atol=1e-6)


# ------------------------------------------------------------------------------------------
def _nll_case(rng, rows, vocab, sigma=2.0, frac_masked=0.1):
    logits = (rng.standard_normal((rows, vocab)) * sigma).astype(np.float32)
    target = rng.integers(0, vocab, rows).astype(np.int32)
    target[rng.random(rows) < frac_masked] = -100
    return logits, target


@pytest.mark.parametrize("rows,vocab", [(64, 250880), (7, 1001), (3, 40), (2, 8), (300, 4096)])
def test_nll_f32(ops, rows, vocab):
    rng = np.random.default_rng(rows + vocab)
    logits, target = _nll_case(rng, rows, vocab)
    if rows >= 3:
        target[0] = -100; target[1] = vocab - 1; target[2] = 0
    n = max(int((target >= 0).sum()), 1)
    total_ref, rl_ref, dl_ref = orc.logsoftmax_nll(logits, target, grad_scale=1.0 / n)
    rl = ops.logsoftmax_nll(dev(logits), dev(target))
    assert relerr(host(rl), rl_ref) <= TOL32
    rl2, dl = ops.logsoftmax_nll_backward(dev(logits), dev(target), 1.0 / n)
    assert relerr(host(rl2), rl_ref) <= TOL32
    assert relerr(host(dl), dl_ref) <= TOL32
    assert (host(dl)[target < 0] == 0).all() and (host(rl)[target < 0] == 0).all()
    total = float(host(ops.sum_f32(rl))[0])
    assert abs(total - total_ref) <= 1e-4 * abs(total_ref) + 1e-6


@pytest.mark.parametrize("rows,vocab", [(48, 250880), (5, 1000)])
def test_nll_f16_inplace_gradient(ops, rows, vocab):
    rng = np.random.default_rng(11)
    logits, target = _nll_case(rng, rows, vocab)
    logits = h16(logits)
    n = max(int((target >= 0).sum()), 1)
    total_ref, rl_ref, dl_ref = orc.logsoftmax_nll(logits, target, grad_scale=1.0)
    z = dev(logits, torch.float16)
    rl, dl = ops.logsoftmax_nll_backward(z, dev(target), 1.0, dlogits=z)   # gradient over the logits
    assert dl.data_ptr() == z.data_ptr()
    assert abs(float(host(rl).sum()) - total_ref) <= 1e-3 * abs(total_ref)   # loss: 1e-3 relative
    assert relerr(host(dl), dl_ref) <= TOL16


def test_loss_targets_bit_exact(ops):
    rng = np.random.default_rng(3)
    b, t = 4, 512
    ids = rng.integers(0, 250880, (b, t)).astype(np.int32)
    lens = [512, 1, 300, 0]
    mask = np.zeros((b, t), np.int32)
    for i, n in enumerate(lens):
        mask[i, :n] = 1
    mask[2, 100] = 0   # a hole: not right-padded
    tg_ref, items_ref = orc.loss_targets(ids, mask)
    tg, cnt = ops.loss_targets(dev(ids), dev(mask))
    assert host(tg).tobytes() == tg_ref.tobytes()
    assert int(host(cnt)[0]) == items_ref


# ------------------------------------------------------------------------------------------
def test_alibi_and_mask_bit_exact(ops):
    for heads, t in ((16, 128), (32, 512), (4, 5)):
        assert host(ops.alibi(heads, t)).tobytes() == orc.alibi(heads, t).tobytes()
    rng = np.random.default_rng(4)
    b, t = 3, 77
    mask = np.zeros((b, t), np.int32)
    mask[0, :77] = 1; mask[1, :20] = 1; mask[2, :50] = 1; mask[2, 10] = 0
    assert host(ops.xmask(dev(mask))).tobytes() == orc.build_xmask(mask).tobytes()


def test_gather_bit_exact(ops):
    rng = np.random.default_rng(8)
    for dtype, h in ((np.float32, 1024), (np.float16, 4096), (np.float32, 30)):
        table = rng.standard_normal((500, h)).astype(dtype)
        ids = rng.integers(0, 500, (2, 33)).astype(np.int32)
        out = ops.embedding_gather(dev(table), dev(ids))
        assert out.cpu().numpy().tobytes() == table[ids].tobytes()


def test_add_transpose_colsum_softmax(ops):
    rng = np.random.default_rng(9)
    b, h, t, d = 2, 4, 24, 16
    s = rng.standard_normal((b, h, t, t)).astype(np.float32)
    al = rng.standard_normal((1, h, 1, t)).astype(np.float32)
    xm = rng.standard_normal((b, 1, t, t)).astype(np.float32)
    sd = dev(s)
    ops.add(sd, dev(al), out=sd)
    ops.add(sd, dev(xm), out=sd)
    ref = orc.add_bcast(orc.add_bcast(s, al), xm)
    assert host(sd).tobytes() == ref.tobytes()
    a = rng.standard_normal((3, 5, 7)).astype(np.float32)
    assert host(ops.add(dev(a), dev(a * 2))).tobytes() == (a + a * 2).tobytes()
    x = rng.standard_normal((b, t, h, d)).astype(np.float32)
    assert host(ops.transpose_0213(dev(x))).tobytes() == orc.transpose_0213(x).tobytes()
    x3 = rng.standard_normal((2, 3, 5, 3)).astype(np.float32)
    assert host(ops.transpose_0213(dev(x3))).tobytes() == orc.transpose_0213(x3).tobytes()
    m = rng.standard_normal((300, 70)).astype(np.float32)
    assert relerr(host(ops.colsum(dev(m))), m.sum(0)) <= TOL32
    p_ref = orc.softmax(ref)
    p = ops.softmax(sd, out=sd)
    assert relerr(host(p), p_ref) <= TOL32
    g = rng.standard_normal(s.shape).astype(np.float32)
    assert relerr(host(ops.softmax_backward(dev(g), p)), orc.softmax_backward(g, p_ref)) <= TOL32


def test_cast_and_fill(ops):
    rng = np.random.default_rng(10)
    x = rng.standard_normal(1001).astype(np.float32)
    assert host(ops.cast(dev(x), torch.float16)).tobytes() == x.astype(np.float16).astype(np.float32).tobytes()
    t = torch.empty(77, dtype=torch.float32, device="cuda")
    assert (host(ops.fill(t, 1.5)) == 1.5).all() and (host(ops.fill(t, 0.0)) == 0).all()


# ------------------------------------------------------------------------------------------
def test_gemm_variants_f32(ops):
    rng = np.random.default_rng(12)
    for (m, n, k) in ((64, 64, 16), (70, 33, 19), (1, 5, 300), (130, 257, 64)):
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((k, n)).astype(np.float32)
        ref = a.astype(np.float64) @ b.astype(np.float64)
        for ta in (False, True):
            for tb in (False, True):
                A = dev(a.T.copy() if ta else a)
                B = dev(b.T.copy() if tb else b)
                C = torch.empty((m, n), dtype=torch.float32, device="cuda")
                ops.gemm(A, B, C, m, n, k, ta, tb, A.shape[1], B.shape[1], n)
                assert relerr(host(C), ref) <= TOL32, (m, n, k, ta, tb)


def test_linear_and_attention_ops_f32(ops):
    rng = np.random.default_rng(13)
    n, i, o = 48, 96, 160
    x = rng.standard_normal((2, n // 2, i)).astype(np.float32)
    w = (rng.standard_normal((o, i)) * 0.1).astype(np.float32)
    bias = rng.standard_normal(o).astype(np.float32)
    dy = rng.standard_normal((2, n // 2, o)).astype(np.float32)
    assert relerr(host(ops.linear(dev(x), dev(w), dev(bias))), orc.linear(x, w, bias)) <= TOL32
    xg_ref, wg_ref, bg_ref = orc.linear_backward(dy, x, w)
    xd = dev(np.concatenate([x, np.zeros((2, n // 2, o - i), np.float32)], -1))[..., :i].contiguous()
    xg, wg, bg = ops.linear_backward(dev(dy), xd, dev(w), x_g=xd)     # x_g over x
    assert relerr(host(xg), xg_ref) <= TOL32 and relerr(host(wg), wg_ref) <= TOL32 and relerr(host(bg), bg_ref) <= TOL32
    b, h, t, d = 2, 3, 20, 16
    q = rng.standard_normal((b, h, t, d)).astype(np.float32)
    k = rng.standard_normal((b, h, t, d)).astype(np.float32)
    v = rng.standard_normal((b, h, t, d)).astype(np.float32)
    s_ref = orc.qk(q, k)
    assert relerr(host(ops.qk(dev(q), dev(k))), s_ref) <= TOL32
    p_ref = orc.softmax(s_ref)
    assert relerr(host(ops.attn(dev(p_ref), dev(v))), orc.attn(p_ref, v)) <= TOL32
    do = rng.standard_normal((b, h, t, d)).astype(np.float32)
    ds_ref, dv_ref = orc.softmax_attn_backward(do, p_ref, v)
    pd = dev(p_ref)
    ds, dv = ops.softmax_attn_backward(dev(do), pd, dev(v), ds=pd)     # dS over P
    assert relerr(host(ds), ds_ref) <= TOL32 and relerr(host(dv), dv_ref) <= TOL32
    dq_ref, dk_ref = orc.qk_backward(ds_ref, q, k)
    dq, dk = ops.qk_backward(dev(ds_ref), dev(q), dev(k))
    assert relerr(host(dq), dq_ref) <= TOL32 and relerr(host(dk), dk_ref) <= TOL32


def test_error_codes_on_device(ops):
    from blackriver_b200 import brk
    x = torch.zeros(64, device="cuda")
    # workspace too small for the vector path of LayerNorm backward
    st = brk.raw("brk_layernorm_bwd", x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                 x.data_ptr(), x.data_ptr(), 1, 64, 1e-5, x.data_ptr(), 8, 0, brk.F32, 0)
    assert st == brk.ATTR_ERROR
    a = (brk.i64 * 4)(1, 1, 2, 8); b = (brk.i64 * 4)(1, 1, 3, 8)
    assert brk.raw("brk_add_bcast", x.data_ptr(), x.data_ptr(), x.data_ptr(), a, b, brk.F32, 0) == brk.INPUT_ERROR


def test_colsum_two_stage(ops):
    from blackriver_b200 import brk
    rng = np.random.default_rng(21)
    for dtype, tdt, tol in ((np.float32, brk.F32, TOL32), (np.float16, brk.F16, TOL16)):
        for rows, cols in ((2048, 4096), (300, 72), (1000, 16384)):
            x = rng.standard_normal((rows, cols)).astype(dtype)
            dx = torch.from_numpy(x).cuda()
            out = torch.from_numpy(np.full(cols, 2.0, dtype)).cuda()
            ws = torch.empty(brk.lib().brk_colsum_workspace_bytes(rows, cols), dtype=torch.uint8, device="cuda")
            brk.call("brk_colsum_ws", dx.data_ptr(), out.data_ptr(), rows, cols, 1, tdt, ws.data_ptr(), ws.numel(), ops.stream())
            assert relerr(host(out), x.astype(np.float64).sum(0) + 2.0) <= tol
