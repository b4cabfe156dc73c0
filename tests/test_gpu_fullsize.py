"""The hot-path kernels at the benchmark's full sizes (8192 tokens, hidden 4096 / 16384, vocabulary 250880,
the 7b1 GEMM and attention shapes), where the CPU oracle would take minutes.

Each kernel is compared with an fp32 torch evaluation of the same formula on the same fp16-rounded inputs, on
the device, and checked for the size-independent properties its definition gives (normalised rows, odd/even
symmetry of GELU, gradient rows that sum to zero, linearity of the backward passes).  Tolerances are the fp16
storage tolerances of the small-size tests: 2e-2 relative to the largest reference entry for tensors, 1e-3 for
the loss."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOKENS, HIDDEN, HIDDEN4, VOCAB = 8192, 4096, 16384, 250880
TOL16 = 2e-2


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from blackriver_b200 import ops as _ops
    return _ops


def gen(seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return g


def relerr(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-30))


def test_layernorm_full_size(ops):
    g = gen(1)
    x = (torch.randn(TOKENS, HIDDEN, generator=g, device="cuda") * 1.5 + 0.25).half()
    gamma = (1 + 0.1 * torch.randn(HIDDEN, generator=g, device="cuda")).half()
    beta = (0.1 * torch.randn(HIDDEN, generator=g, device="cuda")).half()
    dy = torch.randn(TOKENS, HIDDEN, generator=g, device="cuda").half()
    y, mean, var = ops.layernorm(x, gamma, beta, 1e-5)
    xf, gf, bf = x.float(), gamma.float(), beta.float()
    mu = xf.mean(-1)
    v = xf.var(-1, unbiased=False) + 1e-5
    y_ref = (xf - mu[:, None]) * torch.rsqrt(v)[:, None] * gf + bf
    assert relerr(y, y_ref) <= TOL16
    assert relerr(var, v) <= 1e-3 and float((mean - mu).abs().max()) <= 1e-3
    # every row of (y - beta) / gamma is normalised
    xhat = (y.float() - bf) / gf
    assert float(xhat.mean(-1).abs().max()) <= 5e-3
    assert float((xhat.var(-1, unbiased=False) - 1).abs().max()) <= 2e-2

    dg, db, dx = ops.layernorm_backward(dy, gamma, beta, var, y, 1e-5)
    gy = dy.float() * gf
    dx_ref = (gy - gy.mean(-1, keepdim=True) - xhat * (gy * xhat).mean(-1, keepdim=True)) * torch.rsqrt(var)[:, None]
    assert relerr(dx, dx_ref) <= TOL16
    assert relerr(dg, (dy.float() * xhat).sum(0)) <= TOL16
    assert relerr(db, dy.float().sum(0)) <= TOL16
    # every row of dx sums to zero (the mean of the row's gradient has been taken out)
    scale = float(dx_ref.abs().max())
    assert float(dx.float().sum(-1).abs().max()) <= 2e-2 * scale * HIDDEN ** 0.5
    # linear in dy
    dg2, db2, dx2 = ops.layernorm_backward(dy * 2, gamma, beta, var, y, 1e-5)
    assert float((dx2.float() - 2 * dx.float()).abs().max()) <= 2e-3 * scale
    assert relerr(db2, 2 * db.float()) <= 2e-3


def test_gelu_full_size(ops):
    g = gen(2)
    x = (torch.randn(TOKENS, HIDDEN4, generator=g, device="cuda") * 2).half()
    dy = torch.randn(TOKENS, HIDDEN4, generator=g, device="cuda").half()
    y = ops.gelu(x)
    xf = x.float()
    t = torch.tanh(0.79788456 * xf * (1 + 0.044715 * xf * xf))
    assert relerr(y, 0.5 * xf * (1 + t)) <= TOL16
    # gelu(x) - gelu(-x) = x
    y_neg = ops.gelu(-x)
    assert float((y.float() - y_neg.float() - xf).abs().max()) <= 4e-3 * float(xf.abs().max())
    dx = ops.gelu_backward(dy, x)
    d_ref = (0.5 * xf * ((1 - t * t) * (0.79788456 + 0.1070322243 * xf * xf)) + 0.5 * (1 + t)) * dy.float()
    assert relerr(dx, d_ref) <= TOL16
    # the derivative is even in x: backward(dy, x) = backward(dy, -x) shifted by dy: gelu'(x) + gelu'(-x) = 1
    dx_neg = ops.gelu_backward(dy, -x)
    assert float((dx.float() + dx_neg.float() - dy.float()).abs().max()) <= 4e-3 * float(dy.float().abs().max())


def test_nll_full_size(ops):
    g = gen(3)
    logits = torch.empty(TOKENS, VOCAB, dtype=torch.float16, device="cuda")
    for r0 in range(0, TOKENS, 1024):      # filled in bands: no 8 GB fp32 temporary
        logits[r0:r0 + 1024] = (torch.randn(1024, VOCAB, generator=g, device="cuda") * 2).half()
    target = torch.randint(0, VOCAB, (TOKENS,), generator=g, device="cuda", dtype=torch.int32)
    ignored = torch.rand(TOKENS, generator=g, device="cuda") < 0.1
    target[ignored] = -100
    row_loss, dlogits = ops.logsoftmax_nll_backward(logits, target, 1.0)
    torch.cuda.synchronize()
    worst_loss, worst_grad, worst_sum = 0.0, 0.0, 0.0
    for r0 in range(0, TOKENS, 512):
        lf = logits[r0:r0 + 512].float()
        tg = target[r0:r0 + 512].long()
        valid = tg >= 0
        lse = torch.logsumexp(lf, -1)
        ref = torch.where(valid, lse - lf.gather(1, tg.clamp_min(0)[:, None])[:, 0], torch.zeros_like(lse))
        worst_loss = max(worst_loss, float((row_loss[r0:r0 + 512] - ref).abs().max() / ref.abs().max()))
        p = torch.softmax(lf, -1)
        p[torch.arange(512, device="cuda")[valid], tg[valid]] -= 1.0
        p[~valid] = 0.0
        got = dlogits[r0:r0 + 512].float()
        worst_grad = max(worst_grad, float((got - p).abs().max()))          # largest reference entry is 1 (the target's)
        worst_sum = max(worst_sum, float(got.sum(-1).abs().max()))
        assert bool((got[~valid] == 0).all())                               # ignored rows: gradient exactly zero
    assert worst_loss <= 1e-3
    assert worst_grad <= TOL16
    assert worst_sum <= 1e-2                                                # softmax minus one-hot sums to zero
    total = ops.sum_f32(row_loss)
    assert abs(float(total) - float(row_loss.double().sum())) <= 1e-5 * float(row_loss.double().sum())
    # scaling the gradient scales it exactly (power of two)
    row_loss2, dlogits2 = ops.logsoftmax_nll_backward(logits[:256], target[:256], 0.5)
    assert torch.equal(row_loss2, row_loss[:256])
    assert float((dlogits2.float() * 2 - dlogits[:256].float()).abs().max()) <= 2e-7


@pytest.mark.parametrize("m,n,k,ta,tb", [
    (2048, 12288, 4096, 0, 1),      # fused QKV projection of one micro-batch
    (2048, 16384, 4096, 0, 1),      # h -> 4h
    (2048, 4096, 16384, 0, 0),      # input gradient of h -> 4h
    (16384, 4096, 2048, 1, 0),      # weight gradient of h -> 4h
    (2048, 4096, 4096, 0, 1),       # attention dense
])
def test_gemm_7b1_shapes(ops, m, n, k, ta, tb):
    from blackriver_b200 import brk
    g = gen(m + n + k)
    a = torch.randn((k, m) if ta else (m, k), generator=g, device="cuda").half()
    b = torch.randn((n, k) if tb else (k, n), generator=g, device="cuda").half()
    c = torch.empty(m, n, dtype=torch.float16, device="cuda")
    ops.gemm_f16(a, b, c, m, n, k, ta, tb, a.shape[1], b.shape[1], n)
    torch.cuda.synchronize()
    assert brk.lib().brk_gemm_f16_status() == 0
    ref = (a.float().t() if ta else a.float()) @ (b.float().t() if tb else b.float())
    assert relerr(c, ref) <= 2e-3           # fp16 rounding of the output; accumulation is fp32
    # linear in A: doubling A doubles every accumulator exactly (entries in fp16's subnormal range may round differently)
    c2 = torch.empty_like(c)
    ops.gemm_f16(a * 2, b, c2, m, n, k, ta, tb, a.shape[1], b.shape[1], n)
    assert float((c2.float() - 2 * c.float()).abs().max()) <= 1e-6


def test_attention_7b1_shape(ops):
    """One micro-batch of the fine-tune step: batch 2 x 1024 tokens x 32 heads x 128, one padded sequence."""
    import ctypes as C
    from blackriver_b200 import brk
    B, T, heads, d = 2, 1024, 32, 128
    H = heads * d
    lens = [1024, 611]
    g = gen(5)
    qkv = torch.randn(B * T, 3 * H, generator=g, device="cuda").half()
    out = torch.empty(B * T, H, dtype=torch.float16, device="cuda")
    lse = torch.empty(B, heads, T, dtype=torch.float32, device="cuda")
    dl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    sl = (C.c_double * heads)()
    brk.lib().brk_alibi_slopes(heads, sl)
    slopes = torch.tensor(list(sl), dtype=torch.float64).float().cuda()
    base = qkv.data_ptr()
    brk.call("brk_flash_attn_fwd", base, base + 2 * H, base + 4 * H, 3 * H, out.data_ptr(), H, lse.data_ptr(), dl.data_ptr(),
             slopes.data_ptr(), B, T, heads, d, ops.stream())
    torch.cuda.synchronize()
    assert brk.lib().brk_flash_attn_status() == 0
    q, k, v = (qkv[:, i * H:(i + 1) * H].float().reshape(B, T, heads, d).permute(0, 2, 1, 3) for i in range(3))
    key = torch.arange(T, device="cuda")
    s = q @ k.transpose(-1, -2) / d ** 0.5 + slopes[None, :, None, None] * key[None, None, None, :].float()
    allowed = (key[None, :] <= key[:, None])[None, None] & (key[None, None, None, :] < dl.long()[:, None, None, None])
    s = s.masked_fill(~allowed, float("-inf"))
    ref = (torch.softmax(s, -1) @ v).permute(0, 2, 1, 3).reshape(B * T, H)
    assert relerr(out, ref) <= TOL16
    assert float((lse - torch.logsumexp(s, -1)).abs().max()) <= 2e-2
    # rows of a softmax-weighted average stay inside the range of the values they average
    vmax = v.abs().amax()
    assert float(out.float().abs().max()) <= float(vmax) * 1.01
