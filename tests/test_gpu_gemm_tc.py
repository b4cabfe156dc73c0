"""tcgen05 / TMEM fp16 GEMM through the C ABI against fp32 references.

Small problems are checked against the CPU oracle's linear operator, larger ones against a
float64 numpy product of the same fp16-rounded operands.  fp16 storage tolerance from the task:
2e-2 (the observed error is the fp16 rounding of the output, ~4e-4).  After every case the
kernel's status word must be 0 (no bounded wait gave up)."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL16 = 2e-2


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from blackriver_b200 import ops as _ops
    return _ops


def relerr(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def h16(a):
    return np.asarray(a, np.float32).astype(np.float16)


def gelu_ref(x):
    return x * 0.5 * (1 + np.tanh(0.79788456 * x * (1 + 0.044715 * x * x)))


def run(ops, m, n, k, ta, tb, seed, bias=False, res=False, acc=False, gelu=False, mode=0, epi=0, bias_offset=0):
    from blackriver_b200 import brk
    brk.lib().brk_gemm_f16_set_mode(mode)      # 1 = single-CTA tiles, 2 = CTA-pair (cta_group::2) tiles
    brk.lib().brk_gemm_f16_set_epilogue(epi)   # 0 = TMA store / reduce epilogue where it applies, 1 = register epilogue
    rng = np.random.default_rng(seed)
    A = h16(rng.standard_normal((k, m) if ta else (m, k)))
    B = h16(rng.standard_normal((n, k) if tb else (k, n)))
    C0 = h16(rng.standard_normal((m, n)))
    bs = h16(rng.standard_normal(n)) if bias else None
    R = h16(rng.standard_normal((m, n))) if res else None
    dev = lambda x: None if x is None else torch.from_numpy(x).cuda()
    C = dev(C0); G = torch.empty_like(C) if gelu else None
    dbias = dev(bs)
    if bias and bias_offset:        # a bias that starts at an element offset inside a larger buffer: not 16-byte aligned
        pad = torch.zeros(n + bias_offset, dtype=torch.float16, device="cuda")
        pad[bias_offset:] = dbias
        dbias = pad[bias_offset:]
        assert dbias.data_ptr() % 16 != 0
    ops.gemm_f16(dev(A), dev(B), C, m, n, k, ta, tb, A.shape[1], B.shape[1], n, bias=dbias, residual=dev(R), ldr=n,
                 gelu_out=G, ldg=n, accumulate=acc)
    torch.cuda.synchronize()
    brk.lib().brk_gemm_f16_set_mode(0)
    brk.lib().brk_gemm_f16_set_epilogue(0)
    assert brk.lib().brk_gemm_f16_status() == 0
    a = (A.T if ta else A).astype(np.float64); b = (B.T if tb else B).astype(np.float64)
    ref = a @ b
    if bias: ref = ref + bs.astype(np.float64)
    if res: ref = ref + R.astype(np.float64)
    if acc: ref = ref + C0.astype(np.float64)
    assert relerr(C.float().cpu().numpy(), ref) <= TOL16
    if gelu:
        assert relerr(G.float().cpu().numpy(), gelu_ref(ref)) <= TOL16


@pytest.mark.parametrize("mode,epi", [(1, 0), (2, 0), (2, 1)])
@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 1), (1, 0)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 512, 128), (200, 328, 136), (130, 72, 40), (1, 8, 8), (384, 1000, 264),
                                   (520, 264, 72)])
def test_all_layouts_and_tails(ops, m, n, k, ta, tb, mode, epi):
    if (ta and m % 8) or (not tb and n % 8):
        pytest.skip("this storage order needs a leading dimension that is a multiple of 8")
    run(ops, m, n, k, ta, tb, seed=m + n + k, mode=mode, epi=epi)


def test_epilogues(ops):
    run(ops, 256, 512, 128, 0, 1, 1, bias=True)
    run(ops, 256, 512, 128, 0, 1, 2, bias=True, res=True)
    run(ops, 256, 512, 128, 1, 0, 3, acc=True)
    run(ops, 200, 328, 136, 0, 1, 4, bias=True, res=True, acc=True, gelu=True)
    run(ops, 200, 328, 136, 0, 1, 4, bias=True, res=True, acc=True, gelu=True, mode=1)
    # the staged epilogue with tails in both directions: plain, bias, accumulate (TMA reduction), both; and its register twin
    for epi in (0, 1):
        run(ops, 520, 328, 136, 1, 0, 5, acc=True, epi=epi)
        run(ops, 520, 328, 136, 0, 1, 6, bias=True, epi=epi)
        run(ops, 520, 1000, 72, 0, 0, 7, bias=True, acc=True, epi=epi)
        run(ops, 304, 264, 72, 1, 1, 8, epi=epi)


def test_bias_at_an_odd_element_offset(ops):
    """A bias vector that is a view at an element offset of a larger buffer (possible through op.view) is not
    16-byte aligned: every epilogue has to read it with scalar loads."""
    for mode, epi in ((1, 0), (2, 0), (2, 1)):
        run(ops, 256, 512, 128, 0, 1, 21, bias=True, mode=mode, epi=epi, bias_offset=1)
        run(ops, 200, 328, 136, 0, 1, 22, bias=True, res=True, gelu=True, mode=mode, epi=epi, bias_offset=3)


def test_sixteen_accumulations_stay_within_tolerance(ops):
    """Weight gradients are summed over the micro-batches of a step by the GEMM itself (accumulate): 16 different
    products added into one fp16 C must stay within the fp16 tolerance of the float64 sum, in both epilogues."""
    from blackriver_b200 import brk
    m, n, k = 512, 384, 256
    rng = np.random.default_rng(31)
    for epi in (0, 1):
        brk.lib().brk_gemm_f16_set_epilogue(epi)
        C = torch.zeros((m, n), dtype=torch.float16, device="cuda")
        ref = np.zeros((m, n), np.float64)
        for i in range(16):
            A = h16(rng.standard_normal((k, m))); B = h16(rng.standard_normal((k, n)))
            ops.gemm_f16(torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), C, m, n, k, 1, 0, m, n, n, accumulate=True)
            ref += A.T.astype(np.float64) @ B.astype(np.float64)
        torch.cuda.synchronize()
        brk.lib().brk_gemm_f16_set_epilogue(0)
        assert brk.lib().brk_gemm_f16_status() == 0
        assert relerr(C.float().cpu().numpy(), ref) <= TOL16


def test_matches_oracle_linear_and_backward(ops):
    rng = np.random.default_rng(7)
    n_tok, i, o = 96, 128, 192
    x = h16(rng.standard_normal((n_tok, i))); w = h16(rng.standard_normal((o, i)) * 0.1); b = h16(rng.standard_normal(o))
    dy = h16(rng.standard_normal((n_tok, o)))
    dev = lambda a: torch.from_numpy(a).cuda()
    y = torch.empty((n_tok, o), dtype=torch.float16, device="cuda")
    ops.gemm_f16(dev(x), dev(w), y, n_tok, o, i, 0, 1, i, i, o, bias=dev(b))
    assert relerr(y.float().cpu().numpy(), orc.linear(x.astype(np.float32), w.astype(np.float32), b.astype(np.float32))) <= TOL16
    xg_ref, wg_ref, _ = orc.linear_backward(dy.astype(np.float32), x.astype(np.float32), w.astype(np.float32))
    wg = torch.empty((o, i), dtype=torch.float16, device="cuda"); xg = torch.empty((n_tok, i), dtype=torch.float16, device="cuda")
    ops.gemm_f16(dev(dy), dev(x), wg, o, i, n_tok, 1, 0, o, i, i)       # W_g = dy^T x
    ops.gemm_f16(dev(dy), dev(w), xg, n_tok, i, o, 0, 0, o, i, i)       # x_g = dy W
    assert relerr(wg.float().cpu().numpy(), wg_ref) <= TOL16 and relerr(xg.float().cpu().numpy(), xg_ref) <= TOL16


def test_model_shape_against_numpy(ops):
    run(ops, 2048, 4096, 4096, 0, 1, 11, bias=True)


def test_split_k_items(ops):
    """Few pair tiles and a long k: each tile's k range is cut into several work items that add their partial products
    into C through the TMA reduction (C cleared first; the bias rides on one item; accumulate keeps the old C).  Tails in
    both directions, every storage order, and the same calls with the splitting switched off."""
    from blackriver_b200 import brk
    for off in (0, 1):
        brk.lib().brk_gemm_f16_set_split_k(off)
        try:
            run(ops, 520, 328, 8192, 0, 1, 41, bias=True, mode=2)
            run(ops, 520, 328, 8192, 0, 0, 42, mode=2)
            run(ops, 520, 328, 6208, 1, 0, 43, acc=True, mode=2)
            run(ops, 304, 264, 8192, 1, 1, 44, bias=True, acc=True, mode=2)
            run(ops, 2048, 4096, 12288, 0, 0, 45)        # the QKV input gradient of one micro-batch: 128 tiles, 4 items each
        finally:
            brk.lib().brk_gemm_f16_set_split_k(0)


def test_rejects_unsupported_layout(ops):
    from blackriver_b200 import brk
    a = torch.zeros(64, device="cuda", dtype=torch.float16)
    assert brk.lib().brk_gemm_f16_supported(8, 8, 12, 0, 1, 12, 12, a.data_ptr(), a.data_ptr()) == 0
    assert brk.raw("brk_gemm_f16", a.data_ptr(), a.data_ptr(), a.data_ptr(), 8, 8, 12, 0, 1, 12, 12, 8, 0, 0, 0, 0, 0, 0, 0) == brk.ATTR_ERROR
