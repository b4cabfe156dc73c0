"""LayerNorm backward through the entry point that brings its own scratch memory.

Some users of the kernel library cannot provide a workspace when they call it -- code running
inside an engine that already owns all device memory, a process on a fixed GPU memory quota, or
a call made while a stream is being captured.  `brk_layernorm_bwd_static` serves them from an
array compiled into the library.  This test drives it through the C ABI and checks it against
the ordinary entry point on the same inputs, twice in a row with different problem sizes (the
second call reuses the array with the first call's leftovers in it), and checks that a problem
too large for the array is refused instead of overrunning it.

The file sorts last on purpose: if it fails, `pytest -x` has already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-4   # same bound as the other fp32 kernel tests: max |a-b| / max |b|


def relerr(a, b):
    a = a.double().cpu().numpy(); b = b.double().cpu().numpy()
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def run_both(brk, ops, rows, hidden, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    tdt = torch.float32 if dtype == brk.F32 else torch.float16
    x = torch.randn(rows, hidden, generator=g, device="cuda").to(tdt)
    dy = torch.randn(rows, hidden, generator=g, device="cuda").to(tdt)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g, device="cuda")).to(tdt)
    beta = (0.1 * torch.randn(hidden, generator=g, device="cuda")).to(tdt)
    y, _, var = ops.layernorm(x, gamma, beta, 1e-5)
    ref = ops.layernorm_backward(dy, gamma, beta, var, y, 1e-5)            # caller-provided workspace
    out = [torch.full_like(gamma, 7.0), torch.full_like(beta, -7.0), torch.full_like(dy, 3.0)]
    brk.call("brk_layernorm_bwd_static", dy.data_ptr(), gamma.data_ptr(), beta.data_ptr(), var.data_ptr(), y.data_ptr(),
             out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), rows, hidden, 1e-5, 0, dtype, ops.stream())
    torch.cuda.synchronize()
    for got, want, name in zip(out, ref, ("dgamma", "dbeta", "dx")):
        assert relerr(got, want) <= TOL, (name, rows, hidden)


def test_static_scratch_matches_workspace_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from blackriver_b200 import brk, ops
    assert brk.lib().brk_layernorm_bwd_static_capacity() == 16 << 20
    # first call: many rows, wide; second call: fewer CTAs and narrower rows over the leftovers
    run_both(brk, ops, rows=4096, hidden=4096, dtype=brk.F16, seed=1)
    run_both(brk, ops, rows=100, hidden=1024, dtype=brk.F32, seed=2)
    run_both(brk, ops, rows=4096, hidden=4096, dtype=brk.F16, seed=3)


def test_static_scratch_refuses_oversized_problem():
    from blackriver_b200 import brk
    rows, hidden = 100000, 8192
    need = brk.lib().brk_layernorm_bwd_workspace_bytes(rows, hidden)
    assert need > brk.lib().brk_layernorm_bwd_static_capacity()
    t = torch.zeros(16, device="cuda")
    ptr = t.data_ptr()   # never dereferenced: the size check comes first
    st = brk.raw("brk_layernorm_bwd_static", ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, rows, hidden, 1e-5, 0, brk.F32, 0)
    assert st == brk.ATTR_ERROR
    assert b"built-in array" in brk.lib().brk_last_cuda_error()
