"""CPU-side checks of the C ABI: the kernel library loads without a GPU and exports every
symbol that include/brk.h declares; argument validation answers without launching anything."""
import os
import re

import pytest

from blackriver_b200 import brk

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            txt = open(os.path.join(ROOT, "include", fn)).read()
            names += re.findall(r"^BRK_API[^;(]*?\b(brk_\w+)\s*\(", txt, flags=re.M)
    return names


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 20
    lib = brk.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported by libbrk.so"
    assert set(names) == set(brk.SIGNATURES), "python binding table and header disagree"


def test_host_library_exports_every_declared_symbol():
    from blackriver_b200 import host
    txt = open(os.path.join(ROOT, "include", "br_host.h")).read()
    names = re.findall(r"^BRH_API[^;(]*?\b(brh_\w+)\s*\(", txt, flags=re.M)
    assert len(names) >= 25
    lib = host.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/br_host.h but not exported by libbr_host.so"
    assert set(names) == set(host.SIGNATURES), "python binding table and header disagree"


def test_every_declaration_cites_the_reference():
    txt = open(os.path.join(ROOT, "include", "brk.h")).read()
    assert txt.count("blackriver/") >= 10


def test_argument_validation_without_gpu():
    # null pointers / bad sizes are rejected before any CUDA call
    assert brk.raw("brk_layernorm_fwd", 0, 0, 0, 0, 0, 0, 4, 8, 1e-5, brk.F32, 0) == brk.INPUT_ERROR
    assert brk.raw("brk_gelu_fwd", 16, 0, 8, brk.F32, 0) == brk.OUTPUT_ERROR
    assert brk.raw("brk_gelu_fwd", 16, 16, -1, brk.F32, 0) == brk.ATTR_ERROR
    assert brk.raw("brk_gelu_fwd", 16, 16, 8, 7, 0) == brk.ATTR_ERROR
    assert brk.raw("brk_logsoftmax_nll_fwd", 0, 0, 0, 0, 1, 1, brk.F16, 0) == brk.INPUT_ERROR
    assert brk.raw("brk_gelu_fwd", 16, 16, 0, brk.F32, 0) == brk.OK  # empty input is a no-op
    assert brk.lib().brk_layernorm_bwd_workspace_bytes(0, 64) == 0
    assert brk.lib().brk_layernorm_bwd_workspace_bytes(8192, 4096) >= 2 * 4096 * 4


def test_alibi_slopes_host_helper_matches_oracle():
    import ctypes as C
    import numpy as np
    from oracle import oracle as orc
    for heads in (4, 16, 32):
        sl = (C.c_double * heads)()
        brk.lib().brk_alibi_slopes(heads, sl)
        assert np.array(list(sl)).tobytes() == orc.alibi_slopes(heads).tobytes()


def test_split_k_rule_without_gpu():
    """Work items per tile of the CTA-pair GEMM: 128 tiles on 74 CTA pairs leave the second wave 73 % full, four items
    per tile fill 6.9 waves; never fewer than 32 k-blocks per item, and nothing to gain when the waves are full."""
    from blackriver_b200 import brk
    f = brk.lib().brk_gemm_f16_split_items
    assert f(128, 74, 192) == 4 and f(128, 74, 256) == 4 and f(128, 74, 3920) == 4      # dX of QKV, of h->4h, of the LM head
    assert f(128, 74, 64) == 1                       # k = 4096: two items would leave the fill unchanged, more are too short
    assert f(256, 74, 32) == 1                       # weight gradients: k = 2048 tokens is too short to cut
    assert f(512, 74, 64) == 1 and f(7840, 74, 64) == 1
    assert f(4, 74, 128) == 3                        # a handful of tiles with a long k
    assert f(0, 74, 64) == 1 and f(128, 0, 64) == 1 and f(128, 74, 0) == 1
