"""Fused attention (tcgen05) through the C ABI against the CPU oracle's unfused chain
qk -> +alibi -> +mask -> softmax -> attn on the same fp16-rounded inputs (fp16 tolerance 2e-2)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu
TOL16 = 2e-2


def relerr(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def reference(q, k, v, lens, heads):
    """q, k, v: [B,T,h,d] float32 -> (out [B,T,h,d], lse [B,h,T], probs [B,h,T,T])."""
    B, T, h, d = q.shape
    mask = np.zeros((B, T), np.int32)
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    zq, zk, zv = (orc.transpose_0213(x) for x in (q, k, v))
    s = orc.add_bcast(orc.add_bcast(orc.qk(zq, zk), orc.alibi(heads, T)), orc.build_xmask(mask))
    p = orc.softmax(s)
    out = orc.transpose_0213(orc.attn(p, zv))
    s64 = s.astype(np.float64)
    m = s64.max(-1, keepdims=True)
    lse = (m + np.log(np.exp(s64 - m).sum(-1, keepdims=True)))[..., 0]
    return out, lse, p


def slopes_f32(heads):
    return orc.alibi_slopes(heads).astype(np.float32)


@pytest.mark.parametrize("B,T,heads,d,lens", [
    (2, 128, 4, 64, (128, 77)),
    (2, 300, 2, 128, (300, 131)),
    (1, 512, 2, 128, (512,)),
    (3, 200, 2, 64, (1, 200, 129)),
    (1, 2048, 2, 128, (2048,)),          # the long-context prefill shape: 2048 positions, head dimension 128, no padding
])
def test_flash_attention_forward(B, T, heads, d, lens):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from blackriver_b200 import brk, ops
    rng = np.random.default_rng(T + d)
    H = heads * d
    qkv = rng.standard_normal((B * T, 3 * H)).astype(np.float16)       # fused projection output
    q, k, v = (qkv[:, i * H:(i + 1) * H].astype(np.float32).reshape(B, T, heads, d) for i in range(3))
    out_ref, lse_ref, _ = reference(q, k, v, lens, heads)
    dqkv = torch.from_numpy(qkv).cuda()
    out = torch.full((B * T, H), 9.0, dtype=torch.float16, device="cuda")
    lse = torch.empty((B, heads, T), dtype=torch.float32, device="cuda")
    dl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ds = torch.from_numpy(slopes_f32(heads)).cuda()
    base = dqkv.data_ptr()
    brk.call("brk_flash_attn_fwd", base, base + 2 * H, base + 4 * H, 3 * H, out.data_ptr(), H, lse.data_ptr(), dl.data_ptr(),
             ds.data_ptr(), B, T, heads, d, ops.stream())
    torch.cuda.synchronize()
    assert brk.lib().brk_flash_attn_status() == 0
    got = out.float().cpu().numpy().reshape(B, T, heads, d)
    assert relerr(got, out_ref) <= TOL16
    # rows of padded queries still attend to the valid prefix; compare the log-sum-exp everywhere
    assert np.abs(lse.cpu().numpy() - lse_ref).max() <= 2e-2


def test_flash_attention_empty_sequence_and_no_alibi():
    from blackriver_b200 import brk, ops
    rng = np.random.default_rng(1)
    B, T, heads, d = 2, 128, 2, 64
    H = heads * d
    q, k, v = (torch.from_numpy(rng.standard_normal((B * T, H)).astype(np.float16)).cuda() for _ in range(3))
    out = torch.full((B * T, H), 9.0, dtype=torch.float16, device="cuda")
    dl = torch.tensor([0, 128], dtype=torch.int32, device="cuda")
    brk.call("brk_flash_attn_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), H, out.data_ptr(), H, 0, dl.data_ptr(), 0, B, T,
             heads, d, ops.stream())
    torch.cuda.synchronize()
    assert brk.lib().brk_flash_attn_status() == 0
    o = out.float().cpu().numpy().reshape(B, T, heads, d)
    assert (o[0] == 0).all()
    qf, kf, vf = (x.float().cpu().numpy().reshape(B, T, heads, d)[1:] for x in (q, k, v))
    s = np.einsum("bihd,bjhd->bhij", qf, kf) / np.sqrt(d)
    s = np.where(np.tril(np.ones((T, T), bool))[None, None], s, -np.inf)
    pr = np.exp(s - s.max(-1, keepdims=True)); pr /= pr.sum(-1, keepdims=True)
    ref = np.einsum("bhij,bjhd->bihd", pr, vf)
    assert relerr(o[1:], ref) <= TOL16


@pytest.mark.parametrize("B,T,heads,d,lens", [
    (2, 128, 4, 64, (128, 77)),
    (2, 300, 2, 128, (300, 131)),
    (1, 512, 2, 128, (512,)),
    (3, 200, 2, 64, (1, 200, 0)),
    (1, 2048, 2, 128, (2048,)),
])
def test_flash_attention_backward(B, T, heads, d, lens):
    from blackriver_b200 import brk, ops
    rng = np.random.default_rng(T * 3 + d)
    H = heads * d
    qkv = rng.standard_normal((B * T, 3 * H)).astype(np.float16)
    dout = rng.standard_normal((B * T, H)).astype(np.float16)
    q, k, v = (qkv[:, i * H:(i + 1) * H].astype(np.float32).reshape(B, T, heads, d) for i in range(3))
    # oracle: unfused backward chain of the layer_backward word
    ref_lens = [max(n, 0) for n in lens]
    out_ref, lse_ref, p = reference(q, k, v, ref_lens, heads)
    if 0 in ref_lens:                      # an empty sequence has no visible key: probabilities are all zero
        for b, n in enumerate(ref_lens):
            if n == 0:
                p[b] = 0
    zb = orc.transpose_0213(dout.astype(np.float32).reshape(B, T, heads, d))
    zq, zk, zv = (orc.transpose_0213(x) for x in (q, k, v))
    ds_ref, dv_ref = orc.softmax_attn_backward(zb, p, zv)
    dq_ref, dk_ref = orc.qk_backward(ds_ref, zq, zk)
    dq_ref, dk_ref, dv_ref = (orc.transpose_0213(x) for x in (dq_ref, dk_ref, dv_ref))

    dqkv = torch.from_numpy(qkv).cuda()
    ddo = torch.from_numpy(dout).cuda()
    out = torch.empty((B * T, H), dtype=torch.float16, device="cuda")
    lse = torch.empty((B, heads, T), dtype=torch.float32, device="cuda")
    dl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    dsl = torch.from_numpy(slopes_f32(heads)).cuda()
    grads = torch.full((B * T, 3 * H), 5.0, dtype=torch.float16, device="cuda")
    ws = torch.empty(brk.lib().brk_flash_attn_bwd_workspace_bytes(B, T, heads), dtype=torch.uint8, device="cuda")
    base, gb = dqkv.data_ptr(), grads.data_ptr()
    brk.call("brk_flash_attn_fwd", base, base + 2 * H, base + 4 * H, 3 * H, out.data_ptr(), H, lse.data_ptr(), dl.data_ptr(),
             dsl.data_ptr(), B, T, heads, d, ops.stream())
    brk.call("brk_flash_attn_bwd", base, base + 2 * H, base + 4 * H, 3 * H, out.data_ptr(), ddo.data_ptr(), H, lse.data_ptr(),
             gb, gb + 2 * H, gb + 4 * H, 3 * H, dl.data_ptr(), dsl.data_ptr(), B, T, heads, d, ws.data_ptr(), ws.numel(), ops.stream())
    torch.cuda.synchronize()
    assert brk.lib().brk_flash_attn_status() == 0
    g = grads.float().cpu().numpy()
    got = [g[:, i * H:(i + 1) * H].reshape(B, T, heads, d) for i in range(3)]
    for name, a, r in zip(("dq", "dk", "dv"), got, (dq_ref, dk_ref, dv_ref)):
        assert relerr(a, r) <= TOL16, name
