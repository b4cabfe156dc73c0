"""Thin torch-tensor front end over the C ABI (libbrk.so) for tests and benchmarks.

torch is used for device memory and streams only; every operator below is one or more calls
into the hand-written CUDA kernels.  Nothing here computes on the host or through torch ops,
and a missing library or a non-CUDA tensor raises.
"""
import torch

from . import brk

_DT = {torch.float32: brk.F32, torch.float16: brk.F16}


def _dt(t):
    if t.dtype not in _DT:
        raise TypeError(f"unsupported dtype {t.dtype}")
    return _DT[t.dtype]


def _chk(*ts):
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("blackriver_b200 operators run on CUDA tensors only (no CPU path)")
        if not t.is_contiguous():
            raise RuntimeError("tensors must be contiguous")


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def stream():
    return torch.cuda.current_stream().cuda_stream


def layernorm(x, gamma, beta, eps=1e-5, out=None):
    _chk(x, gamma, beta, out)
    h = x.shape[-1]
    rows = x.numel() // h
    y = torch.empty_like(x) if out is None else out
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    var = torch.empty(rows, dtype=torch.float32, device=x.device)
    brk.call("brk_layernorm_fwd", _ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), _ptr(mean), _ptr(var), rows, h, eps,
             _dt(x), stream())
    return y, mean, var


def layernorm_backward(dy, gamma, beta, var, y, eps=1e-5, dgamma=None, dbeta=None, dx=None, accumulate=False,
                       workspace=None, residual=None):
    _chk(dy, gamma, beta, var, y, dgamma, dbeta, dx, workspace, residual)
    h = dy.shape[-1]
    rows = dy.numel() // h
    dgamma = torch.empty_like(gamma) if dgamma is None else dgamma
    dbeta = torch.empty_like(beta) if dbeta is None else dbeta
    dx = torch.empty_like(dy) if dx is None else dx
    need = brk.lib().brk_layernorm_bwd_workspace_bytes(rows, h)
    if workspace is None:
        workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=dy.device)
    if residual is None:
        brk.call("brk_layernorm_bwd", _ptr(dy), _ptr(gamma), _ptr(beta), _ptr(var), _ptr(y), _ptr(dgamma), _ptr(dbeta),
                 _ptr(dx), rows, h, eps, _ptr(workspace), workspace.numel() * workspace.element_size(), int(accumulate),
                 _dt(dy), stream())
    else:
        brk.call("brk_layernorm_bwd_residual", _ptr(dy), _ptr(gamma), _ptr(beta), _ptr(var), _ptr(y), _ptr(residual), _ptr(dgamma),
                 _ptr(dbeta), _ptr(dx), rows, h, eps, _ptr(workspace), workspace.numel() * workspace.element_size(),
                 int(accumulate), _dt(dy), stream())
    return dgamma, dbeta, dx


def gelu(x, out=None):
    _chk(x, out)
    y = torch.empty_like(x) if out is None else out
    brk.call("brk_gelu_fwd", _ptr(x), _ptr(y), x.numel(), _dt(x), stream())
    return y


def gelu_backward(dy, x, out=None):
    _chk(dy, x, out)
    dx = torch.empty_like(x) if out is None else out
    brk.call("brk_gelu_bwd", _ptr(dy), _ptr(x), _ptr(dx), x.numel(), _dt(x), stream())
    return dx


def logsoftmax_nll(logits, target, row_loss=None, row_lse=None):
    _chk(logits, target, row_loss, row_lse)
    rows, vocab = logits.shape
    row_loss = torch.empty(rows, dtype=torch.float32, device=logits.device) if row_loss is None else row_loss
    brk.call("brk_logsoftmax_nll_fwd", _ptr(logits), _ptr(target), _ptr(row_loss), _ptr(row_lse), rows, vocab,
             _dt(logits), stream())
    return row_loss


def logsoftmax_nll_backward(logits, target, grad_scale, row_loss=None, dlogits=None):
    _chk(logits, target, row_loss, dlogits)
    rows, vocab = logits.shape
    row_loss = torch.empty(rows, dtype=torch.float32, device=logits.device) if row_loss is None else row_loss
    dlogits = torch.empty_like(logits) if dlogits is None else dlogits
    brk.call("brk_logsoftmax_nll_fwd_bwd", _ptr(logits), _ptr(target), _ptr(row_loss), _ptr(dlogits), rows, vocab,
             float(grad_scale), _dt(logits), stream())
    return row_loss, dlogits


def sum_f32(x, out=None):
    _chk(x, out)
    out = torch.empty(1, dtype=torch.float32, device=x.device) if out is None else out
    brk.call("brk_sum_f32", _ptr(x), _ptr(out), x.numel(), stream())
    return out


def loss_targets(ids, mask):
    _chk(ids, mask)
    b, t = ids.shape
    target = torch.empty_like(ids)
    count = torch.empty(1, dtype=torch.int32, device=ids.device)
    brk.call("brk_loss_targets", _ptr(ids), _ptr(mask), _ptr(target), _ptr(count), b, t, stream())
    return target, count


def add(a, b, out=None):
    _chk(a, b, out)
    c = torch.empty_like(a) if out is None else out
    brk.call("brk_add_bcast", _ptr(a), _ptr(b), _ptr(c), brk.dims4(a.shape), brk.dims4(b.shape), _dt(a), stream())
    return c


def fill(x, value):
    _chk(x)
    brk.call("brk_fill", _ptr(x), float(value), x.numel(), _dt(x), stream())
    return x


def cast(x, dtype):
    _chk(x)
    y = torch.empty(x.shape, dtype=dtype, device=x.device)
    brk.call("brk_cast", _ptr(x), _dt(x), _ptr(y), _DT[dtype], x.numel(), stream())
    return y


def transpose_0213(x, out=None):
    _chk(x, out)
    a, b, c, d = x.shape
    y = torch.empty((a, c, b, d), dtype=x.dtype, device=x.device) if out is None else out
    brk.call("brk_transpose_0213", _ptr(x), _ptr(y), a, b, c, d, _dt(x), stream())
    return y


def colsum(x, out=None, accumulate=False):
    _chk(x, out)
    rows, cols = x.shape
    out = torch.empty(cols, dtype=x.dtype, device=x.device) if out is None else out
    brk.call("brk_colsum", _ptr(x), _ptr(out), rows, cols, int(accumulate), _dt(x), stream())
    return out


def softmax(x, out=None):
    _chk(x, out)
    cols = x.shape[-1]
    y = torch.empty_like(x) if out is None else out
    brk.call("brk_softmax_fwd", _ptr(x), _ptr(y), x.numel() // cols, cols, _dt(x), stream())
    return y


def softmax_backward(dy, out, dx=None):
    _chk(dy, out, dx)
    cols = dy.shape[-1]
    dx = torch.empty_like(dy) if dx is None else dx
    brk.call("brk_softmax_bwd", _ptr(dy), _ptr(out), _ptr(dx), dy.numel() // cols, cols, _dt(dy), stream())
    return dx


def embedding_gather(table, ids):
    _chk(table, ids)
    vocab, h = table.shape
    out = torch.empty(tuple(ids.shape) + (h,), dtype=table.dtype, device=table.device)
    brk.call("brk_embedding_gather", _ptr(table), _ptr(ids), _ptr(out), ids.numel(), h, vocab, _dt(table), stream())
    return out


def alibi(heads, tokens, device="cuda"):
    import ctypes as C
    sl = (C.c_double * heads)()
    brk.lib().brk_alibi_slopes(heads, sl)
    slopes = torch.tensor(list(sl), dtype=torch.float64, device=device)
    out = torch.empty((1, heads, 1, tokens), dtype=torch.float32, device=device)
    brk.call("brk_alibi_build", _ptr(slopes), _ptr(out), heads, tokens, stream())
    return out


def xmask(mask):
    _chk(mask)
    b, t = mask.shape
    out = torch.empty((b, 1, t, t), dtype=torch.float32, device=mask.device)
    brk.call("brk_xmask_build", _ptr(mask), _ptr(out), b, t, stream())
    return out


def gemm(a, b, c, m, n, k, trans_a, trans_b, lda, ldb, ldc, batch=1, sa=0, sb=0, sc=0, alpha=1.0, beta=0.0, bias=None):
    _chk(a, b, c, bias)
    brk.call("brk_gemm", _ptr(a), _ptr(b), _ptr(c), m, n, k, int(trans_a), int(trans_b), lda, ldb, ldc, batch, sa, sb, sc,
             float(alpha), float(beta), _ptr(bias), _dt(a), stream())
    return c


def gemm_f16(a, b, c, m, n, k, trans_a, trans_b, lda, ldb, ldc, bias=None, residual=None, ldr=0, gelu_out=None, ldg=0,
             accumulate=False):
    """fp16 tensor-core GEMM (tcgen05/TMEM); raises if the layout is not supported."""
    _chk(a, b, c, bias, residual, gelu_out)
    brk.call("brk_gemm_f16", _ptr(a), _ptr(b), _ptr(c), m, n, k, int(trans_a), int(trans_b), lda, ldb, ldc, _ptr(bias),
             _ptr(residual), ldr, _ptr(gelu_out), ldg, int(accumulate), stream())
    return c


# --- operator-level compositions with the reference's semantics (blackriver/cuda_tensor.cpp) ---
def linear(x, w, bias, out=None):
    """op_linear (:147-193): y[n,o] = sum_i x[n,i] w[o,i] + b[o]."""
    o, i = w.shape
    n = x.numel() // i
    y = torch.empty(tuple(x.shape[:-1]) + (o,), dtype=x.dtype, device=x.device) if out is None else out
    return gemm(x, w, y, n, o, i, False, True, i, i, o, bias=bias)


def linear_backward(dy, x, w, x_g=None, w_g=None, b_g=None):
    """op_linear_backward (:731-812): b_g, then W_g = dy^T x, then x_g = dy W (x_g may alias x)."""
    o, i = w.shape
    n = x.numel() // i
    b_g = torch.empty(o, dtype=w.dtype, device=w.device) if b_g is None else b_g
    w_g = torch.empty_like(w) if w_g is None else w_g
    x_g = torch.empty_like(x) if x_g is None else x_g
    colsum(dy.view(n, o), out=b_g)
    gemm(dy, x, w_g, o, i, n, True, False, o, i, i)
    gemm(dy, w, x_g, n, i, o, False, False, o, i, i)
    return x_g, w_g, b_g


def qk(q, k, out=None):
    """op_qk (:278-330): S = Q K^T / sqrt(d), per (batch, head)."""
    b, h, t, d = q.shape
    s = torch.empty((b, h, t, t), dtype=q.dtype, device=q.device) if out is None else out
    return gemm(q, k, s, t, t, d, False, True, d, d, t, batch=b * h, sa=t * d, sb=t * d, sc=t * t, alpha=d ** -0.5)


def attn(p, v, out=None):
    """op_attn (:359-398): O = P V."""
    b, h, t, d = v.shape
    o = torch.empty_like(v) if out is None else out
    return gemm(p, v, o, t, d, t, False, False, t, d, d, batch=b * h, sa=t * t, sb=t * d, sc=t * d)


def softmax_attn_backward(dout, p, v, ds=None, dv=None):
    """op_softmax_attn_backward (:921-1002): dV = P^T dO; dS = softmax_bwd(P, dO V^T); ds may be p."""
    b, h, t, d = v.shape
    dv = torch.empty_like(v) if dv is None else dv
    ds = torch.empty_like(p) if ds is None else ds
    gemm(p, dout, dv, t, d, t, True, False, t, d, d, batch=b * h, sa=t * t, sb=t * d, sc=t * d)
    dp = torch.empty_like(p)
    gemm(dout, v, dp, t, t, d, False, True, d, d, t, batch=b * h, sa=t * d, sb=t * d, sc=t * t)
    softmax_backward(dp, p, dx=ds)
    return ds, dv


def qk_backward(ds, q, k, dq=None, dk=None):
    """op_qk_backward (:1005-1063): dQ = dS K / sqrt(d); dK = dS^T Q / sqrt(d)."""
    b, h, t, d = q.shape
    dq = torch.empty_like(q) if dq is None else dq
    dk = torch.empty_like(k) if dk is None else dk
    sc = d ** -0.5
    gemm(ds, k, dq, t, d, t, False, False, t, d, d, batch=b * h, sa=t * t, sb=t * d, sc=t * d, alpha=sc)
    gemm(ds, q, dk, t, d, t, True, False, t, d, d, batch=b * h, sa=t * t, sb=t * d, sc=t * d, alpha=sc)
    return dq, dk
