"""numpy front end of the CPU oracle (libbr_oracle.so) -- TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the CPU-baseline leg of the benchmark import this
module.  It is the checker, never the thing measured as the product and never a fallback.

Besides one wrapper per oracle function it holds `layer_forward` / `layer_backward`, which
chain the operators in exactly the order of the reference's `layer_forward` /
`layer_backward` words (bloomz-7b/train.words:137-248), including the in-place steps.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    """Compile the oracle with its Makefile (gcc, OpenMP)."""
    subprocess.run(["make", "-C", _HERE, "--no-print-directory"], check=True,
                   stdout=subprocess.DEVNULL)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libbr_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = C.CDLL(path)
        _LIB.orc_logsoftmax_nll.restype = C.c_double
        _LIB.orc_loss_backward.restype = C.c_float
        _LIB.orc_loss_targets.restype = C.c_int
        _LIB.orc_num_threads.restype = C.c_int
    return _LIB


def num_threads():
    return int(lib().orc_num_threads())


def use_all_cores():
    """OpenMP threads = the cores this process may run on, whatever OMP_NUM_THREADS a launcher exported
    (torch.distributed.run sets it to 1 for its workers).  Returns the count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(C.c_int(n))
    return num_threads()


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _i64(v):
    return C.c_int64(int(v))


def layernorm(x, gamma, beta, eps=1e-5):
    x = _f(x); gamma = _f(gamma); beta = _f(beta)
    h = x.shape[-1]; rows = x.size // h
    y = np.empty_like(x); mean = np.empty(rows, np.float32); var = np.empty(rows, np.float32)
    lib().orc_layernorm(_p(x), _p(gamma), _p(beta), _p(y), _p(mean), _p(var), _i64(rows), _i64(h), C.c_float(eps))
    return y, mean, var


def layernorm_backward(dy, gamma, beta, var, y, eps=1e-5):
    dy = _f(dy); gamma = _f(gamma); beta = _f(beta); var = _f(var); y = _f(y)
    h = dy.shape[-1]; rows = dy.size // h
    dgamma = np.empty(h, np.float32); dbeta = np.empty(h, np.float32); dx = np.empty_like(dy)
    lib().orc_layernorm_backward(_p(dy), _p(gamma), _p(beta), _p(var), _p(y), _p(dgamma), _p(dbeta), _p(dx),
                                 _i64(rows), _i64(h), C.c_float(eps))
    return dgamma, dbeta, dx


def gelu(x):
    x = _f(x); y = np.empty_like(x)
    lib().orc_gelu(_p(x), _p(y), _i64(x.size))
    return y


def gelu_backward(dy, x):
    dy = _f(dy); x = _f(x); dx = np.empty_like(x)
    lib().orc_gelu_backward(_p(dy), _p(x), _p(dx), _i64(x.size))
    return dx


def linear(x, w, b):
    x = _f(x); w = _f(w)
    b = None if b is None else _f(b)
    out, inn = w.shape
    n = x.size // inn
    y = np.empty(x.shape[:-1] + (out,), np.float32)
    lib().orc_linear(_p(x), _p(w), _p(b), _p(y), _i64(n), _i64(inn), _i64(out))
    return y


def linear_backward(dy, x, w):
    dy = _f(dy); x = _f(x); w = _f(w)
    out, inn = w.shape
    n = x.size // inn
    x_g = np.empty_like(x); w_g = np.empty_like(w); b_g = np.empty(out, np.float32)
    lib().orc_linear_backward(_p(dy), _p(x), _p(w), _p(x_g), _p(w_g), _p(b_g), _i64(n), _i64(inn), _i64(out))
    return x_g, w_g, b_g


def transpose_0213(x):
    x = _f(x)
    a, b, c, d = x.shape
    y = np.empty((a, c, b, d), np.float32)
    lib().orc_transpose_0213(_p(x), _p(y), _i64(a), _i64(b), _i64(c), _i64(d))
    return y


def qk(q, k):
    q = _f(q); k = _f(k)
    b, h, t, d = q.shape
    s = np.empty((b, h, t, t), np.float32)
    lib().orc_qk(_p(q), _p(k), _p(s), _i64(b * h), _i64(t), _i64(d))
    return s


def add_bcast(a, b):
    a = _f(a); b = _f(b)
    ad = (C.c_int64 * 4)(*([1] * (4 - a.ndim) + list(a.shape)))
    bd = (C.c_int64 * 4)(*([1] * (4 - b.ndim) + list(b.shape)))
    c = np.empty_like(a)
    lib().orc_add_bcast(_p(a), _p(b), _p(c), ad, bd)
    return c


def softmax(x):
    x = _f(x); y = np.empty_like(x)
    cols = x.shape[-1]
    lib().orc_softmax(_p(x), _p(y), _i64(x.size // cols), _i64(cols))
    return y


def softmax_backward(dy, out):
    dy = _f(dy); out = _f(out); dx = np.empty_like(dy)
    cols = dy.shape[-1]
    lib().orc_softmax_backward(_p(dy), _p(out), _p(dx), _i64(dy.size // cols), _i64(cols))
    return dx


def attn(p, v):
    p = _f(p); v = _f(v)
    b, h, t, d = v.shape
    o = np.empty_like(v)
    lib().orc_attn(_p(p), _p(v), _p(o), _i64(b * h), _i64(t), _i64(d))
    return o


def attn_backward(dout, p, v):
    dout = _f(dout); p = _f(p); v = _f(v)
    b, h, t, d = v.shape
    dp = np.empty_like(p); dv = np.empty_like(v)
    lib().orc_attn_backward(_p(dout), _p(p), _p(v), _p(dp), _p(dv), _i64(b * h), _i64(t), _i64(d))
    return dp, dv


def softmax_attn_backward(dout, p, v):
    dout = _f(dout); p = _f(p); v = _f(v)
    b, h, t, d = v.shape
    ds = np.empty_like(p); dv = np.empty_like(v)
    lib().orc_softmax_attn_backward(_p(dout), _p(p), _p(v), _p(ds), _p(dv), _i64(b * h), _i64(t), _i64(d))
    return ds, dv


def qk_backward(ds, q, k):
    ds = _f(ds); q = _f(q); k = _f(k)
    b, h, t, d = q.shape
    dq = np.empty_like(q); dk = np.empty_like(k)
    lib().orc_qk_backward(_p(ds), _p(q), _p(k), _p(dq), _p(dk), _i64(b * h), _i64(t), _i64(d))
    return dq, dk


def alibi_slopes(heads):
    s = np.empty(heads, np.float64)
    lib().orc_alibi_slopes(C.c_int(heads), _p(s))
    return s


def alibi(heads, tokens):
    out = np.empty((1, heads, 1, tokens), np.float32)
    lib().orc_alibi(C.c_int(heads), C.c_int(tokens), _p(out))
    return out


def build_xmask(mask):
    mask = np.ascontiguousarray(mask, dtype=np.int32)
    b, t = mask.shape
    out = np.empty((b, 1, t, t), np.float32)
    lib().orc_build_xmask(_p(mask), C.c_int(b), C.c_int(t), _p(out))
    return out


def embedding_gather(table, ids):
    table = _f(table); ids = np.ascontiguousarray(ids, dtype=np.int32)
    h = table.shape[1]
    out = np.empty(ids.shape + (h,), np.float32)
    lib().orc_embedding_gather(_p(table), _p(ids), _p(out), _i64(ids.size), _i64(h))
    return out


def loss_targets(ids, mask):
    ids = np.ascontiguousarray(ids, dtype=np.int32); mask = np.ascontiguousarray(mask, dtype=np.int32)
    b, t = ids.shape
    tg = np.empty((b, t), np.int32)
    items = lib().orc_loss_targets(_p(ids), _p(mask), C.c_int(b), C.c_int(t), _p(tg))
    return tg, int(items)


def logsoftmax_nll(logits, target, grad_scale=None):
    """Returns (sum of row losses, row_loss[rows], dlogits or None)."""
    logits = _f(logits); target = np.ascontiguousarray(target, dtype=np.int32)
    rows, vocab = logits.shape
    row_loss = np.empty(rows, np.float32)
    dl = np.empty_like(logits) if grad_scale is not None else None
    total = lib().orc_logsoftmax_nll(_p(logits), _p(target), _p(row_loss), _p(dl), _i64(rows), _i64(vocab),
                                     C.c_float(0.0 if grad_scale is None else grad_scale))
    return float(total), row_loss, dl


def loss_backward(x, ids, mask, w, w_g=None):
    """Returns (mean NLL, x_g, w_g); w_g is accumulated into when given."""
    x = _f(x); w = _f(w)
    ids = np.ascontiguousarray(ids, dtype=np.int32); mask = np.ascontiguousarray(mask, dtype=np.int32)
    b, t, h = x.shape
    v = w.shape[0]
    x_g = np.empty_like(x)
    if w_g is None:
        w_g = np.zeros_like(w)
    loss = lib().orc_loss_backward(_p(x), _p(ids), _p(mask), _p(w), _p(x_g), _p(w_g),
                                   C.c_int(b), C.c_int(t), _i64(h), _i64(v))
    return float(loss), x_g, w_g


def last_logits(x, mask, w):
    x = _f(x); w = _f(w); mask = np.ascontiguousarray(mask, dtype=np.int32)
    b, t, h = x.shape
    v = w.shape[0]
    out = np.empty((b, v), np.float32)
    lib().orc_last_logits(_p(x), _p(mask), _p(w), _p(out), C.c_int(b), C.c_int(t), _i64(h), _i64(v))
    return out


def adam(w, m, v, g, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, step=1, grad_scale=1.0):
    """In place on w, m, v (float32 contiguous arrays)."""
    for a in (w, m, v):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    g = _f(g)
    lib().orc_adam(_p(w), _p(m), _p(v), _p(g), _i64(w.size), C.c_float(lr), C.c_float(beta1), C.c_float(beta2),
                   C.c_float(eps), C.c_int(step), C.c_float(grad_scale))


# ---------------------------------------------------------------------------------------
# One decoder layer, operator by operator, as the words scripts chain them.
# ---------------------------------------------------------------------------------------
LAYER_PARAMS = (
    "input_layernorm.weight", "input_layernorm.bias",
    "query_key_value.weight", "query_key_value.bias",
    "dense.weight", "dense.bias",
    "post_attention_layernorm.weight", "post_attention_layernorm.bias",
    "dense_h_to_4h.weight", "dense_h_to_4h.bias",
    "dense_4h_to_h.weight", "dense_4h_to_h.bias",
)


def layer_forward(x, p, alibi_t, xmask, heads, eps=1e-5):
    """train.words:137-192.  x [B,T,H]; p maps LAYER_PARAMS names to arrays; the fused
    query_key_value weight is [3H,H] with rows 0..H-1 = Q, H..2H-1 = K, 2H..3H-1 = V
    (init.words:38-44).  Returns (output, saved activations for layer_backward)."""
    b, t, h = x.shape
    d = h // heads
    s = {}
    s["xinput"] = x
    s["xattn_in"], _, s["input_ln_var"] = layernorm(x, p["input_layernorm.weight"], p["input_layernorm.bias"], eps)
    wqkv = p["query_key_value.weight"]; bqkv = p["query_key_value.bias"]
    q = linear(s["xattn_in"], wqkv[0:h], bqkv[0:h])
    k = linear(s["xattn_in"], wqkv[h:2 * h], bqkv[h:2 * h])
    v = linear(s["xattn_in"], wqkv[2 * h:], bqkv[2 * h:])
    s["zquery"] = transpose_0213(q.reshape(b, t, heads, d))
    s["zkey"] = transpose_0213(k.reshape(b, t, heads, d))
    s["zvalue"] = transpose_0213(v.reshape(b, t, heads, d))
    sc = qk(s["zquery"], s["zkey"])
    sc = add_bcast(sc, alibi_t)
    sc = add_bcast(sc, xmask)
    s["xll"] = softmax(sc)
    ctx = attn(s["xll"], s["zvalue"])
    s["xattn_out"] = transpose_0213(ctx).reshape(b, t, h)
    dense = linear(s["xattn_out"], p["dense.weight"], p["dense.bias"])
    xa = dense + x
    s["xa"] = xa
    s["xb"], _, s["post_ln_var"] = layernorm(xa, p["post_attention_layernorm.weight"],
                                             p["post_attention_layernorm.bias"], eps)
    s["x4a"] = linear(s["xb"], p["dense_h_to_4h.weight"], p["dense_h_to_4h.bias"])
    s["x4b"] = gelu(s["x4a"])
    xc = linear(s["x4b"], p["dense_4h_to_h.weight"], p["dense_4h_to_h.bias"])
    out = xa + xc
    return out, s


def layer_backward(yout_g, p, s, heads, eps=1e-5):
    """train.words:194-248.  Returns (dx, grads) with grads keyed `<param>_g`."""
    b, t, h = yout_g.shape
    d = h // heads
    g = {}
    d4b, g["dense_4h_to_h.weight_g"], g["dense_4h_to_h.bias_g"] = linear_backward(yout_g, s["x4b"], p["dense_4h_to_h.weight"])
    d4a = gelu_backward(d4b, s["x4a"])
    dxb, g["dense_h_to_4h.weight_g"], g["dense_h_to_4h.bias_g"] = linear_backward(d4a, s["xb"], p["dense_h_to_4h.weight"])
    (g["post_attention_layernorm.weight_g"], g["post_attention_layernorm.bias_g"], dxa) = layernorm_backward(
        dxb, p["post_attention_layernorm.weight"], p["post_attention_layernorm.bias"], s["post_ln_var"], s["xb"], eps)
    yg = yout_g + dxa
    dctx, g["dense.weight_g"], g["dense.bias_g"] = linear_backward(yg, s["xattn_out"], p["dense.weight"])
    zb = transpose_0213(dctx.reshape(b, t, heads, d))
    ds, dv = softmax_attn_backward(zb, s["xll"], s["zvalue"])
    dq, dk = qk_backward(ds, s["zquery"], s["zkey"])
    xvalue = transpose_0213(dv).reshape(b, t, h)
    xquery = transpose_0213(dq).reshape(b, t, h)
    xkey = transpose_0213(dk).reshape(b, t, h)
    wqkv = p["query_key_value.weight"]
    wg = np.empty_like(wqkv); bg = np.empty(3 * h, np.float32)
    acc = np.zeros((b, t, h), np.float32)
    for i, dd in enumerate((xquery, xkey, xvalue)):
        dxi, wg[i * h:(i + 1) * h], bg[i * h:(i + 1) * h] = linear_backward(dd, s["xattn_in"], wqkv[i * h:(i + 1) * h])
        acc = acc + dxi
    g["query_key_value.weight_g"] = wg
    g["query_key_value.bias_g"] = bg
    (g["input_layernorm.weight_g"], g["input_layernorm.bias_g"], dxin) = layernorm_backward(
        acc, p["input_layernorm.weight"], p["input_layernorm.bias"], s["input_ln_var"], s["xattn_in"], eps)
    dx = dxin + yg
    return dx, g
