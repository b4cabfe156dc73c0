"""Generates tests/golden/*.npz by EXECUTING the reference's own PyTorch model.

Run where the reference checkout is available:

    python tests/golden/gen_golden.py [path/to/reference]

It imports `bloomz-7b/model.py` from the reference (never copied into this repository),
draws seeded inputs, runs the reference code on CPU in fp32 and stores inputs and outputs.
The committed .npz files are what the CPU oracle is pinned against.

Parameter layout note: the reference's weight dump re-orders the fused QKV weight from the
HF layout [heads,3,d,H] to [3,heads*d,H] (bloomz-7b/dump_weights.py:23-44); the fixtures
store the latter (the layout init.words:38-44 slices), and this script permutes to the HF
layout only to feed model.py.
"""
import os
import sys

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BLACKRIVER_REFERENCE", os.path.join(os.sep, "root", "reference"))
sys.path.insert(0, os.path.join(REF, "bloomz-7b"))
import model as refmodel  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def to_hf_qkv(w, heads):
    """[3, heads*d, ...] -> HF interleaved [heads, 3, d, ...] flattened on the first axis."""
    three_h = w.shape[0]
    h = three_h // 3
    d = h // heads
    rest = w.shape[1:]
    return w.reshape(3, heads, d, *rest).transpose(1, 0, 2, *range(3, 3 + len(rest))).reshape(three_h, *rest)


def from_hf_qkv(w, heads):
    three_h = w.shape[0]
    h = three_h // 3
    d = h // heads
    rest = w.shape[1:]
    return w.reshape(heads, 3, d, *rest).transpose(1, 0, 2, *range(3, 3 + len(rest))).reshape(three_h, *rest)


def gen_block(name, B, T, H, heads, lens, seed):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, std=1.0: (torch.randn(*s, generator=g) * std)
    p = {
        "input_layernorm.weight": 1.0 + rn(H, std=0.1),
        "input_layernorm.bias": rn(H, std=0.1),
        "query_key_value.weight": rn(3 * H, H, std=0.05),
        "query_key_value.bias": rn(3 * H, std=0.05),
        "dense.weight": rn(H, H, std=0.05),
        "dense.bias": rn(H, std=0.05),
        "post_attention_layernorm.weight": 1.0 + rn(H, std=0.1),
        "post_attention_layernorm.bias": rn(H, std=0.1),
        "dense_h_to_4h.weight": rn(4 * H, H, std=0.05),
        "dense_h_to_4h.bias": rn(4 * H, std=0.05),
        "dense_4h_to_h.weight": rn(H, 4 * H, std=0.05),
        "dense_4h_to_h.bias": rn(H, std=0.05),
    }
    x = rn(B, T, H)
    dy = rn(B, T, H)
    mask = torch.zeros(B, T, dtype=torch.int64)
    for b, n in enumerate(lens):
        mask[b, :n] = 1

    cfg = refmodel.LLMConfig(hidden_size=H, n_head=heads, n_layer=1, vocab_size=16)
    blk = refmodel.BloomBlock(cfg).float()
    sd = {
        "input_layernorm.weight": p["input_layernorm.weight"],
        "input_layernorm.bias": p["input_layernorm.bias"],
        "self_attention.query_key_value.weight": torch.from_numpy(to_hf_qkv(p["query_key_value.weight"].numpy(), heads).copy()),
        "self_attention.query_key_value.bias": torch.from_numpy(to_hf_qkv(p["query_key_value.bias"].numpy(), heads).copy()),
        "self_attention.dense.weight": p["dense.weight"],
        "self_attention.dense.bias": p["dense.bias"],
        "post_attention_layernorm.weight": p["post_attention_layernorm.weight"],
        "post_attention_layernorm.bias": p["post_attention_layernorm.bias"],
        "mlp.dense_h_to_4h.weight": p["dense_h_to_4h.weight"],
        "mlp.dense_h_to_4h.bias": p["dense_h_to_4h.bias"],
        "mlp.dense_4h_to_h.weight": p["dense_4h_to_h.weight"],
        "mlp.dense_4h_to_h.bias": p["dense_4h_to_h.bias"],
    }
    blk.load_state_dict(sd)
    blk.train()

    bm = refmodel.BloomModel.__new__(refmodel.BloomModel)  # only _prepare_attn_mask is used
    amask = refmodel.BloomModel._prepare_attn_mask(bm, mask, (B, T), 0)
    alibi = refmodel.build_alibi_tensor(mask, heads, torch.float32)

    xin = x.clone().requires_grad_(True)
    out = blk(xin, alibi=alibi, attention_mask=amask)[0]
    out.backward(dy)

    res = {"x": x.numpy(), "dy": dy.numpy(), "mask": mask.numpy().astype(np.int32),
           "heads": np.int32(heads), "out": out.detach().numpy(), "dx": xin.grad.numpy(),
           "ref_alibi": alibi.numpy()}
    for k, v in p.items():
        res["p." + k] = v.numpy()
    named = dict(blk.named_parameters())
    for k_ref, k_hf in (("input_layernorm.weight", "input_layernorm.weight"),
                        ("input_layernorm.bias", "input_layernorm.bias"),
                        ("dense.weight", "self_attention.dense.weight"),
                        ("dense.bias", "self_attention.dense.bias"),
                        ("post_attention_layernorm.weight", "post_attention_layernorm.weight"),
                        ("post_attention_layernorm.bias", "post_attention_layernorm.bias"),
                        ("dense_h_to_4h.weight", "mlp.dense_h_to_4h.weight"),
                        ("dense_h_to_4h.bias", "mlp.dense_h_to_4h.bias"),
                        ("dense_4h_to_h.weight", "mlp.dense_4h_to_h.weight"),
                        ("dense_4h_to_h.bias", "mlp.dense_4h_to_h.bias")):
        res["g." + k_ref] = named[k_hf].grad.numpy()
    res["g.query_key_value.weight"] = from_hf_qkv(named["self_attention.query_key_value.weight"].grad.numpy(), heads)
    res["g.query_key_value.bias"] = from_hf_qkv(named["self_attention.query_key_value.bias"].grad.numpy(), heads)
    np.savez_compressed(os.path.join(HERE, name), **res)
    print("wrote", name, {k: getattr(v, "shape", None) for k, v in res.items() if k in ("x", "out", "dx")})


def gen_pointwise(seed=11):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(4, 96, generator=g) * 2.0
    x[0, :8] = torch.tensor([0.0, -0.0, 1e-4, -1e-4, 8.0, -8.0, 20.0, -20.0])
    dy = torch.randn(4, 96, generator=g)
    y = refmodel.bloom_gelu_forward(x)
    dx = refmodel.bloom_gelu_back(dy, (x,))
    H = 96
    gamma = 1.0 + 0.2 * torch.randn(H, generator=g)
    beta = 0.2 * torch.randn(H, generator=g)
    ln = refmodel.LayerNorm(H, eps=1e-5)
    with torch.no_grad():
        ln.weight.copy_(gamma)
        ln.bias.copy_(beta)
    xi = x.clone().requires_grad_(True)
    ly = ln(xi)
    ly.backward(dy)
    np.savez_compressed(os.path.join(HERE, "pointwise.npz"), x=x.numpy(), dy=dy.numpy(), gelu=y.numpy(),
                        gelu_dx=dx.numpy(), gamma=gamma.numpy(), beta=beta.numpy(), ln_y=ly.detach().numpy(),
                        ln_dx=xi.grad.numpy(), ln_dgamma=ln.weight.grad.numpy(), ln_dbeta=ln.bias.grad.numpy())
    print("wrote pointwise.npz")


def gen_loss(seed=12):
    """Shifted-logits CrossEntropyLoss exactly as BloomForCausalLM.forward does it
    (model.py:795-804): labels = ids on valid positions, -100 on padding."""
    g = torch.Generator().manual_seed(seed)
    B, T, H, V = 2, 10, 24, 40
    x = torch.randn(B, T, H, generator=g)
    w = torch.randn(V, H, generator=g) * 0.3
    ids = torch.randint(0, V, (B, T), generator=g)
    mask = torch.zeros(B, T, dtype=torch.int64)
    mask[0, :10] = 1
    mask[1, :4] = 1
    labels = torch.where(mask != 0, ids, torch.full_like(ids, -100))
    xi = x.clone().requires_grad_(True)
    wi = w.clone().requires_grad_(True)
    logits = torch.nn.functional.linear(xi, wi)
    shift_logits = logits[..., :-1, :].contiguous()
    shift_labels = labels[..., 1:].contiguous()
    loss = refmodel.CrossEntropyLoss()(shift_logits.view(B * (T - 1), V), shift_labels.view(B * (T - 1)))
    loss.backward()
    np.savez_compressed(os.path.join(HERE, "loss.npz"), x=x.numpy(), w=w.numpy(), ids=ids.numpy().astype(np.int32),
                        mask=mask.numpy().astype(np.int32), loss=np.float32(loss.item()), x_g=xi.grad.numpy(),
                        w_g=wi.grad.numpy(), logits=logits.detach().numpy())
    print("wrote loss.npz loss=", loss.item())


def gen_inputs_fixture():
    """The reference's only data files (bloomz-7b/xinput.{ids,mask}.bin, [2,512] int32) are
    not copied.  Stored instead: the valid lengths, and SHA-256 digests of the loss targets
    and of the additive attention mask computed here with an independent numpy formulation,
    so a CPU test that can read the reference files checks the oracle's builders on them."""
    import hashlib
    ids = np.fromfile(os.path.join(REF, "bloomz-7b", "xinput.ids.bin"), dtype=np.int32).reshape(2, 512)
    mask = np.fromfile(os.path.join(REF, "bloomz-7b", "xinput.mask.bin"), dtype=np.int32).reshape(2, 512)
    B, T = ids.shape
    valid = (mask[:, :-1] != 0) & (mask[:, 1:] != 0)
    target = np.full((B, T), -100, np.int32)
    target[:, :-1] = np.where(valid, ids[:, 1:], -100)
    prefix_ok = np.cumprod(mask != 0, axis=1).astype(bool)           # keys before the first pad
    causal = np.tril(np.ones((T, T), bool))
    xmask = np.where(causal[None] & prefix_ok[:, None, :], np.float32(0), -np.finfo(np.float32).max).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "xinput_digest.npz"), lens=mask.sum(1).astype(np.int32),
                        items=np.int32(valid.sum()),
                        target_sha256=hashlib.sha256(target.tobytes()).hexdigest(),
                        xmask_sha256=hashlib.sha256(xmask.tobytes()).hexdigest())
    print("wrote xinput_digest.npz lens=", mask.sum(1), "items=", valid.sum())


if __name__ == "__main__":
    torch.set_num_threads(4)
    gen_block("block_small.npz", B=2, T=12, H=64, heads=4, lens=(12, 7), seed=7)
    gen_block("block_b3.npz", B=3, T=20, H=64, heads=8, lens=(20, 1, 13), seed=8)
    gen_pointwise()
    gen_loss()
    gen_inputs_fixture()
