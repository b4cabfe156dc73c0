"""Generator of the model scripts (the "words" programs the driver runs).

The reference ships two hand-written scripts for one fixed model size, `bloomz-7b/init.words`
and `bloomz-7b/train.words`.  The words they define -- create_layer_weight, create_layer_grad,
zero_layer_grad, create_var, create_dynamic, layer_forward, layer_backward -- are the interface
its driver calls (blackriver/train_bloom.cpp:128-192).  This module writes scripts that define
the same words, with the same tensor names and the same operator sequence per layer, for any
model size, element type ("float" or "half") and device, so one text serves the 1-layer fp32
parity configuration and the 30-layer fp16 model alike.

Differences from the reference layout (bloomz-7b/train.words:10-135), all inside create_dynamic:
LayerNorm statistics get one float per token (the reference reserves HIDDEN_SIZE floats, which
limits batch*tokens to HIDDEN_SIZE), every view starts on a 16-byte boundary, and the LM-head
weight is not overlaid on the activations.
"""

LAYER_WEIGHTS = (
    # name, shape expression (words), element count expression
    ("input_layernorm.weight", ["HIDDEN_SIZE"]),
    ("input_layernorm.bias", ["HIDDEN_SIZE"]),
    ("post_attention_layernorm.weight", ["HIDDEN_SIZE"]),
    ("post_attention_layernorm.bias", ["HIDDEN_SIZE"]),
    ("query_key_value.weight", ["HIDDEN_SIZE_x3", "HIDDEN_SIZE"]),
    ("query_key_value.bias", ["HIDDEN_SIZE_x3"]),
    ("dense.weight", ["HIDDEN_SIZE", "HIDDEN_SIZE"]),
    ("dense.bias", ["HIDDEN_SIZE"]),
    ("dense_h_to_4h.weight", ["HIDDEN_SIZE_x4", "HIDDEN_SIZE"]),
    ("dense_h_to_4h.bias", ["HIDDEN_SIZE_x4"]),
    ("dense_4h_to_h.weight", ["HIDDEN_SIZE", "HIDDEN_SIZE_x4"]),
    ("dense_4h_to_h.bias", ["HIDDEN_SIZE"]),
)


def _get(name):
    return f'"{name}" @'


def _dims(names):
    return " ".join(_get(n) for n in names) + f" {len(names)}"


def init_words(hidden, heads, vocab, eps=1e-5, dtype="float", max_tokens=8192, weights_path="model/weights/"):
    """Constants and the weight / gradient creation words (cf. bloomz-7b/init.words)."""
    assert hidden % heads == 0
    L = []
    w = L.append
    w(f'"{weights_path}" "MSG_FILES_PATH" !')
    for name, val in (("VOCAB_SIZE", vocab), ("HIDDEN_SIZE", hidden), ("HEADS_NUM", heads), ("HEAD_HIDDEN", hidden // heads),
                      ("LN_EPS", repr(float(eps))), ("HIDDEN_SIZE_x3", 3 * hidden), ("HIDDEN_SIZE_x4", 4 * hidden),
                      ("HIDDEN_SQUARE", hidden * hidden), ("MAX_TOKENS", max_tokens)):
        w(f'{val} "{name}" !')
    w(f'"{dtype}" "DTYPE" !')

    def creation(word, suffix):
        w(f"%def {word}")
        for name, dims in LAYER_WEIGHTS:
            w(f'    {_dims(dims)} $DEVICE @ "DTYPE" @ op.create "{name}{suffix}" !')
        # the fused QKV parameter seen as three [H,H] / [H] tensors: rows 0..H-1 query, then key, then value
        for i, part in enumerate(("query", "key", "value")):
            w(f'    "query_key_value.weight{suffix}" @ "HIDDEN_SQUARE" @ {i} * "HIDDEN_SIZE" @ dup 2 op.view "{part}.weight{suffix}" !')
            w(f'    "query_key_value.bias{suffix}" @ "HIDDEN_SIZE" @ {i} * "HIDDEN_SIZE" @ 1 op.view "{part}.bias{suffix}" !')
        w("%end")

    creation("create_layer_weight", "")
    creation("create_layer_grad", "_g")
    w("%def zero_layer_grad")
    for name, _ in LAYER_WEIGHTS:
        w(f'    "{name}_g" @ op.zero')
    w("%end")

    w("%def create_main_weight")
    for name in ("word_embeddings_layernorm", "ln_f"):
        for part in ("weight", "bias"):
            w(f'    "HIDDEN_SIZE" @ 1 "cuda" "DTYPE" @ op.create "{name}.{part}" !')
    w('    "VOCAB_SIZE" @ "HIDDEN_SIZE" @ 2 "cuda" "DTYPE" @ op.create "lm_head.weight" !')
    w("%end")
    w("%def create_main_grad")
    for name in ("word_embeddings_layernorm", "ln_f"):
        for part in ("weight", "bias"):
            w(f'    "HIDDEN_SIZE" @ 1 "cuda" "DTYPE" @ op.create "{name}.{part}_g" !')
    w('    "VOCAB_SIZE" @ "HIDDEN_SIZE" @ 2 "cuda" "DTYPE" @ op.create "lm_head.weight_g" !')
    w("%end")
    w("%def zero_main_grad")
    for name in ("word_embeddings_layernorm.weight", "word_embeddings_layernorm.bias", "ln_f.weight", "ln_f.bias", "lm_head.weight"):
        w(f'    "{name}_g" @ op.zero')
    w("%end")

    w("%def load_layer_weight")
    w('    "header" !')
    for name, _ in LAYER_WEIGHTS:
        w(f'    "{name}" @ "MSG_FILES_PATH" @ "header" @ | ".{name}.bin" | io.load')
    w('    "header" !!')
    w("%end")
    w("%def save_layer_weight")
    w('    "header" !')
    for name, _ in LAYER_WEIGHTS:
        w(f'    "{name}" @ "MSG_FILES_PATH" @ "header" @ | ".{name}.bin" | io.save')
    w('    "header" !!')
    w("%end")
    return "\n".join(L) + "\n"


def train_words():
    """create_var, create_dynamic, layer_forward, layer_backward (cf. bloomz-7b/train.words)."""
    L = []
    w = L.append
    # ( elements -- )  the single activation buffer plus host-side id / mask tensors
    w("%def create_var")
    w('    1 "cuda" "DTYPE" @ op.create "_var_" !')
    w('    "MAX_TOKENS" @ 4 * 1 "cuda" "float" op.create "_stat_" !')
    w('    "MAX_TOKENS" @ 1 "cpu" "int" op.create "_ids_" !')
    w('    "MAX_TOKENS" @ 1 "cpu" "int" op.create "_mask_" !')
    w("%end")

    BT = "$batch @ $tokens @"
    S = f"{BT} * \"HIDDEN_SIZE\" @ *"          # elements of one [B,T,H] activation
    views3 = f'{BT} "HIDDEN_SIZE" @ 3'
    views_y = f'{BT} "HEADS_NUM" @ "HEAD_HIDDEN" @ 4'
    views_z = f'$batch @ "HEADS_NUM" @ $tokens @ "HEAD_HIDDEN" @ 4'

    def carve(names_shapes, size_expr):
        """Views that share one region of _var_; the running offset stays on the stack."""
        for name, shape in names_shapes:
            w(f'    dup "_var_" @ swap {shape} op.view "{name}" !')
        w(f"    {size_expr} +")

    # ( batch tokens -- )
    w("%def create_dynamic")
    w("    0 #")
    w("    $tokens ! $batch !")
    w(f'    "_ids_" @ 0 {BT} 2 op.view "ids_" !')
    w(f'    "_mask_" @ 0 {BT} 2 op.view "mask_" !')
    # per-token LayerNorm statistics, fp32 whatever the activation type
    for i, name in enumerate(("ln_mean", "input_ln_var", "post_ln_var", "aux_ln_var")):
        w(f'    "_stat_" @ "MAX_TOKENS" @ {i} * {BT} * 1 op.view "{name}" !')
    w("    0")  # running element offset into _var_
    carve([("xinput", views3)], S)
    carve([("yout_g", views3)], S)
    carve([("alibi", f'1 "HEADS_NUM" @ 1 $tokens @ 4')], '"HEADS_NUM" @ $tokens @ *')
    carve([("xmask", f"$batch @ 1 $tokens @ $tokens @ 4")], f"{BT} $tokens @ * *")
    for n in ("a", "b", "c"):
        carve([(f"x{n}", views3), (f"y{n}", views_y), (f"z{n}", views_z)], S)
    carve([("xattn_in", views3)], S)
    carve([("xattn_out", views3), ("yattn_out", views_y)], S)
    for n in ("query", "key", "value"):
        carve([(f"x{n}", views3), (f"y{n}", views_y), (f"z{n}", views_z)], S)
    carve([("x4a", f'{BT} "HIDDEN_SIZE_x4" @ 3')], f"{S} 4 *")
    carve([("x4b", f'{BT} "HIDDEN_SIZE_x4" @ 3')], f"{S} 4 *")
    carve([("xll", f'$batch @ "HEADS_NUM" @ $tokens @ $tokens @ 4')], f'$batch @ "HEADS_NUM" @ * $tokens @ $tokens @ * *')
    # the rest of the buffer holds bands of logits for the loss
    w('    "_var_" @ swap 0 "VOCAB_SIZE" @ 2 op.view "all_logits" !')
    w("%end")

    def g(*names):
        return " ".join(_get(n) for n in names)

    w("%def layer_forward")
    w(f'    {g("xinput", "ln_mean", "input_ln_var", "input_layernorm.weight", "input_layernorm.bias", "xattn_in", "LN_EPS")} op.layernorm')
    for part, out in (("query", "xa"), ("key", "xb"), ("value", "xc")):
        w(f'    {g("xattn_in", part + ".weight", part + ".bias", out)} op.linear')
    for src, dst in (("ya", "zquery"), ("yb", "zkey"), ("yc", "zvalue")):
        w(f"    {g(src, dst)} op.transpos_0213")
    w(f'    {g("zquery", "zkey", "xll")} op.querykey')
    w(f'    {g("xll", "alibi", "xll")} op.add')
    w(f'    {g("xll", "xmask", "xll")} op.add')
    w(f'    {g("xll", "xll")} op.softmax')
    w(f'    {g("xll", "zvalue", "zc")} op.attn')
    w(f'    {g("zc", "yattn_out")} op.transpos_0213')
    w(f'    {g("xattn_out", "dense.weight", "dense.bias", "xb")} op.linear')
    w(f'    {g("xb", "xinput", "xa")} op.add')
    w(f'    {g("xa", "ln_mean", "post_ln_var", "post_attention_layernorm.weight", "post_attention_layernorm.bias", "xb", "LN_EPS")} op.layernorm')
    w(f'    {g("xb", "dense_h_to_4h.weight", "dense_h_to_4h.bias", "x4a")} op.linear')
    w(f'    {g("x4a", "x4b")} op.gelu')
    w(f'    {g("x4b", "dense_4h_to_h.weight", "dense_4h_to_h.bias", "xc")} op.linear')
    w(f'    {g("xa", "xc", "xa")} op.add')
    w("%end")

    w("%def layer_backward")
    w(f'    {g("yout_g", "x4b", "dense_4h_to_h.weight", "dense_4h_to_h.bias", "x4b", "dense_4h_to_h.weight_g", "dense_4h_to_h.bias_g")} op.linear_backward')
    w(f'    {g("x4b", "x4a", "x4a")} op.gelu_backward')
    w(f'    {g("x4a", "xb", "dense_h_to_4h.weight", "dense_h_to_4h.bias", "xa", "dense_h_to_4h.weight_g", "dense_h_to_4h.bias_g")} op.linear_backward')
    w(f'    {g("xa", "post_attention_layernorm.weight", "post_attention_layernorm.bias", "post_ln_var", "xb", "post_attention_layernorm.weight_g", "post_attention_layernorm.bias_g", "xc", "LN_EPS")} op.layernorm_backward')
    w(f'    {g("yout_g", "xc", "yout_g")} op.add')
    w(f'    {g("yout_g", "xattn_out", "dense.weight", "dense.bias", "xa", "dense.weight_g", "dense.bias_g")} op.linear_backward')
    w(f'    {g("ya", "zb")} op.transpos_0213')
    w(f'    {g("zb", "xll", "zvalue", "xll", "za")} op.softmax_attn_backward')
    w(f'    {g("xll", "zquery", "zkey", "zb", "zc")} op.qk_backward')
    for src, dst in (("za", "yvalue"), ("zb", "yquery"), ("zc", "ykey")):
        w(f"    {g(src, dst)} op.transpos_0213")
    w(f'    {g("xa")} op.zero')
    for part in ("query", "key", "value"):
        w(f'    {g("x" + part, "xattn_in", part + ".weight", part + ".bias", "xb", part + ".weight_g", part + ".bias_g")} op.linear_backward')
        w(f'    {g("xa", "xb", "xa")} op.add')
    w(f'    {g("xa", "input_layernorm.weight", "input_layernorm.bias", "input_ln_var", "xattn_in", "input_layernorm.weight_g", "input_layernorm.bias_g", "xb", "LN_EPS")} op.layernorm_backward')
    w(f'    {g("xb", "yout_g", "xa")} op.add')
    w("%end")
    return "\n".join(L) + "\n"


def var_elements(batch, tokens, hidden, heads, vocab, logits_rows):
    """Elements `create_var` must reserve for `create_dynamic(batch, tokens)` plus a logits band."""
    s = batch * tokens * hidden
    n = 2 * s + heads * tokens + batch * tokens * tokens + 3 * s + 2 * s + 3 * s + 8 * s + batch * heads * tokens * tokens
    return n + logits_rows * vocab


# ==========================================================================================
# Fused training scripts: whole model (or one pipeline stage of it) resident in HBM.
#
# Hash table 0 holds the constants, the stage-level parameters (embedding table / LM head,
# embedding LayerNorm, final LayerNorm), the input tensors and the gradient scratch shared by all
# layers; hash table i (1..n_layers) holds layer i-1 of the stage: its parameters as views of one
# flat buffer (so the optimizer is one launch per layer), the matching flat gradient / master /
# moment buffers, and the activations its backward pass needs.  Where the reference copies a
# layer's weights from host memory into one device working set before every use (sync_layer,
# bloomz-7b/init.words:237-293), here a layer is "brought in" by switching the hash table.
# ==========================================================================================
def _layer_param_layout(hidden):
    """(name, shape, elements) in flat-buffer order; every offset is a multiple of 8 elements."""
    h = hidden
    spec = [
        ("input_layernorm.weight", (h,)), ("input_layernorm.bias", (h,)),
        ("query_key_value.weight", (3 * h, h)), ("query_key_value.bias", (3 * h,)),
        ("dense.weight", (h, h)), ("dense.bias", (h,)),
        ("post_attention_layernorm.weight", (h,)), ("post_attention_layernorm.bias", (h,)),
        ("dense_h_to_4h.weight", (4 * h, h)), ("dense_h_to_4h.bias", (4 * h,)),
        ("dense_4h_to_h.weight", (h, 4 * h)), ("dense_4h_to_h.bias", (h,)),
    ]
    out, off = [], 0
    for name, shape in spec:
        n = 1
        for d in shape:
            n *= d
        out.append((name, shape, off, n))
        off += (n + 7) // 8 * 8
    return out, off


def layer_param_elements(hidden):
    return _layer_param_layout(hidden)[1]


# tensors of the two halves of a layer: "A" = input LayerNorm, QKV, attention, dense (+ residual); "M" = post-attention
# LayerNorm, h -> 4h (+ GELU), 4h -> h (+ residual)
HALF_PARAMS = {
    "A": ("input_layernorm.weight", "input_layernorm.bias", "query_key_value.weight", "query_key_value.bias", "dense.weight", "dense.bias"),
    "M": ("post_attention_layernorm.weight", "post_attention_layernorm.bias", "dense_h_to_4h.weight", "dense_h_to_4h.bias",
          "dense_4h_to_h.weight", "dense_4h_to_h.bias"),
}
# saved activations (per slot) and gradients kept for a deferred weight-gradient pass (per slot, overlap only)
HALF_SAVED = {"A": (("xattn_in", 1), ("qkv", 3), ("attn_out", 1)), "M": (("xb", 1), ("x4a", 4), ("x4b", 4))}
HALF_STATS = {"A": ("input_ln_var",), "M": ("post_ln_var",)}


def fused_words(hidden, heads, vocab, n_layers, batch, tokens, dtype="half", eps=1e-5, first_stage=True, last_stage=True,
                logits_rows=None, init_std=0.02, seed=0, layer_offset=0, n_slots=1, prev_rank=None, next_rank=None,
                overlap=False, n_micro=1, kinds=None, async_optimizer=False):
    """Script text defining the whole stage.  After executing it:
         build_model            allocates everything (call once)
         init_model             seeded random initialisation (weights N(0, init_std), biases 0, LN 1/0)
         model_forward / model_backward / zero_grads / ( lr step grad_scale -- ) optimizer_step
         model_score            after model_forward, on the last stage: per-token next-token NLL into "token_nll" (fp32
                                [batch, tokens], 0 where no target is counted), forward only; stage_score = stage_forward + it
       Inputs: one device int tensor "inp" in hash 0 holding ids [batch, tokens], mask [batch, tokens] and lens [batch]
       back to back (the views "ids_", "mask_", "lens_" are what the operators read).  On a stage that is not the first
       the incoming activations are "stage_in" and the outgoing gradient is "stage_in_g"; on a stage that is not the
       last "stage_out" / "stage_out_g" play the same roles.
       Pipeline use: n_slots > 1 keeps that many micro-batches' saved activations at once; `slot_k` selects the set the
       next forward / backward works on, and stage_forward / stage_backward add the NCCL receive from / send to
       prev_rank and next_rank around model_forward / model_backward.
       A last stage that is not also the first may have n_layers == 0 (final LayerNorm + LM head only).

       overlap=True (needs n_slots > 1 and the one-sided links, `io.link.open` being part of build_model) defines the
       three tasks of the overlapped schedule instead, each preceded by `slot_k` (k = micro-batch % n_slots):
         stage_f      wait for the activations in this slot's window, forward, send on, release the window
         ( name -- ) stage_b   input gradients only (the micro-batch's mean loss goes to the view of "loss_all" called
                      name, "loss@j"); send to the previous rank
         stage_w      weight gradients of the slot's micro-batch from the kept dy tensors; releases the gradient window
       The stage's incoming tensors are then the link windows themselves (no copy on arrival).

       kinds (overlap only): one entry per layer hash of the stage, "AM" for a whole layer, "M" when only the MLP half
       of the stage's first layer is here (its attention half closes the previous stage) and "A" when only the
       attention half of the last layer is here.  layer_offset is the model-wide index of the stage's first layer."""
    assert n_layers >= 1 or (last_stage and not first_stage)
    assert not overlap or (n_slots > 1 and not (first_stage and last_stage))
    kinds = list(kinds) if kinds is not None else ["AM"] * n_layers
    assert len(kinds) == n_layers and all(k in ("AM", "A", "M") for k in kinds)
    assert all(k == "AM" for k in kinds[1:-1]) and (n_layers < 2 or ("A" in kinds[-1] and "M" in kinds[0]))
    assert overlap or all(k == "AM" for k in kinds), "half layers exist in the overlapped pipeline only"
    assert not (first_stage and kinds and "A" not in kinds[0]) and not (last_stage and kinds and "M" not in kinds[-1])

    def slot_names(name):
        return [name] if n_slots == 1 else [f"{name}@{k}" for k in range(n_slots)]
    assert hidden % heads == 0 and hidden % 8 == 0
    layout, flat = _layer_param_layout(hidden)
    n = batch * tokens
    logits_rows = logits_rows or n
    L = []
    w = L.append
    for name, val in (("VOCAB_SIZE", vocab), ("HIDDEN_SIZE", hidden), ("HEADS_NUM", heads), ("HEAD_HIDDEN", hidden // heads),
                      ("LN_EPS", repr(float(eps))), ("HIDDEN_SIZE_x3", 3 * hidden), ("HIDDEN_SIZE_x4", 4 * hidden),
                      ("LAYER_PARAMS", flat), ("TOKENS", n)):
        w(f'{val} "{name}" !')
    w(f'"{dtype}" "DTYPE" !')
    w(f"{batch} $batch !  {tokens} $tokens !")
    BTH = f'{batch} {tokens} "HIDDEN_SIZE" @ 3'

    def g(*names):
        return " ".join(_get(x) for x in names)

    def act(name, cols, slotted):
        for nm in (slot_names(name) if slotted else [name]):
            w(f'    {batch} {tokens} {cols * hidden} 3 "cuda" "{dtype}" op.create "{nm}" !')

    # names a layer of a given kind reads / writes at its two ends
    def in_name(kind):
        return "xinput" if "A" in kind else "xa"

    def out_name(kind):
        return "xout" if "M" in kind else "xa"

    def gin_name(kind):          # gradient arriving from the layer (or stage) after it
        return "yout_g" if "M" in kind else "dh2"

    def gout_name(kind):         # gradient handed to the layer (or stage) before it
        return "xin_g" if "A" in kind else "dh2"

    # ---- per-kind words (run inside the layer's hash table, so sizes and types are spelled out) ----
    for kind in sorted(set(kinds)) or ["AM"]:
        tag = "fused" if kind == "AM" else kind
        w(f"%def create_layer_{tag}")
        # the parameter buffers are whole-layer sized for every kind (one optimizer launch per layer hash; the half
        # that lives on another rank just never receives a gradient)
        for suffix, dt in (("", dtype), ("_g", dtype), (".master", "float"), (".m", "float"), (".v", "float")):
            w(f'    {flat} 1 "cuda" "{dt}" op.create "_flat{suffix}" !')
        for suffix in ("", "_g", ".master", ".m", ".v"):     # fp32 master / moment views are what a checkpoint stores
            for name, shape, off, cnt in layout:
                dims = " ".join(str(d) for d in shape)
                w(f'    "_flat{suffix}" @ {off} {dims} {len(shape)} op.view "{name}{suffix}" !')
        for half in "AM":
            if half not in kind:
                continue
            for name, cols in HALF_SAVED[half]:
                act(name, cols, True)
            for name in HALF_STATS[half]:
                for nm in slot_names(name):
                    w(f'    {n} 1 "cuda" "float" op.create "{nm}" !')
        if "A" in kind:
            for nm in slot_names("lse"):
                w(f'    {batch} {heads} {tokens} 3 "cuda" "float" op.create "{nm}" !')
            if overlap:
                act("dqkv", 3, True)
                if "M" in kind:
                    act("dh2", 1, True)          # an "A" layer's dh2 is the gradient that arrives from the next stage
        if "M" in kind and overlap:
            act("d4", 4, True)
            act("yout_g", 1, True)               # what the layer after this one writes (bound as its outgoing gradient)
        if kind == "AM" or kind == "A":
            act("xa", 1, False)                  # for "M" the stage's incoming window plays this part
        if "M" in kind:
            act("xout", 1, False)
        w(f'    {n} 1 "cuda" "float" op.create "ln_mean" !')
        w("%end")

        def forward_A():
            w(f'    {g("xinput", "ln_mean", "input_ln_var", "input_layernorm.weight", "input_layernorm.bias", "xattn_in", "LN_EPS")} op.layernorm')
            w(f'    {g("xattn_in", "query_key_value.weight", "query_key_value.bias", "qkv")} op.linear')
            w(f'    {g("qkv", "lens_", "attn_out", "lse", "HEADS_NUM")} op.flash_attn')
            w(f'    {g("attn_out", "dense.weight", "dense.bias", "xinput", "xa")} op.linear_residual')

        def forward_M():
            w(f'    {g("xa", "ln_mean", "post_ln_var", "post_attention_layernorm.weight", "post_attention_layernorm.bias", "xb", "LN_EPS")} op.layernorm')
            w(f'    {g("xb", "dense_h_to_4h.weight", "dense_h_to_4h.bias", "x4a", "x4b")} op.linear_gelu')
            w(f'    {g("x4b", "dense_4h_to_h.weight", "dense_4h_to_h.bias", "xa", "xout")} op.linear_residual')

        w(f"%def layer_forward_{tag}")
        if "A" in kind:
            forward_A()
        if "M" in kind:
            forward_M()
        w("%end")

        if kind == "AM":
            w("%def layer_backward_fused")
            w(f'    {g("yout_g", "x4b", "dense_4h_to_h.weight", "dense_4h_to_h.bias", "d4", "dense_4h_to_h.weight_g", "dense_4h_to_h.bias_g")} op.linear_backward')
            w(f'    {g("d4", "x4a", "d4")} op.gelu_backward')
            w(f'    {g("d4", "xb", "dense_h_to_4h.weight", "dense_h_to_4h.bias", "dh1", "dense_h_to_4h.weight_g", "dense_h_to_4h.bias_g")} op.linear_backward')
            w(f'    {g("dh1", "post_attention_layernorm.weight", "post_attention_layernorm.bias", "post_ln_var", "xb", "post_attention_layernorm.weight_g", "post_attention_layernorm.bias_g", "dh2", "yout_g", "LN_EPS")} op.layernorm_backward_residual')
            w(f'    {g("dh2", "attn_out", "dense.weight", "dense.bias", "dh1", "dense.weight_g", "dense.bias_g")} op.linear_backward')
            w(f'    {g("dh1", "qkv", "attn_out", "lse", "lens_", "dqkv", "HEADS_NUM")} op.flash_attn_backward')
            w(f'    {g("dqkv", "xattn_in", "query_key_value.weight", "query_key_value.bias", "dh1", "query_key_value.weight_g", "query_key_value.bias_g")} op.linear_backward')
            w(f'    {g("dh1", "input_layernorm.weight", "input_layernorm.bias", "input_ln_var", "xattn_in", "input_layernorm.weight_g", "input_layernorm.bias_g", "xin_g", "dh2", "LN_EPS")} op.layernorm_backward_residual')
            w("%end")

        # the same backward in two passes: input gradients (what the previous stage waits for), then weight gradients
        w(f"%def layer_backward_x_{tag}")
        if "M" in kind:
            w(f'    {g("yout_g", "dense_4h_to_h.weight", "d4")} op.linear_backward_x')
            w(f'    {g("d4", "x4a", "d4")} op.gelu_backward')
            w(f'    {g("d4", "dense_h_to_4h.weight", "dh1")} op.linear_backward_x')
            w(f'    {g("dh1", "post_attention_layernorm.weight", "post_attention_layernorm.bias", "post_ln_var", "xb", "post_attention_layernorm.weight_g", "post_attention_layernorm.bias_g", "dh2", "yout_g", "LN_EPS")} op.layernorm_backward_residual')
        if "A" in kind:
            w(f'    {g("dh2", "dense.weight", "dh1")} op.linear_backward_x')
            w(f'    {g("dh1", "qkv", "attn_out", "lse", "lens_", "dqkv", "HEADS_NUM")} op.flash_attn_backward')
            w(f'    {g("dqkv", "query_key_value.weight", "dh1")} op.linear_backward_x')
            w(f'    {g("dh1", "input_layernorm.weight", "input_layernorm.bias", "input_ln_var", "xattn_in", "input_layernorm.weight_g", "input_layernorm.bias_g", "xin_g", "dh2", "LN_EPS")} op.layernorm_backward_residual')
        w("%end")
        w(f"%def layer_backward_w_{tag}")
        if "M" in kind:
            w(f'    {g("yout_g", "x4b", "dense_4h_to_h.weight_g", "dense_4h_to_h.bias_g")} op.linear_backward_w')
            w(f'    {g("d4", "xb", "dense_h_to_4h.weight_g", "dense_h_to_4h.bias_g")} op.linear_backward_w')
        if "A" in kind:
            w(f'    {g("dh2", "attn_out", "dense.weight_g", "dense.bias_g")} op.linear_backward_w')
            w(f'    {g("dqkv", "xattn_in", "query_key_value.weight_g", "query_key_value.bias_g")} op.linear_backward_w')
        w("%end")

    # ---- ( seed -- ) seeded initialisation of one layer (every tensor, whichever half is used here: the two ranks that
    # share a layer then hold the same values as a single-stage model) ----
    w("%def init_layer_fused")
    w('    "seed_" !')
    w('    "_flat" @ op.zero')
    for i, (name, shape, off, cnt) in enumerate(layout):
        if name.endswith("layernorm.weight"):
            w(f'    "{name}" @ 1.0 op.fill')
        elif name.endswith(".weight"):
            w(f'    "{name}" @ 0.0 {init_std} "seed_" @ 100 * {i} + op.randn')
    w('    "_flat.master" @ "_flat" @ op.copy  "_flat.m" @ op.zero  "_flat.v" @ op.zero  "_flat_g" @ op.zero')
    w('    "seed_" !!')
    w("%end")

    def tag_of(i):
        return "fused" if kinds[i - 1] == "AM" else kinds[i - 1]

    # ---- whole stage ----
    act_bytes = batch * tokens * hidden * (2 if dtype == "half" else 4)
    n_logit_bufs = n_slots if (overlap and last_stage) else 1      # a deferred LM-head weight gradient keeps its dlogits
    w("%def build_model")
    w("    0 #")
    # token ids, mask and lengths of the micro-batch being worked on, on the device (one buffer, three views)
    w(f'    {2 * n + batch} 1 "cuda" "int" op.create "inp" !')
    w(f'    "inp" @ 0 {batch} {tokens} 2 op.view "ids_" !  "inp" @ {n} {batch} {tokens} 2 op.view "mask_" !  "inp" @ {2 * n} {batch} 1 op.view "lens_" !')
    w(f'    {max(n_micro, 1)} 1 "cuda" "float" op.create "loss_all" !')
    for j in range(max(n_micro, 1)):
        w(f'    "loss_all" @ {j} 1 1 op.view "loss@{j}" !')
    shared_scratch = [("dh1", 1), ("gA", 1), ("gB", 1)] + ([] if overlap else [("d4", 4), ("dqkv", 3), ("dh2", 1)])
    for name, cols in shared_scratch:
        w(f'    {batch} {tokens} {cols * hidden} 3 "cuda" "DTYPE" @ op.create "{name}" !')
    w(f'    {n} 1 "cuda" "float" op.create "ln_mean" !')
    for nm in slot_names("emb_ln_var") + slot_names("ln_f_var"):
        w(f'    {n} 1 "cuda" "float" op.create "{nm}" !')
    if overlap:
        w(f"    {act_bytes} {n_slots} io.link.open")
    main_params = []
    if first_stage:
        main_params += [("word_embeddings.weight", (vocab, hidden)), ("word_embeddings_layernorm.weight", (hidden,)),
                        ("word_embeddings_layernorm.bias", (hidden,))]
        w(f'    {BTH} "cuda" "DTYPE" @ op.create "emb_raw" !')
        for nm in slot_names("emb_out"):
            w(f'    {BTH} "cuda" "DTYPE" @ op.create "{nm}" !')
    elif overlap:
        for k in range(n_slots):          # the activations arrive in this rank's own windows
            w(f'    0 {k} {BTH} "DTYPE" @ io.link.window "stage_in@{k}" !')
    else:
        w(f'    {BTH} "cuda" "DTYPE" @ op.create "stage_in" !')
    if last_stage:
        if not first_stage:
            main_params += [("word_embeddings.weight", (vocab, hidden))]       # the tied LM head lives on this stage too
        main_params += [("ln_f.weight", (hidden,)), ("ln_f.bias", (hidden,))]
        w(f'    {BTH} "cuda" "DTYPE" @ op.create "xf_g" !')
        for nm in slot_names("xf"):
            w(f'    {BTH} "cuda" "DTYPE" @ op.create "{nm}" !')
        if n_logit_bufs == 1:
            w(f'    {logits_rows} "VOCAB_SIZE" @ 2 "cuda" "DTYPE" @ op.create "all_logits" !')
        else:
            assert logits_rows >= n, "deferring the LM-head weight gradient needs a logits band that covers the micro-batch"
            for k in range(n_logit_bufs):
                w(f'    {logits_rows} "VOCAB_SIZE" @ 2 "cuda" "DTYPE" @ op.create "all_logits@{k}" !')
        w(f'    {batch} {tokens} 2 "cuda" "float" op.create "token_nll" !')
        if overlap and n_layers >= 1:
            for k in range(n_slots):      # what the final LayerNorm's backward hands to the last layer, kept for its W pass
                w(f'    {BTH} "cuda" "DTYPE" @ op.create "stage_out_g@{k}" !')
    elif overlap:
        for k in range(n_slots):          # the gradients arrive in this rank's own windows
            w(f'    1 {k} {BTH} "DTYPE" @ io.link.window "stage_out_g@{k}" !')
    for name, shape in main_params:
        dims = " ".join(str(d) for d in shape)
        for suffix, dt in (("", '"DTYPE" @'), ("_g", '"DTYPE" @'), (".master", '"float"'), (".m", '"float"'), (".v", '"float"')):
            w(f'    {dims} {len(shape)} "cuda" {dt} op.create "{name}{suffix}" !')
    if (first_stage != last_stage) and (prev_rank is not None or next_rank is not None):
        w(f'    "VOCAB_SIZE" @ "HIDDEN_SIZE" @ 2 "cuda" "DTYPE" @ op.create "tied_recv" !')
    for i in range(1, n_layers + 1):
        w(f"    {i} # create_layer_{tag_of(i)}")
    # bindings: scratch and inputs into every layer hash; activations chained layer to layer
    shared = ("dh1", "lens_", "LN_EPS", "HEADS_NUM") + (() if overlap else ("d4", "dqkv", "dh2"))
    for i in range(1, n_layers + 1):
        kind = kinds[i - 1]
        for name in shared:
            w(f'    0 # "{name}" @ {i} # "{name}" !')
        src = (f'{i - 1} # "{out_name(kinds[i - 2])}" @' if i > 1 else ('0 # "emb_out" @' if first_stage else '0 # "stage_in" @'))
        if not (i == 1 and n_slots > 1 and (first_stage or overlap)):      # with slots the stage input is bound by slot_k
            w(f'    {src} {i} # "{in_name(kind)}" !')
        if not overlap:
            # gradient buffers alternate so a layer never reads and writes the same one
            gin, gout = ("gA", "gB") if (n_layers - i) % 2 == 0 else ("gB", "gA")
            w(f'    0 # "{gin}" @ {i} # "yout_g" !  0 # "{gout}" @ {i} # "xin_g" !')
    w("    0 #")
    if overlap:
        # every layer keeps its incoming gradient per slot (bound by slot_k); the first layer's outgoing gradient
        # is a shared buffer, consumed at once (embedding backward) or copied out by the link before it is reused
        if n_layers >= 1:
            w(f'    "gA" @ 1 # "{gout_name(kinds[0])}" !  0 #  "gA" @ "stage_in_g" !  {n_layers} # "{out_name(kinds[-1])}" @ 0 # "stage_out" !')
        else:
            w('    "gA" @ "stage_in_g" !')
    elif n_layers >= 1:
        w(f'    {n_layers} # "xout" @ 0 # "stage_out" !  {n_layers} # "yout_g" @ 0 # "stage_out_g" !  1 # "xin_g" @ 0 # "stage_in_g" !  0 #')
    else:             # head-only stage: what arrives is what the final LayerNorm reads
        w('    "stage_in" @ "stage_out" !  "gA" @ "stage_out_g" !  "gA" @ "stage_in_g" !')
    w("%end")

    # ---- slot selection: which micro-batch's saved activations the layer words see ----
    def slotted_of(kind):
        names = []
        for half in "AM":
            if half in kind:
                names += [nm for nm, _ in HALF_SAVED[half]] + list(HALF_STATS[half])
        if "A" in kind:
            names.append("lse")
            if overlap:
                names.append("dqkv")
                if "M" in kind:
                    names.append("dh2")
        if "M" in kind and overlap:
            names.append("d4")
        return names

    for k in range(n_slots):
        w(f"%def slot_{k}")
        if n_slots > 1:
            w("    0 #")
            w(f'    {k} "slot_" !')
            for name in (["emb_out", "emb_ln_var"] if first_stage else []) + (["xf", "ln_f_var"] if last_stage else []):
                w(f'    "{name}@{k}" @ "{name}" !')
            if overlap:
                if not first_stage:
                    w(f'    "stage_in@{k}" @ "stage_in" !')
                if not (last_stage and n_layers == 0):
                    w(f'    "stage_out_g@{k}" @ "stage_out_g" !')
                if last_stage and n_logit_bufs > 1:
                    w(f'    "all_logits@{k}" @ "all_logits" !')
                if n_layers == 0:
                    w('    "stage_in" @ "stage_out" !')
            if first_stage:
                w(f'    "emb_out" @ 1 # "xinput" ! 0 #')
            elif overlap and n_layers >= 1:
                w(f'    "stage_in" @ 1 # "{in_name(kinds[0])}" ! 0 #')
            for i in range(1, n_layers + 1):
                kind = kinds[i - 1]
                w(f"    {i} #  " + "  ".join(f'"{name}@{k}" @ "{name}" !' for name in slotted_of(kind)))
                if overlap:
                    # layer i reads the gradient the layer after it (or the stage's successor) produced for this slot
                    if i < n_layers:
                        w(f'    "yout_g@{k}" @ "yout_g" !')
                    else:
                        w(f'    0 # "stage_out_g" @ {i} # "{gin_name(kind)}" !')
                    if i > 1:
                        w(f'    {i - 1} # "yout_g@{k}" @ {i} # "{gout_name(kind)}" !')
        w("    0 #")
        w("%end")

    w("%def init_model")
    w("    0 #")
    sd = seed * 1000003
    for k, (name, shape) in enumerate(main_params):
        if name.endswith("layernorm.weight") or name == "ln_f.weight":
            w(f'    "{name}" @ 1.0 op.fill')
        elif name.endswith(".bias"):
            w(f'    "{name}" @ op.zero')
        else:
            w(f'    "{name}" @ 0.0 {init_std} {sd + 7} op.randn')       # same seed on every stage that holds the tied table
        w(f'    "{name}.master" @ "{name}" @ op.copy  "{name}.m" @ op.zero  "{name}.v" @ op.zero  "{name}_g" @ op.zero')
    for i in range(1, n_layers + 1):
        w(f"    {i} # {sd + 11 + layer_offset + i} init_layer_fused")
    w("    0 #")
    w("%end")

    w("%def zero_grads")
    w("    0 #")
    for name, _ in main_params:
        w(f'    "{name}_g" @ op.zero')
    for i in range(1, n_layers + 1):
        w(f'    {i} # "_flat_g" @ op.zero')
    w("    0 #")
    w("%end")

    w("%def model_forward")
    w("    0 #")
    # with the optimizer on the side stream (optimizer_async) every group of parameters is waited for where it is first
    # read: mark 0 = the stage-level parameters, mark i = layer i
    if first_stage:
        if async_optimizer:
            w("    0 op.event.wait")
        w(f'    {g("ids_", "word_embeddings.weight", "emb_raw")} op.embed')
        w(f'    {g("emb_raw", "ln_mean", "emb_ln_var", "word_embeddings_layernorm.weight", "word_embeddings_layernorm.bias", "emb_out", "LN_EPS")} op.layernorm')
    for i in range(1, n_layers + 1):
        if async_optimizer:
            w(f"    {i} op.event.wait")
        w(f"    {i} # layer_forward_{tag_of(i)}")
    w("    0 #")
    if last_stage:
        if async_optimizer and not first_stage:
            w("    0 op.event.wait")
        w(f'    {g("stage_out", "ln_mean", "ln_f_var", "ln_f.weight", "ln_f.bias", "xf", "LN_EPS")} op.layernorm')
    w("%end")

    # forward-only scoring (prefill): per-token NLL of the next token into "token_nll", mean kept for op.last_loss
    w("%def model_score")
    w("    0 #")
    if last_stage:
        w(f'    {g("xf", "ids_", "mask_", "word_embeddings.weight", "all_logits", "token_nll")} op.token_nll')
    w("%end")

    def embedding_backward():
        w(f'    {g("stage_in_g", "word_embeddings_layernorm.weight", "word_embeddings_layernorm.bias", "emb_ln_var", "emb_out", "word_embeddings_layernorm.weight_g", "word_embeddings_layernorm.bias_g", "emb_raw", "LN_EPS")} op.layernorm_backward')
        w(f'    {g("emb_raw", "ids_", "word_embeddings.weight_g")} op.embed_backward')

    if not overlap:
        w("%def model_backward")
        w("    0 #")
        if last_stage:
            w(f'    {g("xf", "ids_", "mask_", "word_embeddings.weight", "all_logits", "xf_g", "word_embeddings.weight_g")} op.loss_backward')
            w(f'    {g("xf_g", "ln_f.weight", "ln_f.bias", "ln_f_var", "xf", "ln_f.weight_g", "ln_f.bias_g", "stage_out_g", "LN_EPS")} op.layernorm_backward')
        for i in range(n_layers, 0, -1):
            w(f"    {i} # layer_backward_fused")
        w("    0 #")
        if first_stage:
            embedding_backward()
        w("%end")

        # ( name -- ) the same backward queued without any host round trip; name = the one-element view of "loss_all"
        # that receives this micro-batch's mean loss ("loss@j")
        w("%def model_backward_async")
        w('    0 # @ "loss_" !')
        if last_stage:
            w(f'    {g("xf", "ids_", "mask_", "word_embeddings.weight", "all_logits", "xf_g", "word_embeddings.weight_g", "loss_")} 0 op.loss_backward_async')
            w(f'    {g("xf_g", "ln_f.weight", "ln_f.bias", "ln_f_var", "xf", "ln_f.weight_g", "ln_f.bias_g", "stage_out_g", "LN_EPS")} op.layernorm_backward')
        for i in range(n_layers, 0, -1):
            w(f"    {i} # layer_backward_fused")
        w("    0 #")
        if first_stage:
            embedding_backward()
        w('    0 # "loss_" !!')
        w("%end")

    # ( lr step grad_scale -- )  Adam on every parameter of the stage; optimizer_layers / optimizer_main are its two parts
    adam = '"lr_" @ 0.9 0.999 1e-08 "step_" @ "gs_" @ op.adam'
    w("%def optimizer_layers")
    w('    0 #  "gs_" ! "step_" ! "lr_" !')
    for i in range(1, n_layers + 1):
        w(f'    0 # "lr_" @ "step_" @ "gs_" @  {i} # "gs_" ! "step_" ! "lr_" !  {g("_flat", "_flat_g", "_flat.master", "_flat.m", "_flat.v")} {adam}  "gs_" !! "step_" !! "lr_" !!')
    w('    0 #  "gs_" !! "step_" !! "lr_" !!')
    w("%end")
    w("%def optimizer_main")
    w('    0 #  "gs_" ! "step_" ! "lr_" !')
    for name, _ in main_params:
        w(f'    {g(name, name + "_g", name + ".master", name + ".m", name + ".v")} {adam}')
    w('    "gs_" !! "step_" !! "lr_" !!')
    w("%end")
    w("%def optimizer_step")
    w('    0 #  "all_gs_" ! "all_step_" ! "all_lr_" !')
    w('    "all_lr_" @ "all_step_" @ "all_gs_" @ optimizer_main  0 # "all_lr_" @ "all_step_" @ "all_gs_" @ optimizer_layers')
    w('    0 #  "all_gs_" !! "all_step_" !! "all_lr_" !!')
    w("%end")

    if async_optimizer:
        # ( lr step grad_scale -- ) / ( peer lr step grad_scale -- )  the same update queued on the transfer stream, so that
        # it runs beside the next step's first forward: every group of parameters is followed by the clearing of its
        # gradients and by a mark that the forward waits for (model_forward), and the groups come in the order in which
        # the forward reads them -- the stage-level parameters first on the stage that embeds, last on the others.
        # The tied-table exchange, where there is one, is queued first so that the peer is not kept waiting.
        def main_group():
            for name, _ in main_params:
                w(f'    {g(name, name + "_g", name + ".master", name + ".m", name + ".v")} {adam}  "{name}_g" @ op.zero')
            w("    0 op.event.record")

        def layer_groups():
            for i in range(1, n_layers + 1):
                w(f'    0 # "lr_" @ "step_" @ "gs_" @  {i} # "gs_" ! "step_" ! "lr_" !  {g("_flat", "_flat_g", "_flat.master", "_flat.m", "_flat.v")} {adam}  "_flat_g" @ op.zero  "gs_" !! "step_" !! "lr_" !!  {i} op.event.record')
            w("    0 #")

        for tied in (False, True):
            w("%def optimizer_async_tied" if tied else "%def optimizer_async")
            w('    0 #  "gs_" ! "step_" ! "lr_" !' + ('  "peer_" !' if tied else ""))
            w("    1 op.stream.side")
            if tied:
                w('    "word_embeddings.weight_g" @ "tied_recv" @ "peer_" @ io.nccl.sendrecv')
            add_tied = '    "word_embeddings.weight_g" @ "tied_recv" @ "word_embeddings.weight_g" @ op.add'
            if first_stage:
                if tied:
                    w(add_tied)
                main_group()
                layer_groups()
            else:
                layer_groups()
                if tied:
                    w(add_tied)
                main_group()
            w("    0 op.stream.side")
            w('    0 #  "gs_" !! "step_" !! "lr_" !!' + ('  "peer_" !!' if tied else ""))
            w("%end")

    if overlap:
        # ---- the three tasks of the overlapped schedule (each runs after slot_k) ----
        w("%def stage_f")
        w("    0 #")
        if prev_rank is not None:
            w('    0 "slot_" @ io.link.wait')
        if next_rank is not None:
            w("    1 io.link.fence")                 # the previous micro-batch's output has left "stage_out"
        w("    model_forward")
        if next_rank is not None:
            w('    0 # "stage_out" @ 1 "slot_" @ io.link.send')
        if prev_rank is not None:
            w('    0 # 0 "slot_" @ io.link.release')
        w("%end")
        w("%def stage_score")
        w("    stage_f model_score")
        w("%end")
        w("%def stage_b")                            # ( name -- )  name = the view of "loss_all" for this micro-batch
        w('    0 # @ "loss_" !')
        if next_rank is not None:
            w('    1 "slot_" @ io.link.wait')
        if prev_rank is not None:
            w("    0 io.link.fence")                 # the previous micro-batch's gradient has left "stage_in_g"
        if last_stage:
            # the LM-head weight gradient waits for stage_w; with no layers on this stage the final LayerNorm writes
            # straight into the buffer that is sent back
            w(f'    {g("xf", "ids_", "mask_", "word_embeddings.weight", "all_logits", "xf_g", "word_embeddings.weight_g", "loss_")} 1 op.loss_backward_async')
            dst = "stage_out_g" if n_layers >= 1 else "stage_in_g"
            w(f'    {g("xf_g", "ln_f.weight", "ln_f.bias", "ln_f_var", "xf", "ln_f.weight_g", "ln_f.bias_g", dst, "LN_EPS")} op.layernorm_backward')
        for i in range(n_layers, 0, -1):
            w(f"    {i} # layer_backward_x_{tag_of(i)}")
        w("    0 #")
        if first_stage:
            embedding_backward()
        if prev_rank is not None:
            w('    "stage_in_g" @ 0 "slot_" @ io.link.send')
        w('    "loss_" !!')
        w("%end")
        # the LM-head part of stage_w on its own (the tied table's gradient is complete once every micro-batch's has run,
        # so a list may take these first and start the exchange of that gradient before the layers' parts: stage_wl)
        w("%def stage_h")
        w("    0 #")
        if last_stage:
            w(f'    {g("all_logits", "xf", "word_embeddings.weight_g")} op.loss_backward_w')
        w("%end")
        w("%def stage_wl")
        w("    0 #")
        for i in range(n_layers, 0, -1):
            w(f"    {i} # layer_backward_w_{tag_of(i)}")
        w("    0 #")
        if next_rank is not None:
            w('    1 "slot_" @ io.link.release')
        w("%end")
        w("%def stage_w")
        w("    0 #")
        if last_stage:
            w(f'    {g("all_logits", "xf", "word_embeddings.weight_g")} op.loss_backward_w')
        for i in range(n_layers, 0, -1):
            w(f"    {i} # layer_backward_w_{tag_of(i)}")
        w("    0 #")
        if next_rank is not None:
            w('    1 "slot_" @ io.link.release')
        w("%end")
    else:
        # ---- pipeline hand-offs around the stage's forward / backward (NCCL, in stream order) ----
        w("%def stage_forward")
        if prev_rank is not None:
            w(f'    0 # "stage_in" @ {prev_rank} io.nccl.recv')
        w("    model_forward")
        if next_rank is not None:
            w(f'    0 # "stage_out" @ {next_rank} io.nccl.send')
        w("%end")
        w("%def stage_score")
        w("    stage_forward model_score")
        w("%end")
        w("%def stage_backward")
        if next_rank is not None:
            w(f'    0 # "stage_out_g" @ {next_rank} io.nccl.recv')
        w("    model_backward")
        if prev_rank is not None:
            w(f'    0 # "stage_in_g" @ {prev_rank} io.nccl.send')
        w("%end")
        w("%def stage_backward_async")               # ( name -- )
        if next_rank is not None:
            w(f'    0 # "stage_out_g" @ {next_rank} io.nccl.recv')
        w("    model_backward_async")
        if prev_rank is not None:
            w(f'    0 # "stage_in_g" @ {prev_rank} io.nccl.send')
        w("%end")

    # ---- checkpoint: ( prefix -- ) save_model / load_model ----
    # Weights go out as the reference stores them, one raw fp32 file per tensor named <prefix>h<layer>.<tensor>.bin and
    # <prefix><tensor>.bin (bloomz-7b/init.words:120-235, bloomz-7b/dump_weights.py:105-133; the fused QKV weight keeps this
    # build's [q rows | k rows | v rows] order), taken from the fp32 master copies; the Adam moments follow with .m.bin /
    # .v.bin in place of .bin.  Loading fills master, moments and the fp16 working copy.  A rank writes the tensors of the
    # layer halves it owns; the tied table is written by the first stage only and read by both of its holders.
    for word, io in (("save_model", "io.save"), ("load_model", "io.load")):
        w(f"%def {word}")
        w('    0 # "ckpt_" !')
        for name, _ in main_params:
            if word == "save_model" and name == "word_embeddings.weight" and not first_stage:
                continue
            for suffix, ext in ((".master", ""), (".m", ".m"), (".v", ".v")):
                w(f'    "{name}{suffix}" @ "ckpt_" @ "{name}{ext}.bin" | {io}')
            if word == "load_model":
                w(f'    "{name}" @ "{name}.master" @ op.copy')
        for i in range(1, n_layers + 1):
            gi = layer_offset + i - 1
            owned = [nm for half in "AM" if half in kinds[i - 1] for nm in HALF_PARAMS[half]]
            w(f'    0 # "ckpt_" @ {i} # "ckpt_" !')
            for name in owned:
                for suffix, ext in ((".master", ""), (".m", ".m"), (".v", ".v")):
                    w(f'    "{name}{suffix}" @ "ckpt_" @ "h{gi}.{name}{ext}.bin" | {io}')
                if word == "load_model":
                    w(f'    "{name}" @ "{name}.master" @ op.copy')
            w('    "ckpt_" !!')
        w('    0 # "ckpt_" !!')
        w("%end")

    # ( peer -- )  both holders of the tied embedding / LM-head table sum their gradients.  sync_tied_start queues the
    # exchange on the transfer stream, so that it runs beside what the compute stream does next (the layers' Adam);
    # sync_tied_finish makes the compute stream wait for it and adds what arrived.
    w("%def sync_tied_start")
    w('    0 # "peer_" !')
    w('    op.stream.fork  "word_embeddings.weight_g" @ "tied_recv" @ "peer_" @ io.nccl.sendrecv')
    w('    "peer_" !!')
    w("%end")
    w("%def sync_tied_finish")
    w('    0 # op.stream.join')
    w('    "word_embeddings.weight_g" @ "tied_recv" @ "word_embeddings.weight_g" @ op.add')
    w("%end")
    w("%def sync_tied_grads")
    w("    sync_tied_start sync_tied_finish")
    w("%end")

    # ( -- )  data-parallel replicas: every gradient of the stage (and, on the head's stage, the micro-batch losses)
    # becomes its sum over the replicas, on the transfer stream; the compute stream waits for the last one.
    w("%def sync_replicas")
    w("    0 # op.stream.fork")
    for name, _ in main_params:
        w(f'    "{name}_g" @ io.nccl.allreduce')
    for i in range(1, n_layers + 1):
        w(f'    {i} # "_flat_g" @ io.nccl.allreduce')
    w("    0 #")
    if last_stage:
        w('    "loss_all" @ io.nccl.allreduce')
    w("    op.stream.join")
    w("%end")

    return "\n".join(L) + "\n"
