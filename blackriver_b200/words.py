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
