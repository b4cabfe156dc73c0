"""ctypes binding of libbrk.so (the C ABI in include/brk.h).

Pointers are passed as integers (``tensor.data_ptr()``), streams as the raw ``cudaStream_t``
value.  Every wrapper raises ``BrkError`` on a non-zero status: there is no fallback path.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libbrk.so")

OK, TODO_ERROR, INPUT_ERROR, OUTPUT_ERROR, ATTR_ERROR, CUDA_ERROR = 0, -1, -2, -3, -4, -5
F32, F16 = 0, 1

_STATUS_NAMES = {0: "BRK_OK", -1: "BRK_TODO_ERROR", -2: "BRK_INPUT_ERROR", -3: "BRK_OUTPUT_ERROR",
                 -4: "BRK_ATTR_ERROR", -5: "BRK_CUDA_ERROR"}


class BrkError(RuntimeError):
    def __init__(self, fn, status, detail=""):
        self.status = status
        super().__init__(f"{fn} returned {_STATUS_NAMES.get(status, status)} {detail}".strip())


p, i64, i32, f32, sz = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/brk.h one to one
SIGNATURES = {
    "brk_version": (i32, []),
    "brk_last_cuda_error": (C.c_char_p, []),
    "brk_sm_count": (i32, []),
    "brk_layernorm_fwd": (i32, [p, p, p, p, p, p, i64, i64, f32, i32, p]),
    "brk_layernorm_bwd_workspace_bytes": (sz, [i64, i64]),
    "brk_layernorm_bwd": (i32, [p, p, p, p, p, p, p, p, i64, i64, f32, p, sz, i32, i32, p]),
    "brk_layernorm_bwd_residual": (i32, [p, p, p, p, p, p, p, p, p, i64, i64, f32, p, sz, i32, i32, p]),
    "brk_layernorm_set_mode": (i32, [i32]),
    "brk_layernorm_bwd_static_capacity": (sz, []),
    "brk_layernorm_bwd_static": (i32, [p, p, p, p, p, p, p, p, i64, i64, f32, i32, i32, p]),
    "brk_gelu_fwd": (i32, [p, p, i64, i32, p]),
    "brk_gelu_bwd": (i32, [p, p, p, i64, i32, p]),
    "brk_logsoftmax_nll_fwd": (i32, [p, p, p, p, i64, i64, i32, p]),
    "brk_logsoftmax_nll_fwd_bwd": (i32, [p, p, p, p, i64, i64, f32, i32, p]),
    "brk_logsoftmax_nll_fwd_bwd_counted": (i32, [p, p, p, p, i64, i64, f32, p, i32, p]),
    "brk_sum_f32": (i32, [p, p, i64, p]),
    "brk_sum_div_f32": (i32, [p, p, p, i64, p]),
    "brk_signal_u32": (i32, [p, C.c_uint32, p]),
    "brk_loss_targets": (i32, [p, p, p, p, i32, i32, p]),
    "brk_add_bcast": (i32, [p, p, p, C.POINTER(i64), C.POINTER(i64), i32, p]),
    "brk_fill": (i32, [p, f32, i64, i32, p]),
    "brk_cast": (i32, [p, i32, p, i32, i64, p]),
    "brk_transpose_0213": (i32, [p, p, i64, i64, i64, i64, i32, p]),
    "brk_colsum": (i32, [p, p, i64, i64, i32, i32, p]),
    "brk_colsum_workspace_bytes": (sz, [i64, i64]),
    "brk_colsum_ws": (i32, [p, p, i64, i64, i32, i32, p, sz, p]),
    "brk_softmax_fwd": (i32, [p, p, i64, i64, i32, p]),
    "brk_softmax_bwd": (i32, [p, p, p, i64, i64, i32, p]),
    "brk_embedding_gather": (i32, [p, p, p, i64, i64, i64, i32, p]),
    "brk_alibi_slopes": (None, [i32, C.POINTER(C.c_double)]),
    "brk_alibi_build": (i32, [p, p, i32, i32, p]),
    "brk_xmask_build": (i32, [p, p, i32, i32, p]),
    "brk_gemm": (i32, [p, p, p, i64, i64, i64, i32, i32, i64, i64, i64, i64, i64, i64, i64, f32, f32, p, i32, p]),
    "brk_adam_step": (i32, [p, p, p, p, i32, p, i64, f32, f32, f32, f32, i32, f32, p]),
    "brk_adam_status": (i32, []),
    "brk_embedding_scatter_add": (i32, [p, p, p, i64, i64, i64, i32, p]),
    "brk_init_normal": (i32, [p, i64, f32, f32, C.c_uint64, i32, p]),
    "brk_gemm_f16_supported": (i32, [i64, i64, i64, i32, i32, i64, i64, p, p]),
    "brk_gemm_f16": (i32, [p, p, p, i64, i64, i64, i32, i32, i64, i64, i64, p, p, i64, p, i64, i32, p]),
    "brk_gemm_f16_status": (i32, []),
    "brk_gemm_f16_set_mode": (None, [i32]),
    "brk_gemm_f16_set_epilogue": (None, [i32]),
    "brk_gemm_f16_set_split_k": (None, [i32]),
    "brk_gemm_f16_split_items": (i32, [i32, i32, i32]),
    "brk_flash_attn_fwd": (i32, [p, p, p, i64, p, i64, p, p, p, i32, i32, i32, i32, p]),
    "brk_flash_attn_bwd_workspace_bytes": (sz, [i32, i32, i32]),
    "brk_flash_attn_bwd": (i32, [p, p, p, i64, p, p, i64, p, p, p, p, i64, p, p, i32, i32, i32, i32, p, sz, p]),
    "brk_flash_attn_status": (i32, []),
}

_lib = None


def lib():
    """Loads libbrk.so; raises if it has not been built (there is no other implementation)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`")
        _lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def call(name, *args):
    """Calls a status-returning entry point and raises BrkError on failure."""
    st = getattr(lib(), name)(*args)
    if st != 0:
        detail = ""
        if st == CUDA_ERROR:
            detail = lib().brk_last_cuda_error().decode()
        raise BrkError(name, st, detail)
    return st


def raw(name, *args):
    """Calls an entry point and returns its raw status (for error-path tests)."""
    return getattr(lib(), name)(*args)


def dims4(shape):
    shape = list(shape)
    return (i64 * 4)(*([1] * (4 - len(shape)) + shape))
