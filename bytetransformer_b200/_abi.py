"""ctypes binding of the C ABI declared in include/bt_b200.h.

The shared library is built in-tree by `bytetransformer_b200.build`; loading
fails loudly (ImportError-like RuntimeError) when it is missing — there is no
fallback implementation.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libbt_b200.so")

BT_OK = 0
BT_ERR_INVALID_ARG = 1
BT_ERR_WORKSPACE = 2
BT_ERR_CUDA = 3
BT_ERR_UNSUPPORTED = 4
BT_ERR_DEVICE_STATUS = 5
BT_GELU_ERF = 0
BT_GELU_TANH = 1
BT_EPI_NONE = 0
BT_EPI_BIAS = 1
BT_EPI_BIAS_GELU = 2
BT_EPI_BIAS_RESIDUAL = 3
BT_EPI_BIAS_RESIDUAL_F32OUT = 4
BT_EPI_BIAS_RESIDUAL_LAYERNORM = 5
BT_STATIC_SCRATCH_BYTES = 48 * 1024 * 1024

ERROR_NAMES = {0: "BT_OK", 1: "BT_ERR_INVALID_ARG", 2: "BT_ERR_WORKSPACE", 3: "BT_ERR_CUDA",
               4: "BT_ERR_UNSUPPORTED", 5: "BT_ERR_DEVICE_STATUS"}


class bt_config(C.Structure):
    _fields_ = [("head_num", C.c_int), ("size_per_head", C.c_int), ("max_batch_size", C.c_int),
                ("max_seq_len", C.c_int), ("intermediate_mult", C.c_int), ("ln_eps", C.c_float),
                ("gelu_kind", C.c_int), ("tao", C.c_float), ("gamma_beta_fp32", C.c_int),
                ("device", C.c_int)]


class bt_layer_weights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "qkv_kernel", "qkv_bias", "attr_output_kernel", "attr_output_bias",
        "attr_output_layernorm_gamma", "attr_output_layernorm_beta", "inter_kernel", "inter_bias",
        "output_kernel", "output_bias", "output_layernorm_gamma", "output_layernorm_beta")]


class bt_embedding_weights(C.Structure):
    _fields_ = [("word_emb", C.c_void_p), ("pos_emb", C.c_void_p), ("type_emb", C.c_void_p), ("gamma", C.c_void_p),
                ("beta", C.c_void_p), ("gamma_beta_fp32", C.c_int), ("vocab_size", C.c_int),
                ("max_positions", C.c_int), ("type_vocab_size", C.c_int), ("eps", C.c_float)]


_vp, _i, _f, _sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t

# name -> (restype, argtypes); one entry per declaration in include/bt_b200.h
SIGNATURES = {
    "bt_version": (C.c_char_p, []),
    "bt_create": (_i, [C.POINTER(bt_config), C.POINTER(_vp)]),
    "bt_destroy": (_i, [_vp]),
    "bt_set_layer_weights": (_i, [_vp, _i, C.POINTER(bt_layer_weights)]),
    "bt_workspace_bytes": (_i, [_vp, _i, _i, C.POINTER(_sz)]),
    "bt_workspace_bytes_packed": (_i, [_vp, _i, _i, C.POINTER(_sz)]),
    "bt_last_error": (C.c_char_p, [_vp]),
    "bt_device_status": (_i, [_vp, _vp, C.POINTER(_i)]),
    "bt_embedding_layernorm": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "bt_pooler": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "bt_embedding_layernorm_packed": (_i, [C.POINTER(bt_embedding_weights), _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "bt_stack_forward_ids": (_i, [_vp, _i, C.POINTER(bt_embedding_weights), _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _vp]),
    "bt_selftest_bounded_wait": (_i, [_vp, C.c_longlong, _vp, _vp]),
    "bt_layer_forward_padded": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _sz, _i, _i, _vp]),
    "bt_layer_forward_padded_static": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _vp]),
    "bt_stack_forward_padded": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _sz, _i, _i, _vp]),
    "bt_layer_forward_padded_general": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _vp]),
    "bt_stack_forward_padded_general": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _vp]),
    "bt_mask_is_right_padded": (_i, [_vp, _i, _i, _vp, C.POINTER(_i), _vp]),
    "bt_stack_forward_packed": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _sz, _vp]),
    "bt_build_offsets": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "bt_pack_rows": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "bt_restore_rows": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "bt_gemm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "bt_gemm_layernorm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _f, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "bt_attention": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "bt_add_bias_residual_layernorm": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _f, _vp]),
    "bt_add_bias_residual_layernorm_restore": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _f, _vp]),
    "bt_add_bias_gelu": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "bt_masked_softmax": (_i, [_vp, _vp, _i, _i, _i, _f, _vp]),
    "bt_profile_enable": (_i, [_vp, _i]),
    "bt_profile_read": (_i, [_vp, C.POINTER(C.c_double), C.POINTER(C.c_longlong)]),
}
PROF_KINDS = ("offsets", "pack", "gemm_qkv", "mha", "gemm_attn_out", "layernorm", "gemm_ffn1", "gemm_ffn2",
              "gemm_other")

_lib = None


def load(path: str | None = None) -> C.CDLL:
    """Load libbt_b200.so and attach the prototypes.  Raises if it is not built."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise RuntimeError(
            f"{p} is missing: build it with `python -m bytetransformer_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(p)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    if hasattr(lib, "bt_debug_set"):
        lib.bt_debug_set.restype = _i
        lib.bt_debug_set.argtypes = [_i, C.c_longlong]
    if hasattr(lib, "bt_debug_set_fused_layernorm"):
        lib.bt_debug_set_fused_layernorm.restype = _i
        lib.bt_debug_set_fused_layernorm.argtypes = [_vp, _i]
    if path is None:
        _lib = lib
    return lib


class BtError(RuntimeError):
    def __init__(self, code: int, where: str, detail: str = ""):
        self.code = code
        super().__init__(f"{where}: {ERROR_NAMES.get(code, code)}" + (f" ({detail})" if detail else ""))
