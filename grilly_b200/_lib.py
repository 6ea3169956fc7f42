"""ctypes binding of libgrilly_b200.so (the C ABI declared in include/grilly_b200.h).

This replaces the reference's Vulkan dispatch layer (backend/core.py:14-439):
there is no CPU fallback, so a missing library or a missing GPU raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libgrilly_b200.so"

OK = 0
ERR_INVALID_ARG, ERR_OOM, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_UNSUPPORTED = -1, -2, -3, -4, -5, -6
PREC_TF32, PREC_BF16, PREC_TF32X3 = 0, 1, 2
ACT_NONE, ACT_GELU, ACT_SILU, ACT_RELU = 0, 1, 2, 3
NORM_LAYER, NORM_RMS = 0, 1
ELT_GELU, ELT_SILU, ELT_RELU, ELT_ADD, ELT_SWIGLU, ELT_GCU, ELT_ROSWISH = 1, 2, 3, 4, 5, 6, 7
ROPE_NONE, ROPE_INTERLEAVED, ROPE_ROTATE_HALF = 0, 1, 2
DIST_L2, DIST_COSINE, DIST_DOT = 1, 2, 3
ARCH_POST_LN, ARCH_MODERNBERT = 0, 1
FLAG_OUT_BF16, FLAG_ROUND_TF32, FLAG_SWIGLU_PAIRS = 1, 2, 4


class EncoderConfig(C.Structure):
    _fields_ = [
        ("num_layers", C.c_int), ("hidden", C.c_int), ("num_heads", C.c_int), ("ffn", C.c_int),
        ("vocab", C.c_int), ("max_pos", C.c_int),
        ("embed_ln_eps", C.c_float), ("layer_ln_eps", C.c_float),
        ("has_token_type", C.c_int), ("precision", C.c_int), ("chunk_tokens", C.c_int),
        ("arch", C.c_int), ("rope_base", C.c_float), ("final_ln_eps", C.c_float),
    ]


_vp, _i, _ll, _f, _sz = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_size_t
_pp = C.POINTER(C.c_void_p)

# name -> argument types (all functions return int unless listed in _RESTYPE)
SIGNATURES = {
    "grilly_device_count": [C.POINTER(_i)],
    "grilly_init": [_i, _pp],
    "grilly_shutdown": [_vp],
    "grilly_last_error": [_vp],
    "grilly_set_stream": [_vp, _vp],
    "grilly_sync": [_vp],
    "grilly_set_tuning": [_vp, C.c_char_p, _i],
    "grilly_launch_count": [_vp, C.POINTER(C.c_uint64)],
    "grilly_selftest_wait_timeout": [_vp, _i],
    "grilly_timer_start": [_vp],
    "grilly_timer_stop": [_vp, C.POINTER(C.c_float)],
    "grilly_profile_begin": [_vp],
    "grilly_profile_end": [_vp, C.POINTER(C.c_double)],
    "grilly_alloc": [_vp, _sz, _pp],
    "grilly_free": [_vp, _vp],
    "grilly_upload": [_vp, _vp, _vp, _sz],
    "grilly_download": [_vp, _vp, _vp, _sz],
    "grilly_memset": [_vp, _vp, _i, _sz],
    "grilly_copy_2d": [_vp, _vp, _sz, _vp, _sz, _sz, _sz],
    "grilly_host_alloc": [_vp, _sz, _pp],
    "grilly_host_free": [_vp, _vp],
    "grilly_pool_stats": [_vp, C.POINTER(C.c_uint64)],
    "grilly_round_tf32": [_vp, _vp, _vp, _ll],
    "grilly_cast_f32_to_bf16": [_vp, _vp, _vp, _ll],
    "grilly_cast_bf16_to_f32": [_vp, _vp, _vp, _ll],
    "grilly_linear": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i],
    "grilly_fused_qkv_projection": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i],
    "grilly_fold_layernorm_weights": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i],
    "grilly_layernorm_linear": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _i, _i, _i],
    "grilly_layernorm_linear_noalloc": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _i, _i, _i],
    "grilly_linear_layernorm": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _i],
    "grilly_gemm_mnk": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i],
    "grilly_flash_attention": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _vp, _ll, _vp, _f, _i, _i, _f, _f, _i, _i],
    "grilly_attention_scores": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f],
    "grilly_attention_mask": [_vp, _vp, _vp, _i, _i, _i, _i, _f],
    "grilly_attention_output": [_vp, _vp, _vp, _vp, _i, _i, _i, _i],
    "grilly_attention_output_ex": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i],
    "grilly_apply_rope": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _f, _i],
    "grilly_layernorm": [_vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _f, _i, _i],
    "grilly_softmax": [_vp, _vp, _vp, _ll, _i],
    "grilly_eltwise": [_vp, _i, _vp, _vp, _vp, _ll, _i],
    "grilly_activation_params": [_vp, _i, _vp, _vp, _ll, _f, _f],
    "grilly_embedding_lookup": [_vp, _vp, _vp, _vp, _ll, _i, _i],
    "grilly_embed_layernorm": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i],
    "grilly_mean_pool": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i],
    "grilly_layernorm_backward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _f],
    "grilly_softmax_backward": [_vp, _vp, _vp, _vp, _ll, _i],
    "grilly_attention_backward": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f],
    "grilly_adam_update": [_vp, _vp, _vp, _vp, _vp, _ll, _f, _f, _f, _f, _f, _f, _i],
    "grilly_transpose_2d": [_vp, _vp, _vp, _i, _i],
    "grilly_encoder_create": [_vp, C.POINTER(EncoderConfig), _pp],
    "grilly_encoder_set_weight": [_vp, C.c_char_p, _i, _vp, _sz],
    "grilly_encoder_forward": [_vp, _vp, _vp, _i, _i, _vp],
    "grilly_encoder_forward_device": [_vp, _vp, _vp, _i, _i, _vp],
    "grilly_encoder_io_buffers": [_vp, _i, _i, _vp, _vp],
    "grilly_encoder_keep_hidden": [_vp, _i],
    "grilly_encoder_last_hidden": [_vp, _vp, _ll, C.POINTER(_ll)],
    "grilly_encoder_destroy": [_vp],
    "grilly_gemm_mnk_multi": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _i],
    "grilly_faiss_distances": [_vp, _vp, _vp, _vp, _i, _i, _i, _i],
    "grilly_faiss_search": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "grilly_faiss_topk": [_vp, _vp, _i, _i, _i, _vp, _vp],
    "grilly_gemm_pick_tile": [_i, _i, _i],
    "grilly_plan_chunks": [_vp, _i, _i, _vp, _vp, C.POINTER(_ll)],
}
_RESTYPE = {"grilly_last_error": C.c_char_p}

_lib = None


class GrillyError(RuntimeError):
    """An error status returned by libgrilly_b200.so."""

    def __init__(self, code: int, message: str):
        super().__init__(f"grilly_b200 error {code}: {message}")
        self.code = code


def load():
    """Load the shared library once. Raises RuntimeError if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("GRILLY_B200_LIB", LIB_PATH))
    if not path.exists():
        raise RuntimeError(
            f"{path} not found: build it with `python -m grilly_b200.build` (needs nvcc); "
            "grilly_b200 has no CPU fallback"
        )
    lib = C.CDLL(str(path))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.argtypes = argtypes
        fn.restype = _RESTYPE.get(name, C.c_int)
    _lib = lib
    return lib


def check(ctx, rc: int) -> None:
    """Map a status code to the exception class the reference raises for the same condition."""
    if rc == OK:
        return
    lib = load()
    msg = lib.grilly_last_error(ctx)
    msg = msg.decode() if msg else ""
    if rc == ERR_INVALID_ARG:
        raise ValueError(f"grilly_b200: {msg}")
    if rc == ERR_OOM:
        raise MemoryError(f"grilly_b200: {msg}")
    raise GrillyError(rc, msg)
