"""ctypes binding of libspion_b200.so (the C ABI declared in include/spion_b200.h).

There is no fallback: if the shared library has not been built (``python -m spion_b200.build``)
importing this module raises, and every call that returns a non-zero status raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_int, c_longlong, c_void_p

LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
# SPION_B200_LIBRARY names another build of the same library (e.g. one compiled with developer macros)
LIB_PATH = os.environ.get("SPION_B200_LIBRARY") or os.path.join(LIB_DIR, "libspion_b200.so")

F32, BF16 = 0, 1
CONV_DIAG, CONV_BOX = 0, 1
SELECT_PATHS, SELECT_TOPK = 0, 1
KIND_DENSE, KIND_DENSE_KPM, KIND_BLOCK, KIND_BLOCK_KPM = 0, 1, 2, 3
ENGINE_AUTO, ENGINE_SIMT, ENGINE_TCGEN05, ENGINE_SIMT_STAGED = 0, 1, 2, 3
STAGE_COUNT = 15

# name -> (restype, argtypes); every symbol include/spion_b200.h declares
SIGNATURES = {
    "spion_status_string": (ctypes.c_char_p, [c_int]),
    "spion_version": (c_int, []),
    "spion_create": (c_void_p, [c_int] * 7),
    "spion_destroy": (None, [c_void_p]),
    "spion_set_stream": (c_int, [c_void_p, c_void_p]),
    "spion_set_engine": (c_int, [c_void_p, c_int]),
    "spion_needs_scratch": (c_int, [c_void_p]),
    "spion_check_device_status": (c_int, [c_void_p]),
    "spion_set_head_layout": (c_int, [c_void_p, c_int]),
    "spion_set_block32_path": (c_int, [c_void_p, c_int]),
    "spion_block32_path_in_use": (c_int, [c_void_p]),
    "spion_layernorm_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_int,
                                ctypes.c_float, c_void_p]),
    "spion_layernorm_workspace_floats": (c_longlong, [c_int]),
    "spion_column_sums": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p]),
    "spion_add_layernorm_forward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                        c_void_p, c_void_p, c_longlong, c_int, ctypes.c_float, c_void_p]),
    "spion_add_layernorm_backward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p]),
    "spion_embedding_workspace_floats": (c_longlong, [c_longlong, c_int, c_int]),
    "spion_embedding_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p]),
    "spion_embedding_backward": (c_int, [c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_void_p,
                                         c_void_p]),
    "spion_layernorm_backward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_longlong, c_int, c_void_p]),
    "spion_csr_arrays_are_stable": (c_int, [c_void_p, c_int]),
    "spion_selftest_bounded_wait": (c_int, [c_void_p, c_longlong]),
    "spion_launch_count": (c_longlong, [c_void_p]),
    "spion_profile": (c_int, [c_void_p, c_int]),
    "spion_profile_get": (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
    "spion_profile_reset": (c_int, [c_void_p]),
    "spion_stage_name": (ctypes.c_char_p, [c_int]),
    "spion_block_attn_forward": (c_int, [c_void_p] * 10 + [c_int]),
    "spion_block_attn_backward": (c_int, [c_void_p] * 14 + [c_int]),
    "spion_dense_attn_forward": (c_int, [c_void_p] * 7),
    "spion_dense_attn_backward": (c_int, [c_void_p] * 12),
    "spion_mean_attention_map": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "spion_mean_map_tiles": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "spion_discover_pattern": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_double] + [c_void_p] * 13),
    "spion_build_structure": (c_int, [c_void_p, c_int] + [c_void_p] * 10),
    "spion_expand_csr": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "spion_set_pattern": (c_int, [c_void_p, c_void_p]),
    "spion_pattern_nnzb": (c_int, [c_void_p]),
    "spion_attn_forward_ex": (c_int, [c_void_p] * 8),
    "spion_attn_backward_ex": (c_int, [c_void_p] * 13),
    "spion_supports_fused": (c_int, [c_void_p]),
    "spion_attn_forward_fused": (c_int, [c_void_p] * 8),
    "spion_attn_backward_fused": (c_int, [c_void_p] * 11),
    "spion_mean_map_recompute": (c_int, [c_void_p] * 6),
    "spion_softmax_forward_ex": (c_int, [c_void_p] * 4),
    "spion_softmax_backward_ex": (c_int, [c_void_p] * 4),
    "spion_static_scratch_capacity": (ctypes.c_size_t, []),
    "spion_attn_forward_static": (c_int, [c_void_p] * 9 + [c_int] * 6 + [c_void_p]),
}


class SpionError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build the CUDA library first (python -m spion_b200.build). "
            "spion_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(rc: int, what: str = "spion_b200 call") -> None:
    if rc != 0:
        raise SpionError(f"{what} failed: {lib.spion_status_string(rc).decode()} ({rc})")


def check_operands(want_shape, **tensors) -> None:
    """The native calls take every size from the context they were created with, never from the
    tensors: operands of another shape (a short last batch, an evaluation batch) or on another device
    would make the kernels read and write past the buffers, so they are refused here."""
    dev = None
    for name, t in tensors.items():
        if tuple(t.shape) != tuple(want_shape):
            raise SpionError(f"{name} has shape {tuple(t.shape)}; the attention context was created for "
                             f"{tuple(want_shape)} (batch_size, num_head, max_seq_len, head_dim of its config)")
        if not t.is_cuda:
            raise SpionError(f"{name} is not a CUDA tensor (there is no CPU path)")
        if dev is not None and t.device != dev:
            raise SpionError(f"{name} is on {t.device}, other operands are on {dev}")
        dev = t.device


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else c_void_p(t.data_ptr())


def current_stream_ptr():
    import torch
    return c_void_p(torch.cuda.current_stream().cuda_stream)
