"""Python face of the CUDA kernel library (csrc/): loads the shared library through
ctypes and wraps each entry point in a function that takes torch tensors.

There is no fallback: if the library cannot be built or loaded, or a kernel refuses
its sizes, an exception says so.  Every wrapper launches on torch's current stream,
so calls are captured by a CUDA graph like any torch operation.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
OUT_SAME, OUT_F32, OUT_ADD_F32, OUT_SWIGLU = 0, 1, 2, 3
OUT_GELU = 5        # the tensor-core product alone: bf16 out = gelu_tanh(product)
OUT_GEGLU = 6       # the tensor-core product alone: as OUT_SWIGLU with gelu_tanh on the gate

_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None
_lock = threading.Lock()
launch_count = 0   # kernels launched through this module (bench.py reports it)

_c_int, _c_float, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

_SIGNATURES = {
    "rl_embedding": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_rmsnorm": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_float, _c_void_p],
    "rl_swiglu": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "rl_convert": [_c_void_p, _c_int, _c_void_p, _c_int, _c_ll, _c_void_p],
    "rl_random_fill": [_c_void_p, _c_int, _c_ll, ctypes.c_ulonglong, _c_float, _c_float, _c_void_p],
    "rl_gemm_simt": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                     _c_int, _c_int, _c_void_p],
    "rl_layer_norm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_float, _c_void_p],
    "rl_token_shift_mix": [_c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_ll,
                           _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "rl_tanh_cast": [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p],
    "rl_scaled_add": [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_float, _c_ll, _c_void_p],
    "rl_row_gate_add": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "rl_scale": [_c_void_p, _c_ll, _c_float, _c_void_p],
    "rl_geglu": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "rl_channel_decay_scan": [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                              _c_void_p, _c_int, _c_void_p, _c_ll, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "rl_moe_route_scored": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                            _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_moe_select_scored": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p,
                             _c_void_p],
    "rl_rope_kv_write_mixed": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                               _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                               _c_void_p, _c_void_p],
    "rl_rope_kv_write": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                         _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_attention_simt": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                          _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                          _c_void_p],
    "rl_attention_simt_gated": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                                _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                                _c_int, _c_void_p, _c_int, _c_void_p],
    "rl_attention_simt_masked": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                                 _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                                 _c_int, _c_void_p, _c_int, _c_float, _c_int, _c_void_p],
    "rl_attention_simt_shaped": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                                 _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                                 _c_int, _c_void_p, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "rl_attention_shared_key_supported": [_c_int, _c_int, _c_int],
    "rl_attention_shared_key": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                                _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p,
                                _c_void_p],
    "rl_attention_shared_key_block_tokens": [_c_int, _c_int, _c_int],
    "rl_attention_shared_key_head_blocks": [_c_int, _c_int, _c_int],
    "rl_heads_linear": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "rl_embedding_pair": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_ll,
                          _c_float, _c_ll, _c_ll, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_gelu_tanh": [_c_void_p, _c_void_p, _c_int, _c_ll, _c_void_p],
    "rl_qk_rotate_unit": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                          _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_latent_prepare": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_int,
                          _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_latent_query": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p,
                        _c_int, _c_int, _c_int, _c_void_p],
    "rl_short_conv": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_ll,
                      _c_void_p, _c_int, _c_int, _c_void_p],
    "rl_short_conv_state": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_ll, _c_void_p],
    "rl_qkv_prepare": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_int, _c_void_p, _c_ll, _c_void_p, _c_void_p,
                       _c_float, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_float, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_linear_scan": [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p,
                       _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_ll, _c_void_p, _c_int, _c_int,
                       _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "rl_norm_add": [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_float, _c_void_p, _c_float, _c_float, _c_int, _c_int, _c_void_p,
                    _c_void_p],
    "rl_gated_norm": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_float, _c_int, _c_int, _c_int,
                      _c_void_p, _c_int, _c_void_p],
    "rl_gelu_gate": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_void_p],
    "rl_moe_route_sigmoid": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                             _c_void_p, _c_void_p, _c_void_p],
    "rl_moe_select_sigmoid": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_embedding_pos": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                         _c_void_p, _c_void_p],
    "rl_residual_inject": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "rl_softcap": [_c_void_p, _c_ll, _c_float, _c_void_p],
    "rl_sigmoid_gate": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "rl_moe_route": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p,
                     _c_void_p],
    "rl_moe_select": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_moe_experts": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_moe_plan": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_moe_gather": [_c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_moe_combine": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_gemm_tc_grouped": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                           _c_void_p, _c_int, _c_int, _c_void_p],
    "rl_repeat_penalty": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_float, _c_void_p],
    "rl_argmax": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_sample_temperature": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "rl_sample_candidates": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int,
                             _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "rl_attention_decode": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                            _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p],
    "rl_attention_decode_gated": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                  _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                                  _c_int, _c_void_p, _c_int, _c_void_p],
    "rl_attention_decode_masked": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                   _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                                   _c_int, _c_void_p, _c_int, _c_float, _c_int, _c_void_p],
    "rl_attention_prefill_gated": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                   _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                                   _c_int, _c_void_p, _c_int, _c_void_p],
    "rl_attention_prefill_tc_gated": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                      _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float,
                                      _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p],
    "rl_attention_prefill_tc_masked": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                       _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float,
                                       _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_float, _c_int, _c_void_p],
    "rl_attention_prefill_tc_shaped": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                       _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float,
                                       _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_float, _c_int, _c_int, _c_void_p],
    "rl_attention_decode_headgate": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                     _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int,
                                     _c_int, _c_void_p, _c_int, _c_float, _c_int, _c_int, _c_void_p],
    "rl_attention_prefill_tc_headgate": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                         _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float,
                                         _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_float, _c_int, _c_int, _c_int, _c_void_p],
    "rl_attention_decode_plan": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_attention_decode_order": [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_attention_decode_places": [_c_int],
    "rl_attention_decode_ring_bytes": [_c_int],
    "rl_attention_decode_supported": [_c_int, _c_int, _c_int],
    "rl_attention_prefill": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                             _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p],
    "rl_attention_prefill_supported": [_c_int, _c_int, _c_int],
    "rl_attention_prefill_tc": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float,
                                _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_attention_prefill_tc_supported": [_c_int, _c_int, _c_int],
    "rl_gemm_tc_supported": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int],
    "rl_gemm_tc": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                   _c_void_p, _c_int, _c_void_p, _c_int, _c_float, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p],
    "rl_gemm_tc_splits": [_c_int, _c_int, _c_int],
    "rl_gemm_tc_qkv_rope_supported": [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int],
    "rl_gemm_tc_qkv_rope": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                            _c_void_p, _c_int, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                            _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
}


def library() -> ctypes.CDLL:
    """The loaded kernel library; built on first use."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.build()
                try:
                    lib = ctypes.CDLL(path)
                except OSError as e:
                    raise KernelError(f"cannot load the kernel library {path}: {e}") from e
                lib.rl_last_error.restype = ctypes.c_char_p
                lib.rl_last_error.argtypes = []
                for name, args in _SIGNATURES.items():
                    fn = getattr(lib, name, None)
                    if fn is None:
                        raise KernelError(f"kernel library {path} lacks the entry point {name}")
                    fn.restype = _c_int
                    fn.argtypes = args
                if lib.rl_page_size() != PAGE_SIZE:
                    raise KernelError(f"the kernel library was built for pages of {lib.rl_page_size()} "
                                      f"tokens, the package expects {PAGE_SIZE}")
                _lib = lib
    return _lib


def library_file() -> str:
    library()
    return _build.library_path()


def _check(code: int, name: str) -> None:
    if code != 0:
        msg = library().rl_last_error().decode("utf-8", "replace")
        raise KernelError(f"{name} failed ({code}): {msg}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream of the current device as a raw handle (asked for on every
    launch: during graph capture it is the capturing stream)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not handled by the kernels (float32 and bfloat16 are)") from None


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on CUDA tensors only (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


# ----------------------------------------------------------------------------- wrappers
def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, err_flag: torch.Tensor) -> None:
    """out[m, :] = table[ids[m], :] as float32.  err_flag (int32[1]) is set to 1 on a bad id."""
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32)
    _need(err_flag, "err_flag", torch.int32)
    V, d = table.shape
    M = ids.numel()
    assert out.shape == (M, d)
    _check(library().rl_embedding(table.data_ptr(), _dt(table), ids.data_ptr(), out.data_ptr(), M, d, V,
                                  err_flag.data_ptr(), _stream()), "rl_embedding")
    _count()


def embedding_pos(table: torch.Tensor, pos_table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor,
                  out: torch.Tensor, err_flag: torch.Tensor) -> None:
    """out[m, :] = table[ids[m], :] + pos_table[positions[m], :] as float32.  err_flag (int32[1]) is set
    to 1 on a bad id and to 2 on a position outside ``pos_table``."""
    _need(table, "table"); _need(pos_table, "pos_table", table.dtype); _need(ids, "ids", torch.int32)
    _need(positions, "positions", torch.int32); _need(out, "out", torch.float32); _need(err_flag, "err_flag", torch.int32)
    V, d = table.shape
    M = ids.numel()
    assert out.shape == (M, d) and pos_table.shape[1] == d and positions.numel() == M
    _check(library().rl_embedding_pos(table.data_ptr(), pos_table.data_ptr(), _dt(table), ids.data_ptr(), positions.data_ptr(),
                                      out.data_ptr(), M, d, V, pos_table.shape[0], err_flag.data_ptr(), _stream()),
           "rl_embedding_pos")
    _count()


def embedding_pair(table: torch.Tensor, pair_table: Optional[torch.Tensor], ids: torch.Tensor, positions: torch.Tensor,
                   slot_of_token: torch.Tensor, cu_seqlens: torch.Tensor, last_token: torch.Tensor, scale: float,
                   mul_prev: int, mul_cur: int, buckets: int, out: torch.Tensor, err_flag: torch.Tensor) -> None:
    """out[m, :] = table[ids[m], :] * scale + pair_table[row_m, :] as float32, row_m = (prev_m * mul_prev + ids[m] * mul_cur)
    mod buckets with prev_m the token in front of token m in its sequence; a sequence's first token takes row
    ``buckets``.  ``last_token``: the per-slot state view [slots, >= 4 bytes] (uint8) holding, as an int32, the last token
    each sequence has been fed; read for a step's first token of a sequence that is under way, and updated.
    ``pair_table`` None: the scaled embedding alone."""
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32); _need(err_flag, "err_flag", torch.int32)
    _need(positions, "positions", torch.int32); _need(slot_of_token, "slot_of_token", torch.int32)
    _need(cu_seqlens, "cu_seqlens", torch.int32)
    V, d = table.shape
    M = ids.numel()
    assert out.shape == (M, d) and positions.numel() == M and slot_of_token.numel() == M
    if pair_table is not None:
        _need(pair_table, "pair_table", table.dtype)
        assert pair_table.shape == (buckets + 1, d), (pair_table.shape, buckets)
    sp, ss = _state_args(last_token)
    _check(library().rl_embedding_pair(table.data_ptr(), _ptr(pair_table), _dt(table), ids.data_ptr(), positions.data_ptr(),
                                       slot_of_token.data_ptr(), cu_seqlens.data_ptr(), cu_seqlens.numel() - 1, sp, ss,
                                       float(scale), int(mul_prev), int(mul_cur), int(buckets), out.data_ptr(), M, d, V,
                                       err_flag.data_ptr(), _stream()), "rl_embedding_pair")
    _count()


def gelu_tanh(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), computed in 32-bit; ``out`` may be ``x``."""
    _need(x, "x"); _need(out, "out", x.dtype)
    assert out.shape == x.shape
    _check(library().rl_gelu_tanh(x.data_ptr(), out.data_ptr(), _dt(x), x.numel(), _stream()), "rl_gelu_tanh")
    _count()


def residual_inject(x: torch.Tensor, again: Optional[torch.Tensor], vec: Optional[torch.Tensor]) -> None:
    """x[m, :] += again[m, :] + vec[:] (either may be ``None``); x and again float32 [M, d], vec [d]."""
    _need(x, "x", torch.float32)
    M, d = x.shape
    if again is not None:
        _need(again, "again", torch.float32)
        assert again.shape == x.shape
    if vec is not None:
        _need(vec, "vec")
        assert vec.numel() == d
    if again is None and vec is None:
        return
    _check(library().rl_residual_inject(x.data_ptr(), _ptr(again), _ptr(vec), _dt(vec) if vec is not None else F32, M, d,
                                        _stream()), "rl_residual_inject")
    _count()


def softcap(logits: torch.Tensor, cap: float) -> None:
    """logits = cap * tanh(logits / cap), in place (float32)."""
    _need(logits, "logits", torch.float32)
    _check(library().rl_softcap(logits.data_ptr(), logits.numel(), float(cap), _stream()), "rl_softcap")
    _count()


def sigmoid_gate(y: torch.Tensor, gate: torch.Tensor) -> None:
    """y *= sigmoid(gate), in place; gate [M, n] may be a view with a wider row stride."""
    _need(y, "y", contiguous=False); _need(gate, "gate", y.dtype, contiguous=False)
    M, n = y.shape
    assert gate.shape == (M, n) and y.stride(1) == 1 and gate.stride(1) == 1
    _check(library().rl_sigmoid_gate(y.data_ptr(), y.stride(0) if M > 1 else n, gate.data_ptr(), gate.stride(0) if M > 1 else n,
                                     _dt(y), M, n, _stream()), "rl_sigmoid_gate")
    _count()


def moe_route(x: torch.Tensor, router: torch.Tensor, bias: Optional[torch.Tensor], top: int,
              ids: torch.Tensor, weights: torch.Tensor) -> None:
    """Router of a mixture of experts: logits ``router @ x[m] + bias`` in 32-bit, the ``top`` largest
    chosen (ties to the lower index), their weights the softmax over the chosen logits.
    ids int32 [M, top], weights float32 [M, top], both in the order of falling logits."""
    _need(x, "x", contiguous=False); _need(router, "router", x.dtype); _need(ids, "ids", torch.int32)
    _need(weights, "weights", torch.float32)
    M, d = x.shape
    E = router.shape[0]
    assert router.shape == (E, d) and ids.shape == (M, top) and weights.shape == (M, top) and x.stride(1) == 1
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == E
    _check(library().rl_moe_route(x.data_ptr(), x.stride(0) if M > 1 else d, router.data_ptr(), _ptr(bias), _dt(x), M, d, E,
                                  int(top), ids.data_ptr(), weights.data_ptr(), _stream()), "rl_moe_route")
    _count()


def moe_select(logits: torch.Tensor, top: int, ids: torch.Tensor, weights: torch.Tensor) -> None:
    """The router's second half alone: from float32 logits [M, E] (bias included) the ``top`` largest a token
    (ties to the lower index) and the softmax over them, as ``moe_route`` leaves them."""
    _need(logits, "logits", torch.float32); _need(ids, "ids", torch.int32); _need(weights, "weights", torch.float32)
    M, E = logits.shape
    assert ids.shape == (M, top) and weights.shape == (M, top)
    _check(library().rl_moe_select(logits.data_ptr(), M, E, int(top), ids.data_ptr(), weights.data_ptr(), _stream()), "rl_moe_select")
    _count()


def moe_experts(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                residual: torch.Tensor, interleaved: bool = False) -> None:
    """residual[m] += sum_c weights[m, c] * down[e] (silu(gate[e] x[m]) * (up[e] x[m])), e = ids[m, c], on the
    CUDA cores (any sizes, float32 or bfloat16 storage): every (token, choice) pair reads its expert's rows,
    which is what a step of few tokens needs.  gate_up: [E, 2, F, d] (an expert's gate rows, then its up
    rows) or, ``interleaved``, [E, F, 2, d] (gate_r, up_r in turn); down: [E, d, F]."""
    _need(x, "x", contiguous=False); _need(gate_up, "gate_up", x.dtype); _need(down, "down", x.dtype)
    _need(ids, "ids", torch.int32); _need(weights, "weights", torch.float32); _need(residual, "residual", torch.float32)
    M, d = x.shape
    if interleaved:
        E, F, two, d2 = gate_up.shape
    else:
        E, two, F, d2 = gate_up.shape
    top = ids.shape[1]
    assert two == 2 and d2 == d and down.shape == (E, d, F) and residual.shape == (M, d) and x.stride(1) == 1
    assert ids.shape == (M, top) and weights.shape == (M, top)
    h = torch.empty((M * top, F), dtype=x.dtype, device=x.device)
    _check(library().rl_moe_experts(x.data_ptr(), x.stride(0) if M > 1 else d, gate_up.data_ptr(), down.data_ptr(), _dt(x),
                                    ids.data_ptr(), weights.data_ptr(), M, d, F, E, top, int(bool(interleaved)), h.data_ptr(),
                                    residual.data_ptr(), _stream()), "rl_moe_experts")
    _count(2)


def moe_token_tile(num_tokens: int, top: int, num_experts: int) -> int:
    """Rows of a token tile for the grouped products: what an expert gets on average, rounded up to a tile the
    tensor-core product has (16 to 128; padding every expert to whole tiles costs the less the smaller the tile)."""
    avg = -(-num_tokens * top // num_experts)
    return 16 if avg <= 16 else 32 if avg <= 32 else 64 if avg <= 64 else 128 if avg < 256 else 256


def moe_experts_grouped_supported(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor) -> bool:
    """bf16, rows TMA can address (hidden size and expert size multiples of 8, 16-byte aligned bases)."""
    return (x.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16 and down.dtype == torch.bfloat16
            and x.shape[1] % 8 == 0 and down.shape[2] % 8 == 0 and x.stride(1) == 1 and (x.stride(0) % 8 == 0 or x.shape[0] == 1)
            and x.data_ptr() % 16 == 0 and gate_up.data_ptr() % 16 == 0 and down.data_ptr() % 16 == 0)


def moe_experts_grouped(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                        residual: torch.Tensor) -> None:
    """The same sum as ``moe_experts`` on the tensor cores, for steps of many tokens: the (token, choice) pairs
    are ordered by expert (every expert's rows padded to whole token tiles), gate and up run as one grouped
    product with the activation in its epilogue, down as a second one, and the choices of a token are added
    into the residual in their order.  gate_up: [E, F, 2, d] (gate_r, up_r in turn), down: [E, d, F], bf16."""
    _need(x, "x", torch.bfloat16, contiguous=False); _need(gate_up, "gate_up", torch.bfloat16); _need(down, "down", torch.bfloat16)
    _need(ids, "ids", torch.int32); _need(weights, "weights", torch.float32); _need(residual, "residual", torch.float32)
    M, d = x.shape
    E, F, two, d2 = gate_up.shape
    top = ids.shape[1]
    assert two == 2 and d2 == d and down.shape == (E, d, F) and residual.shape == (M, d)
    pairs = M * top
    bt = moe_token_tile(M, top, E)
    rows = (pairs + min(pairs, E) * (bt - 1)) // bt * bt
    tiles = rows // bt
    dev = x.device
    row = torch.empty(pairs, dtype=torch.int32, device=dev)
    tile_group = torch.empty(tiles, dtype=torch.int32, device=dev)
    xs = torch.empty((rows, d), dtype=torch.bfloat16, device=dev)
    h = torch.empty((rows, F), dtype=torch.bfloat16, device=dev)
    y = torch.empty((rows, d), dtype=torch.float32, device=dev)
    lib, st, err = library(), _stream(), _tc_error_word(dev).data_ptr()
    _check(lib.rl_moe_plan(ids.data_ptr(), pairs, E, bt, tiles, row.data_ptr(), tile_group.data_ptr(), st), "rl_moe_plan")
    _check(lib.rl_moe_gather(x.data_ptr(), x.stride(0) if M > 1 else d, row.data_ptr(), pairs, top, d, xs.data_ptr(), st), "rl_moe_gather")
    _check(lib.rl_gemm_tc_grouped(xs.data_ptr(), gate_up.data_ptr(), h.data_ptr(), OUT_SWIGLU, rows, 2 * F, d, d, F, err,
                                  tile_group.data_ptr(), E, bt, st), "rl_gemm_tc_grouped")
    _check(lib.rl_gemm_tc_grouped(h.data_ptr(), down.data_ptr(), y.data_ptr(), OUT_F32, rows, d, F, F, d, err,
                                  tile_group.data_ptr(), E, bt, st), "rl_gemm_tc_grouped")
    _check(lib.rl_moe_combine(y.data_ptr(), row.data_ptr(), weights.data_ptr(), M, top, d, residual.data_ptr(), st), "rl_moe_combine")
    _count(5)


_TILE_GROUPS = {}


def gemm_tc_row_groups_tile(rows: int) -> int:
    """The token tile for ``gemm_tc_row_groups`` at ``rows`` rows a group (each group is padded to whole tiles)."""
    return 16 if rows <= 16 else 32 if rows <= 32 else 64 if rows <= 64 else 128 if rows <= 1024 else 256


def gemm_tc_row_groups_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous() and a.shape[-1] % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_row_groups(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile: int) -> None:
    """Several products of equal shape with inputs and weights of their own as one grouped tensor-core product:
    out[g] = a[g] @ w[g].T for a [G, rows, K], w [G, N, K], out [G, rows, N], all bfloat16 and contiguous, ``rows`` a
    multiple of ``tile`` (the caller pads; what the padding rows hold does not matter, every row is computed by itself)."""
    _need(a, "a", torch.bfloat16); _need(w, "w", torch.bfloat16); _need(out, "out", torch.bfloat16)
    G, rows, Kd = a.shape
    N = w.shape[1]
    assert w.shape == (G, N, Kd) and out.shape == (G, rows, N) and rows % tile == 0
    per = rows // tile
    key = (a.device, G, per)
    table = _TILE_GROUPS.get(key)
    if table is None:
        table = _TILE_GROUPS[key] = torch.arange(G * per, dtype=torch.int32, device=a.device).div(per, rounding_mode="floor").to(torch.int32)
    _check(library().rl_gemm_tc_grouped(a.data_ptr(), w.data_ptr(), out.data_ptr(), OUT_SAME, G * rows, N, Kd, Kd, N,
                                        _tc_error_word(a.device).data_ptr(), table.data_ptr(), G, tile, _stream()), "rl_gemm_tc_grouped")
    _count()


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rms_norm(x[rows[r]] if rows is given else x[r]) * weight."""
    _need(x, "x", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    d = x.shape[-1]
    n = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        assert rows.numel() == n
    else:
        assert x.shape[0] == n
    assert weight.numel() == d and out.shape[-1] == d
    _check(library().rl_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), _dt(out), _ptr(rows), n, d,
                                float(eps), _stream()), "rl_rmsnorm")
    _count()


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out = silu(gate) * up.  gate_up: [M, 2I] holding the gate in columns [0, I) and up
    in [I, 2I), or, interleaved, gate_i in column 2i and up_i in column 2i + 1."""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    M, two_i = gate_up.shape
    assert two_i % 2 == 0 and out.shape == (M, two_i // 2)
    _check(library().rl_swiglu(gate_up.data_ptr(), out.data_ptr(), _dt(out), M, two_i // 2, int(interleaved), _stream()),
           "rl_swiglu")
    _count()


def convert(src: torch.Tensor, dst: torch.Tensor) -> None:
    _need(src, "src"); _need(dst, "dst")
    assert src.numel() == dst.numel()
    _check(library().rl_convert(src.data_ptr(), _dt(src), dst.data_ptr(), _dt(dst), src.numel(), _stream()), "rl_convert")
    _count()


def random_fill(out: torch.Tensor, seed: int, mean: float, std: float) -> None:
    """out[i] = mean + std * z_i with z_i the library's reproducible near-normal number i of
    ``seed`` (csrc/random_fill.cu): the same values as ``weights.random_init.normal_values``
    computes on the host, bit for bit."""
    _need(out, "out")
    _check(library().rl_random_fill(out.data_ptr(), _dt(out), out.numel(), int(seed) & ((1 << 64) - 1), float(mean), float(std),
                                    _stream()), "rl_random_fill")
    _count()


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, out_mode: int,
              bias: Optional[torch.Tensor] = None) -> None:
    """out = a @ w.T (+ bias) on the CUDA cores.  a: [M, K] (rows may be strided),
    w: [N, K] contiguous, same dtype.  out_mode: OUT_SAME / OUT_F32 / OUT_ADD_F32."""
    _need(a, "a", contiguous=False); _need(w, "w", a.dtype); _need(out, "out", contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and out.stride(1) == 1
    if out_mode == OUT_SAME:
        assert out.dtype == a.dtype
    else:
        assert out.dtype == torch.float32
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == N
    lda = a.stride(0) if M > 1 else K
    ldo = out.stride(0) if M > 1 else N
    _check(library().rl_gemm_simt(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), _dt(a), out_mode,
                                  M, N, K, lda, ldo, _stream()), "rl_gemm_simt")
    _count()


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_of_token: torch.Tensor,
                  page_table: torch.Tensor, inv_freq: torch.Tensor, num_heads: int, num_kv_heads: int,
                  head_dim: int, rotary_dim: int, interleaved: bool,
                  k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], value_dim: Optional[int] = None,
                  v_other: Optional[torch.Tensor] = None, v_mix: Optional[torch.Tensor] = None) -> None:
    """Rotates the query and key heads of qkv ([M, H*hd + G*hd + G*vd]) in place and writes keys
    and values at their tokens' places of the paged pools.  ``value_dim`` (default: head_dim)
    is the width of a value head.  ``v_other`` [M, G*vd] (a view is fine) with ``v_mix`` (a float32 scalar on the
    device): the values become (1 - v_mix) v + v_mix v_other, in 32-bit, before they are cached."""
    vd = head_dim if value_dim is None else value_dim
    _need(qkv, "qkv", contiguous=False); _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    M = qkv.shape[0]
    assert qkv.stride(1) == 1 and (M == 1 or qkv.stride(0) >= qkv.shape[1])
    if k_pool is not None:
        _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype)
        _need(slot_of_token, "slot_of_token", torch.int32); _need(page_table, "page_table", torch.int32)
        assert k_pool.shape[1:] == (num_kv_heads, page_size(), head_dim), k_pool.shape
        assert v_pool.shape[1:] == (num_kv_heads, page_size(), vd), v_pool.shape
        max_pages = page_table.shape[1]
    else:
        max_pages = 0
    assert inv_freq.numel() >= rotary_dim // 2
    ld_other = 0
    if v_other is not None:
        _need(v_other, "v_other", qkv.dtype, contiguous=False); _need(v_mix, "v_mix", torch.float32)
        assert v_other.shape == (M, num_kv_heads * vd) and v_other.stride(1) == 1 and v_mix.numel() == 1
        ld_other = v_other.stride(0) if M > 1 else num_kv_heads * vd
    _check(library().rl_rope_kv_write_mixed(
        qkv.data_ptr(), _dt(qkv), qkv.stride(0), positions.data_ptr(), _ptr(slot_of_token), _ptr(page_table),
        max_pages, inv_freq.data_ptr(), M, num_heads, num_kv_heads, head_dim, vd, rotary_dim, int(interleaved),
        _ptr(k_pool), _ptr(v_pool), _ptr(v_other), ld_other, _ptr(v_mix) if v_other is not None else None, _stream()), "rl_rope_kv_write")
    _count()


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                   slot_of_token: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                   num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                   value_dim: Optional[int] = None, sink: bool = False, gate: Optional[torch.Tensor] = None,
                   softcap: float = 0.0, keep_first: int = 0, chunk: int = 0, values_in_keys: bool = False,
                   gate_per_head: bool = False) -> None:
    """q: [M, >= H*hd] (a view into the qkv buffer is fine), out: [M, H*vd] where vd is
    ``value_dim`` (default: head_dim), the width of a value head.  ``sink``: the softmax's
    denominator has one more term of score 0 (and no value).  ``gate`` [M, H*vd] (a view is
    fine): the output is multiplied by sigmoid(gate) before it is stored.  ``softcap`` > 0: a score s
    (scale included) becomes softcap * tanh(s / softcap).  ``keep_first``: with a window, positions
    [0, keep_first) stay visible after the window has passed them.  ``chunk`` > 0 (instead of a window): a query at
    position p sees positions [p - p % chunk, p].  ``values_in_keys``: the values are the first ``value_dim`` elements
    of the key rows (``v_pool`` is not read).  ``gate_per_head``: ``gate`` is [M, H], one number a head."""
    vd = head_dim if value_dim is None else value_dim
    if values_in_keys:
        assert vd <= head_dim
        v_pool = k_pool
    _need(q, "q", contiguous=False); _need(k_pool, "k_pool", q.dtype); _need(v_pool, "v_pool", q.dtype)
    _need(out, "out", q.dtype); _need(page_table, "page_table", torch.int32)
    _need(slot_of_token, "slot_of_token", torch.int32); _need(positions, "positions", torch.int32)
    M = q.shape[0]
    assert q.stride(1) == 1
    ldq = q.stride(0) if M > 1 else num_heads * head_dim
    ldg = 0
    if gate is not None:
        _need(gate, "gate", q.dtype, contiguous=False)
        assert gate.shape == (M, num_heads if gate_per_head else num_heads * vd) and gate.stride(1) == 1
        ldg = gate.stride(0) if M > 1 else gate.shape[1]
    _check(library().rl_attention_simt_shaped(
        q.data_ptr(), ldq, k_pool.data_ptr(), v_pool.data_ptr(), _dt(q), page_table.data_ptr(),
        page_table.shape[1], slot_of_token.data_ptr(), positions.data_ptr(), out.data_ptr(), out.stride(0),
        M, num_heads, num_kv_heads, head_dim, vd, float(scale), int(window), int(bool(sink)), _ptr(gate), ldg,
        float(softcap or 0.0), int(keep_first or 0), int(chunk or 0), head_dim if values_in_keys else 0,
        int(bool(gate_per_head)), _stream()),
        "rl_attention_simt")
    _count()


def layer_norm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
               weight2: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None) -> None:
    """out[r] = (x[r] - mean) / sqrt(mean of squared deviations + eps) * weight (x[rows[r]] if rows is given); with
    ``weight2`` and ``out2``: also the same row's norm times the second weight, from one read of x."""
    _need(x, "x", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    d = x.shape[-1]
    n = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        assert rows.numel() == n
    else:
        assert x.shape[0] == n
    assert weight.numel() == d and out.shape[-1] == d
    if (weight2 is None) != (out2 is None):
        raise KernelError("layer_norm: a second weight and a second output come together")
    if out2 is not None:
        _need(weight2, "weight2", torch.float32); _need(out2, "out2", out.dtype)
        assert weight2.numel() == d and out2.shape == out.shape
    _check(library().rl_layer_norm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), _ptr(weight2), _ptr(out2), _dt(out), _ptr(rows), n, d,
                                   float(eps), _stream()), "rl_layer_norm")
    _count()


def geglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out = gelu_tanh(gate) * up; layouts as for ``swiglu``."""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    M, two_i = gate_up.shape
    assert two_i % 2 == 0 and out.shape == (M, two_i // 2)
    _check(library().rl_geglu(gate_up.data_ptr(), out.data_ptr(), _dt(out), M, two_i // 2, int(interleaved), _stream()), "rl_geglu")
    _count()


def token_shift_mix(h: torch.Tensor, mu: torch.Tensor, positions: torch.Tensor, slot_of_token: torch.Tensor, cu_seqlens: torch.Tensor,
                    state: torch.Tensor, out: torch.Tensor) -> None:
    """out[s, m] = h[m] + (previous(m) - h[m]) * mu[s] for the n rows of ``mu`` (float32 [n, d]); previous(m) is the
    row in front where it belongs to the same sequence, else the sequence's state (float [d] a slot; zero at position
    0).  Leaves every sequence's last row of the step in its state.  h [M, d] (a view is fine), out [n, rows >= M, d]
    (rows beyond M, padding for a product that reads whole tiles, are left as they are)."""
    _need(h, "h", contiguous=False); _need(mu, "mu", torch.float32); _need(out, "out", h.dtype)
    _need(positions, "positions", torch.int32); _need(slot_of_token, "slot_of_token", torch.int32); _need(cu_seqlens, "cu_seqlens", torch.int32)
    M, d = h.shape
    n = mu.shape[0]
    assert mu.shape == (n, d) and out.shape[0] == n and out.shape[1] >= M and out.shape[2] == d and h.stride(1) == 1
    sp, ss = _state_args(state)
    assert state.shape[1] >= 4 * d
    _check(library().rl_token_shift_mix(h.data_ptr(), h.stride(0) if M > 1 else d, _dt(h), mu.data_ptr(), n, positions.data_ptr(),
                                        slot_of_token.data_ptr(), cu_seqlens.data_ptr(), cu_seqlens.numel() - 1, sp, ss, out.data_ptr(),
                                        out.shape[1], M, d, _stream()), "rl_token_shift_mix")
    _count()


def tanh_cast(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = tanh(x); x float32, out in its own dtype."""
    _need(x, "x", torch.float32); _need(out, "out")
    assert out.numel() == x.numel()
    _check(library().rl_tanh_cast(x.data_ptr(), out.data_ptr(), _dt(out), x.numel(), _stream()), "rl_tanh_cast")
    _count()


def scaled_add(x: torch.Tensor, y0: torch.Tensor, s0: float, y1: Optional[torch.Tensor] = None, s1: float = 0.0) -> None:
    """x += s0 * y0 + s1 * y1, all float32 of one shape (``y1`` may be ``None``)."""
    _need(x, "x", torch.float32); _need(y0, "y0", torch.float32)
    assert y0.shape == x.shape
    if y1 is not None:
        _need(y1, "y1", torch.float32)
        assert y1.shape == x.shape
    _check(library().rl_scaled_add(x.data_ptr(), y0.data_ptr(), float(s0), _ptr(y1), float(s1), x.numel(), _stream()), "rl_scaled_add")
    _count()


def row_gate_add(x: torch.Tensor, y: torch.Tensor, h: torch.Tensor, gate: torch.Tensor) -> None:
    """x[m] += sigmoid(h[m] . gate) * y[m]; x, y float32 [M, d]; h [M, d] and gate [d] in the compute dtype."""
    _need(x, "x", torch.float32); _need(y, "y", torch.float32); _need(h, "h", contiguous=False); _need(gate, "gate", h.dtype)
    M, d = x.shape
    assert y.shape == (M, d) and h.shape == (M, d) and gate.numel() == d and h.stride(1) == 1
    _check(library().rl_row_gate_add(x.data_ptr(), y.data_ptr(), h.data_ptr(), h.stride(0) if M > 1 else d, gate.data_ptr(), _dt(h), M, d,
                                     _stream()), "rl_row_gate_add")
    _count()


def scale(y: torch.Tensor, s: float) -> None:
    """y *= s in place (float32)."""
    _need(y, "y", torch.float32)
    _check(library().rl_scale(y.data_ptr(), y.numel(), float(s), _stream()), "rl_scale")
    _count()


# ----------------------------------------------------------------------------- short convolutions, recurrences, fused norms
def _state_args(state: torch.Tensor):
    """Pointer and row stride (in floats) of a per-slot state view [slots, nbytes] (uint8; a column range of the
    cache's state area, so rows are further apart than they are long)."""
    _need(state, "state", torch.uint8, contiguous=False)
    assert state.dim() == 2 and state.stride(1) == 1 and state.stride(0) % 4 == 0 and state.data_ptr() % 4 == 0
    return state.data_ptr(), state.stride(0) // 4


def short_conv(u: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], silu: bool, slot_of_token: torch.Tensor,
               state: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, c] = act(bias[c] + sum_j weight[c, j] * u[t - taps + 1 + j, c]) along each sequence; inputs of earlier
    steps come from ``state`` (per slot float [taps - 1, C], written by ``short_conv_state`` afterwards)."""
    _need(u, "u", contiguous=False); _need(weight, "weight", torch.float32); _need(out, "out", u.dtype, contiguous=False)
    _need(slot_of_token, "slot_of_token", torch.int32)
    M, C = out.shape
    taps = weight.shape[1]
    assert weight.shape == (C, taps) and u.shape == (M, C) and u.stride(1) == 1 and out.stride(1) == 1
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == C
    sp, ss = _state_args(state)
    assert state.shape[1] >= 4 * (taps - 1) * C
    _check(library().rl_short_conv(u.data_ptr(), u.stride(0), _dt(u), weight.data_ptr(), _ptr(bias), int(bool(silu)), C, taps,
                                   slot_of_token.data_ptr(), sp, ss, out.data_ptr(), out.stride(0), M, _stream()), "rl_short_conv")
    _count()


def short_conv_state(u: torch.Tensor, taps: int, cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, state: torch.Tensor) -> None:
    """After the step's convolution: every sequence's state takes its last ``taps - 1`` inputs."""
    _need(u, "u", contiguous=False); _need(cu_seqlens, "cu_seqlens", torch.int32); _need(seq_slots, "seq_slots", torch.int32)
    M, C = u.shape
    assert u.stride(1) == 1
    sp, ss = _state_args(state)
    assert state.shape[1] >= 4 * (taps - 1) * C
    if taps <= 1:
        return
    _check(library().rl_short_conv_state(u.data_ptr(), u.stride(0), _dt(u), C, int(taps), cu_seqlens.data_ptr(), seq_slots.data_ptr(),
                                         seq_slots.numel(), sp, ss, _stream()), "rl_short_conv_state")
    _count()


def qkv_prepare(u: torch.Tensor, q_out: torch.Tensor, conv_weight: Optional[torch.Tensor], state: Optional[torch.Tensor],
                q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float, positions: torch.Tensor,
                slot_of_token: torch.Tensor, page_table: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, magnitude: float,
                num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor]) -> None:
    """From the projected rows u [M, H*hd + G*hd + G*vd]: a short convolution over time (``conv_weight`` float
    [C, taps] with its per-slot ``state``), an RMS norm of every query and key head (``q_norm``, ``k_norm`` float
    [hd]), the rotary encoding of the first ``rotary_dim`` dimensions (half-split pairs, cos and sin times
    ``magnitude``), queries to ``q_out`` [M, H*hd], keys and values to their pages.  Every stage is optional."""
    _need(u, "u"); _need(q_out, "q_out", u.dtype); _need(positions, "positions", torch.int32)
    _need(slot_of_token, "slot_of_token", torch.int32); _need(page_table, "page_table", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    M = u.shape[0]
    C = (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim
    assert u.shape[1] == C and q_out.shape == (M, num_heads * head_dim) and inv_freq.numel() >= max(1, rotary_dim // 2)
    taps, sp, ss = 0, None, 0
    if conv_weight is not None:
        _need(conv_weight, "conv_weight", torch.float32)
        taps = conv_weight.shape[1]
        assert conv_weight.shape == (C, taps)
        if taps > 1:
            sp, ss = _state_args(state)
            assert state.shape[1] >= 4 * (taps - 1) * C
    for t, name in ((q_norm, "q_norm"), (k_norm, "k_norm")):
        if t is not None:
            _need(t, name, torch.float32)
            assert t.numel() == head_dim
    if k_pool is not None:
        _need(k_pool, "k_pool", u.dtype); _need(v_pool, "v_pool", u.dtype)
        assert k_pool.shape[1:] == (num_kv_heads, PAGE_SIZE, head_dim) and v_pool.shape[1:] == (num_kv_heads, PAGE_SIZE, value_dim)
    _check(library().rl_qkv_prepare(u.data_ptr(), u.stride(0), q_out.data_ptr(), q_out.stride(0), _dt(u), _ptr(conv_weight), taps,
                                    sp, ss, _ptr(q_norm), _ptr(k_norm), float(eps), positions.data_ptr(), slot_of_token.data_ptr(),
                                    page_table.data_ptr(), page_table.shape[1], inv_freq.data_ptr(), int(rotary_dim), float(magnitude),
                                    M, num_heads, num_kv_heads, head_dim, value_dim, _ptr(k_pool), _ptr(v_pool), _stream()),
           "rl_qkv_prepare")
    _count()


def qk_rotate_unit(u: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, slot_of_token: torch.Tensor,
                   page_table: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, interleaved: bool, unit_eps: Optional[float],
                   num_heads: int, num_kv_heads: int, head_dim: int, k_pool: Optional[torch.Tensor],
                   v_pool: Optional[torch.Tensor], value_from_key: bool = False) -> None:
    """From the projected rows u [M, >= (H + G) * hd] (queries, then keys): every head's first ``rotary_dim`` dimensions
    are turned by the token's position, then (``unit_eps`` not None) the head is divided by its root mean square;
    queries to ``q_out`` [M, H*hd] (a view of u is fine), keys to their pages.  ``value_from_key``: the key heads as
    projected are the values and go to ``v_pool``."""
    _need(u, "u", contiguous=False); _need(q_out, "q_out", u.dtype, contiguous=False); _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    M = u.shape[0]
    assert u.stride(1) == 1 and q_out.stride(1) == 1 and u.shape[1] >= (num_heads + num_kv_heads) * head_dim
    assert q_out.shape[1] >= num_heads * head_dim and inv_freq.numel() >= max(1, rotary_dim // 2)
    max_pages = 0
    if k_pool is not None:
        _need(k_pool, "k_pool", u.dtype); _need(slot_of_token, "slot_of_token", torch.int32); _need(page_table, "page_table", torch.int32)
        assert k_pool.shape[1:] == (num_kv_heads, PAGE_SIZE, head_dim), k_pool.shape
        if value_from_key:
            _need(v_pool, "v_pool", u.dtype)
            assert v_pool.shape == k_pool.shape
        max_pages = page_table.shape[1]
    ldu = u.stride(0) if M > 1 else u.shape[1]
    ldq = q_out.stride(0) if M > 1 else q_out.shape[1]
    _check(library().rl_qk_rotate_unit(u.data_ptr(), ldu, q_out.data_ptr(), ldq, _dt(u), positions.data_ptr(), _ptr(slot_of_token),
                                       _ptr(page_table), max_pages, inv_freq.data_ptr(), int(rotary_dim), int(bool(interleaved)),
                                       int(unit_eps is not None), float(unit_eps or 0.0), M, num_heads, num_kv_heads, head_dim,
                                       int(bool(value_from_key)), _ptr(k_pool), _ptr(v_pool) if value_from_key else None, _stream()),
           "rl_qk_rotate_unit")
    _count()


def latent_prepare(u: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, q_weight: Optional[torch.Tensor],
                   kv_weight: torch.Tensor, eps: float, cq: Optional[torch.Tensor], positions: torch.Tensor,
                   slot_of_token: torch.Tensor, page_table: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int,
                   interleaved: bool, k_pool: Optional[torch.Tensor]) -> None:
    """u [M, >= q_rank + kv_rank + rot_dim] = [query latent | key/value latent | shared rotary key] as projected:
    cq = rms_norm(query latent) * q_weight; the token's key row [rms_norm(key/value latent) * kv_weight | turned rotary
    key] goes to its page of ``k_pool`` [pages, 1, PAGE_SIZE, kv_rank + rot_dim]."""
    _need(u, "u", contiguous=False); _need(positions, "positions", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    _need(kv_weight, "kv_weight", torch.float32)
    M = u.shape[0]
    assert u.stride(1) == 1 and u.shape[1] >= q_rank + kv_rank + rot_dim and kv_weight.numel() == kv_rank
    ldc = 0
    if q_rank:
        _need(q_weight, "q_weight", torch.float32); _need(cq, "cq", u.dtype, contiguous=False)
        assert q_weight.numel() == q_rank and cq.shape == (M, q_rank) and cq.stride(1) == 1
        ldc = cq.stride(0) if M > 1 else q_rank
    max_pages = 0
    if k_pool is not None:
        _need(k_pool, "k_pool", u.dtype); _need(slot_of_token, "slot_of_token", torch.int32); _need(page_table, "page_table", torch.int32)
        assert k_pool.shape[1:] == (1, PAGE_SIZE, kv_rank + rot_dim), k_pool.shape
        max_pages = page_table.shape[1]
    ldu = u.stride(0) if M > 1 else u.shape[1]
    _check(library().rl_latent_prepare(u.data_ptr(), ldu, _dt(u), int(q_rank), int(kv_rank), int(rot_dim), _ptr(q_weight),
                                       kv_weight.data_ptr(), float(eps), _ptr(cq) if q_rank else None, ldc, positions.data_ptr(),
                                       _ptr(slot_of_token), _ptr(page_table), max_pages, inv_freq.data_ptr(), int(rotary_dim),
                                       int(bool(interleaved)), M, _ptr(k_pool), _stream()), "rl_latent_prepare")
    _count()


def latent_query(q: torch.Tensor, out: torch.Tensor, num_heads: int, head_dim: int, rot_dim: int, latent_dim: int,
                 positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int, interleaved: bool) -> None:
    """q [M, H * (hd + rd)] (a head: [plain | rotary]); the turned rotary parts go behind the ``latent_dim`` columns of
    each head of ``out`` [M, H * (latent_dim + rd)]."""
    _need(q, "q", contiguous=False); _need(out, "out", q.dtype); _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    M = q.shape[0]
    assert q.stride(1) == 1 and q.shape[1] == num_heads * (head_dim + rot_dim) and out.shape == (M, num_heads * (latent_dim + rot_dim))
    ldq = q.stride(0) if M > 1 else q.shape[1]
    _check(library().rl_latent_query(q.data_ptr(), ldq, _dt(q), num_heads, head_dim, rot_dim, positions.data_ptr(),
                                     inv_freq.data_ptr(), int(rotary_dim), int(bool(interleaved)), out.data_ptr(), out.stride(0),
                                     latent_dim, M, _stream()), "rl_latent_query")
    _count()


HEADS_LINEAR_MAX_K = 768      # inputs a head that ``heads_linear`` holds in shared memory


def heads_linear(x: torch.Tensor, x_head: int, w: torch.Tensor, out: torch.Tensor, out_head: int) -> None:
    """A product a head in one launch, for few tokens: out[m, a * out_head + n] = sum_k w[a, n, k] x[m, a * x_head + k].
    x: [M, >= (H - 1) * x_head + K]; w: [H, N, K]; out: [M, >= (H - 1) * out_head + N]; one dtype, sums in 32-bit."""
    _need(x, "x", contiguous=False); _need(w, "w", x.dtype); _need(out, "out", x.dtype, contiguous=False)
    H, N, Kd = w.shape
    M = x.shape[0]
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == M and Kd <= HEADS_LINEAR_MAX_K
    ldx = x.stride(0) if M > 1 else x.shape[1]
    ldo = out.stride(0) if M > 1 else out.shape[1]
    _check(library().rl_heads_linear(x.data_ptr(), ldx, int(x_head), w.data_ptr(), out.data_ptr(), ldo, int(out_head), _dt(x),
                                     M, H, N, Kd, _stream()), "rl_heads_linear")
    _count()


def linear_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, state: torch.Tensor,
                cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, num_heads: int, heads_per_group: int, dk: int, dv: int,
                rate: torch.Tensor, dt_raw: Optional[torch.Tensor] = None, dt_bias: Optional[torch.Tensor] = None,
                skip: Optional[torch.Tensor] = None, silu: bool = False) -> None:
    """S_t = a_t S_{t-1} + b_t k_t v_t^T, out_t = S_t^T q_t (+ skip[h] v_t) for every head of every sequence of the
    step, the state (float [H, dv, dk] a slot) read from and left in ``state``.  Without ``dt_raw``: a_t = rate[h],
    b_t = 1.  With it: dt = softplus(dt_raw[t, h] + dt_bias[h]), a_t = exp(-exp(rate[h]) * dt), b_t = dt.  q, k
    [M, (H / heads_per_group) * dk], v [M, H * dv] (views are fine), out float32 [M, H * dv].  ``silu``: q, k and v
    pass through silu first."""
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _need(t, name, q.dtype, contiguous=False)
        assert t.stride(1) == 1
    _need(out, "out", torch.float32); _need(rate, "rate", torch.float32)
    _need(cu_seqlens, "cu_seqlens", torch.int32); _need(seq_slots, "seq_slots", torch.int32)
    M = out.shape[0]
    assert out.shape == (M, num_heads * dv) and rate.numel() == num_heads and num_heads % heads_per_group == 0
    assert q.shape == (M, num_heads // heads_per_group * dk) and k.shape == q.shape and v.shape == (M, num_heads * dv)
    mode, lddt = 0, 0
    if dt_raw is not None:
        _need(dt_raw, "dt_raw", q.dtype, contiguous=False); _need(dt_bias, "dt_bias", torch.float32)
        assert dt_raw.shape == (M, num_heads) and dt_raw.stride(1) == 1 and dt_bias.numel() == num_heads
        mode, lddt = 1, dt_raw.stride(0)
    if skip is not None:
        _need(skip, "skip", torch.float32)
        assert skip.numel() == num_heads
    sp, ss = _state_args(state)
    assert state.shape[1] >= 4 * num_heads * dk * dv
    _check(library().rl_linear_scan(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), _ptr(dt_raw), lddt,
                                    _dt(q), _ptr(dt_bias), rate.data_ptr(), _ptr(skip), mode, int(bool(silu)), cu_seqlens.data_ptr(),
                                    seq_slots.data_ptr(), seq_slots.numel(), sp, ss, out.data_ptr(), out.stride(0), num_heads,
                                    heads_per_group, dk, dv, int(M >= 4 * seq_slots.numel()), _stream()), "rl_linear_scan")
    _count()


def channel_decay_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, wlog: torch.Tensor, bonus: torch.Tensor, out: torch.Tensor,
                       state: torch.Tensor, cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, num_heads: int, dk: int, dv: int) -> None:
    """out_t = (S_{t-1} + diag(bonus[h]) k_t v_t^T)^T q_t, then S_t = diag(w_t) S_{t-1} + k_t v_t^T with
    w_t = exp(-exp(wlog_t)), for every head of every sequence of the step; the state (float [H, dv, dk] a slot) is read
    from and left in ``state``.  q, k [M, H * dk], v [M, H * dv] (views are fine), wlog float32 [M, H * dk], bonus
    float32 [H, dk], out float32 [M, H * dv]."""
    for t, name in ((q, "q"), (k, "k"), (v, "v")):
        _need(t, name, q.dtype, contiguous=False)
        assert t.stride(1) == 1
    _need(out, "out", torch.float32); _need(wlog, "wlog", torch.float32, contiguous=False); _need(bonus, "bonus", torch.float32)
    _need(cu_seqlens, "cu_seqlens", torch.int32); _need(seq_slots, "seq_slots", torch.int32)
    M = out.shape[0]
    assert out.shape == (M, num_heads * dv) and q.shape == (M, num_heads * dk) and k.shape == q.shape and v.shape == (M, num_heads * dv)
    assert wlog.shape == (M, num_heads * dk) and wlog.stride(1) == 1 and bonus.numel() == num_heads * dk
    sp, ss = _state_args(state)
    assert state.shape[1] >= 4 * num_heads * dk * dv
    _check(library().rl_channel_decay_scan(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), _dt(q),
                                           wlog.data_ptr(), wlog.stride(0), bonus.data_ptr(), cu_seqlens.data_ptr(), seq_slots.data_ptr(),
                                           seq_slots.numel(), sp, ss, out.data_ptr(), out.stride(0), num_heads, dk, dv,
                                           int(M >= 4 * seq_slots.numel()), _stream()), "rl_channel_decay_scan")
    _count()


def norm_add(x: torch.Tensor, y0: torch.Tensor, s0: float, y1: Optional[torch.Tensor], s1: float, weight: torch.Tensor, eps: float,
             x_bf16: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> None:
    """x += out_scale * rms_norm(s0 * y0 + s1 * y1) * weight, all float32 [M, d] (``y1`` may be ``None``); ``x_bf16``:
    also leave the new x there, rounded."""
    _need(x, "x", torch.float32); _need(y0, "y0", torch.float32); _need(weight, "weight", torch.float32)
    M, d = x.shape
    assert y0.shape == (M, d) and weight.numel() == d
    if y1 is not None:
        _need(y1, "y1", torch.float32)
        assert y1.shape == (M, d)
    if x_bf16 is not None:
        _need(x_bf16, "x_bf16", torch.bfloat16)
        assert x_bf16.shape == (M, d)
    _check(library().rl_norm_add(x.data_ptr(), y0.data_ptr(), float(s0), _ptr(y1), float(s1), weight.data_ptr(), float(eps),
                                 float(out_scale), M, d, _ptr(x_bf16), _stream()), "rl_norm_add")
    _count()


def gated_norm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, groups: int = 1,
               gate_act: str = "silu", gate_first: bool = True) -> None:
    """``gate_first``: out = rms_norm_in_groups(y * act(gate)) * weight; else out = rms_norm(y) * weight * act(gate).
    y float32 [M, n]; gate and out [M, n] in the compute dtype (views are fine); the norm runs over ``groups``
    equal parts of a row, each by its own root mean square."""
    _need(y, "y", torch.float32, contiguous=False); _need(gate, "gate", out.dtype, contiguous=False)
    _need(out, "out", contiguous=False); _need(weight, "weight", torch.float32)
    M, n = y.shape
    assert gate.shape == (M, n) and out.shape == (M, n) and weight.numel() == n and n % groups == 0
    assert y.stride(1) == 1 and gate.stride(1) == 1 and out.stride(1) == 1
    act = {"silu": 0, "sigmoid": 1}[gate_act]
    _check(library().rl_gated_norm(y.data_ptr(), y.stride(0), gate.data_ptr(), gate.stride(0), _dt(out), act, int(bool(gate_first)),
                                   weight.data_ptr(), float(eps), M, groups, n // groups, out.data_ptr(), out.stride(0), _stream()),
           "rl_gated_norm")
    _count()


def gelu_gate(t: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, col0: int, out: torch.Tensor) -> None:
    """out[m, i] = gelu_tanh(t[m, i]) * table[tokens[m], col0 + i]."""
    _need(t, "t"); _need(tokens, "tokens", torch.int32); _need(table, "table", t.dtype); _need(out, "out", t.dtype)
    M, n = t.shape
    assert out.shape == (M, n) and tokens.numel() == M and 0 <= col0 and col0 + n <= table.shape[1]
    _check(library().rl_gelu_gate(t.data_ptr(), t.stride(0), tokens.data_ptr(), table.data_ptr(), table.stride(0), int(col0), n, _dt(t),
                                  out.data_ptr(), out.stride(0), M, _stream()), "rl_gelu_gate")
    _count()


def moe_route_sigmoid(x: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int, keep: int,
                      ids: torch.Tensor, weights: torch.Tensor) -> None:
    """Router with sigmoid scores: s = sigmoid(router @ x[m]) in 32-bit; experts are chosen by s + correction among
    the ``keep`` best of ``groups`` groups of neighbours (a group's score: its two largest choice scores); the
    weights are the chosen experts' s as they are."""
    _need(x, "x", contiguous=False); _need(router, "router", x.dtype); _need(ids, "ids", torch.int32)
    _need(weights, "weights", torch.float32)
    M, d = x.shape
    E = router.shape[0]
    assert router.shape == (E, d) and ids.shape == (M, top) and weights.shape == (M, top) and x.stride(1) == 1
    if correction is not None:
        _need(correction, "correction", torch.float32)
        assert correction.numel() == E
    _check(library().rl_moe_route_sigmoid(x.data_ptr(), x.stride(0) if M > 1 else d, router.data_ptr(), _ptr(correction), _dt(x), M, d,
                                          E, int(top), int(groups), int(keep), ids.data_ptr(), weights.data_ptr(), _stream()),
           "rl_moe_route_sigmoid")
    _count()


def moe_select_sigmoid(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int, keep: int,
                       ids: torch.Tensor, weights: torch.Tensor) -> None:
    """``moe_route_sigmoid``'s second half alone, from float32 logits [M, E]."""
    _need(logits, "logits", torch.float32); _need(ids, "ids", torch.int32); _need(weights, "weights", torch.float32)
    M, E = logits.shape
    assert ids.shape == (M, top) and weights.shape == (M, top)
    _check(library().rl_moe_select_sigmoid(logits.data_ptr(), M, E, int(top), _ptr(correction), int(groups), int(keep), ids.data_ptr(),
                                           weights.data_ptr(), _stream()), "rl_moe_select_sigmoid")
    _count()



def moe_route_scored(x: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int, keep: int,
                     ids: torch.Tensor, weights: torch.Tensor, softmax_all: bool, group_top: int, renorm: bool) -> None:
    """``moe_route_sigmoid`` with its variants as arguments: ``softmax_all`` - scores are the softmax of the logits over
    all experts; ``group_top`` - a group's score is the sum of its 1 or 2 largest choice scores; ``renorm`` - the
    weights are the chosen scores over their sum (+ 1e-20)."""
    _need(x, "x", contiguous=False); _need(router, "router", x.dtype); _need(ids, "ids", torch.int32)
    _need(weights, "weights", torch.float32)
    M, d = x.shape
    E = router.shape[0]
    assert router.shape == (E, d) and ids.shape == (M, top) and weights.shape == (M, top) and x.stride(1) == 1
    if correction is not None:
        _need(correction, "correction", torch.float32)
        assert correction.numel() == E
    _check(library().rl_moe_route_scored(x.data_ptr(), x.stride(0) if M > 1 else d, router.data_ptr(), _ptr(correction), _dt(x), M, d,
                                         E, int(top), int(groups), int(keep), int(bool(softmax_all)), int(group_top), int(bool(renorm)),
                                         ids.data_ptr(), weights.data_ptr(), _stream()), "rl_moe_route_scored")
    _count()


def moe_select_scored(logits: torch.Tensor, correction: Optional[torch.Tensor], top: int, groups: int, keep: int,
                      ids: torch.Tensor, weights: torch.Tensor, softmax_all: bool, group_top: int, renorm: bool) -> None:
    """``moe_route_scored``'s second half alone, from float32 logits [M, E]."""
    _need(logits, "logits", torch.float32); _need(ids, "ids", torch.int32); _need(weights, "weights", torch.float32)
    M, E = logits.shape
    assert ids.shape == (M, top) and weights.shape == (M, top)
    _check(library().rl_moe_select_scored(logits.data_ptr(), M, E, int(top), _ptr(correction), int(groups), int(keep),
                                          int(bool(softmax_all)), int(group_top), int(bool(renorm)), ids.data_ptr(), weights.data_ptr(),
                                          _stream()), "rl_moe_select_scored")
    _count()


def repeat_penalty(logits: torch.Tensor, recent: torch.Tensor, recent_len: torch.Tensor, penalty: float) -> None:
    _need(logits, "logits", torch.float32); _need(recent, "recent", torch.int32)
    _need(recent_len, "recent_len", torch.int32)
    rows, vocab = logits.shape
    assert recent.shape[0] == rows and recent_len.numel() == rows
    _check(library().rl_repeat_penalty(logits.data_ptr(), rows, vocab, recent.data_ptr(), recent_len.data_ptr(),
                                       recent.shape[1], float(penalty), _stream()), "rl_repeat_penalty")
    _count()


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    rows, vocab = logits.shape
    assert out.numel() == rows
    _check(library().rl_argmax(logits.data_ptr(), rows, vocab, out.data_ptr(), _stream()), "rl_argmax")
    _count()


def sample_temperature(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
                       out: torch.Tensor, min_p: Optional[torch.Tensor] = None) -> None:
    _need(logits, "logits", torch.float32); _need(temperature, "temperature", torch.float32)
    _need(uniform, "uniform", torch.float32); _need(out, "out", torch.int32)
    rows, vocab = logits.shape
    assert temperature.numel() == rows and uniform.numel() == rows and out.numel() == rows
    if min_p is not None:
        _need(min_p, "min_p", torch.float32)
    _check(library().rl_sample_temperature(logits.data_ptr(), rows, vocab, temperature.data_ptr(),
                                           uniform.data_ptr(), _ptr(min_p), out.data_ptr(), _stream()),
           "rl_sample_temperature")
    _count()


PAGE_SIZE = 64


def page_size() -> int:
    """Tokens per cache page.  A constant on the Python side so that host-side code
    (allocators, their tests) runs without a GPU; checked against the value the
    kernels were compiled with when the library is loaded."""
    return PAGE_SIZE


# ----------------------------------------------------------------------------- tensor-core GEMM
_tc_err = {}


def _tc_error_word(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _tc_err:
        _tc_err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_err[key]


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """Parts (cluster size) the kernel cuts the K range into for these shapes."""
    return int(library().rl_gemm_tc_splits(M, N, K))


def check_device_errors() -> None:
    """Raise if a kernel recorded an error on the device (a bounded wait that ran
    out).  Synchronizes; call it where the host waits for results anyway."""
    for key, t in _tc_err.items():
        code = int(t.item())
        if code != 0:
            t.zero_()
            raise KernelError(f"a tensor-core kernel on cuda:{key} gave up waiting (code {code}; matrix product: "
                              "1 = for a free stage, 2 = for a TMA load, 3 = for the accumulator, 4 = for a free "
                              "accumulator; prefill attention: 11 = producer, 12/13 = MMA issuer, 14 = softmax)")


def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes these operands (else the caller uses
    the CUDA-core kernel, which takes every shape): bf16, K and the row stride of
    ``a`` multiples of 8 elements, bases 16-byte aligned."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or a.stride(1) != 1:
        return False
    M, K = a.shape
    lda = a.stride(0) if M > 1 else K
    return bool(library().rl_gemm_tc_supported(a.data_ptr(), w.data_ptr(), M, w.shape[0], K, lda))


def norm_pieces(num_columns: int) -> int:
    """How many partial sums of squares a row the matrix product writes for ``num_columns``
    output columns when it prepares the next norm (4 per tile of 128 columns)."""
    return 4 * (-(-num_columns // 128))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, out_mode: int,
            bias: Optional[torch.Tensor] = None, force_splits: int = 0,
            row_sumsq: Optional[torch.Tensor] = None, row_eps: float = 0.0,
            norm_weight: Optional[torch.Tensor] = None, norm_out: Optional[torch.Tensor] = None,
            norm_sumsq: Optional[torch.Tensor] = None) -> None:
    """out = a @ w.T (+ bias) on the tensor cores (tcgen05).  a: [M, K] bf16, w: [N, K] bf16;
    out: bf16 (OUT_SAME) or float32 (OUT_F32 store, OUT_ADD_F32 add), or, with OUT_SWIGLU,
    bf16 [M, N/2] = silu(even columns) * odd columns of the product, or, with OUT_GELU, bf16 [M, N] = the tanh form
    of gelu of the product, computed in 32-bit from the accumulator.  force_splits: 0 = the
    kernel's own choice of K parts; 1 to 8 = as given.

    An RMSNorm around the product can ride along.  ``row_sumsq`` [M, pieces] float32 with
    ``row_eps``: ``a`` holds ``x * norm weight`` and row m of the product is multiplied by
    ``rsqrt(sum(row_sumsq[m]) / K + row_eps)``.  ``norm_weight`` [N], ``norm_out`` [M, N]
    bf16, ``norm_sumsq`` [M, norm_pieces(N)] float32 (OUT_ADD_F32 only): also
    ``norm_out = out * norm_weight`` and the sums of squares of ``out``'s rows, in pieces."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(w, "w", torch.bfloat16); _need(out, "out", contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(1) == 1
    if out_mode in (OUT_SWIGLU, OUT_GEGLU):      # rows of w are (gate_0, up_0, gate_1, ...): out = act(gate) * up, [M, N/2]
        assert N % 2 == 0 and out.shape == (M, N // 2) and out.dtype == torch.bfloat16
    else:
        assert out.shape == (M, N)
        assert out.dtype == (torch.bfloat16 if out_mode in (OUT_SAME, OUT_GELU) else torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == N
    pieces = 0
    if row_sumsq is not None:
        _need(row_sumsq, "row_sumsq", torch.float32)
        assert row_sumsq.dim() == 2 and row_sumsq.shape[0] == M
        pieces = row_sumsq.shape[1]
    if norm_weight is not None:
        _need(norm_weight, "norm_weight", torch.float32); _need(norm_out, "norm_out", torch.bfloat16)
        _need(norm_sumsq, "norm_sumsq", torch.float32)
        assert out_mode == OUT_ADD_F32 and norm_weight.numel() == N and norm_out.shape == (M, N)
        assert norm_sumsq.shape == (M, norm_pieces(N))
    lda = a.stride(0) if M > 1 else K
    ldo = out.stride(0) if M > 1 else out.shape[1]
    _check(library().rl_gemm_tc(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), out_mode, M, N, K, lda, ldo,
                                _tc_error_word(a.device).data_ptr(), int(force_splits),
                                _ptr(row_sumsq), pieces, float(row_eps),
                                _ptr(norm_weight), _ptr(norm_out), N, _ptr(norm_sumsq), _stream()), "rl_gemm_tc")
    _count()


def gemm_tc_qkv_rope_supported(a: torch.Tensor, w: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                               rotary_dim: int) -> bool:
    """Whether the QKV product of these operands can carry the rotary encoding and the cache
    write in its epilogue (head size 128 or 64 rotated whole, up to 64 tokens, a product that
    is split over K)."""
    if not gemm_tc_supported(a, w, None) or w.shape[0] != (num_heads + 2 * num_kv_heads) * head_dim:
        return False
    return bool(library().rl_gemm_tc_qkv_rope_supported(a.shape[0], num_heads, num_kv_heads, head_dim, rotary_dim, a.shape[1]))


def gemm_tc_qkv_rope(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor],
                     positions: torch.Tensor, slot_of_token: torch.Tensor, page_table: torch.Tensor,
                     inv_freq: torch.Tensor, interleaved: bool, num_heads: int, num_kv_heads: int,
                     k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                     row_sumsq: Optional[torch.Tensor] = None, row_eps: float = 0.0) -> None:
    """qkv = a @ w.T (+ bias) with rotary encoding of the query and key heads and the write of
    keys and values into the paged cache, all in the product's epilogue.  Of ``out``
    [M, (H + 2G) * head_dim] bf16 only the query heads are written; keys and values go to the
    pools (``None``: nowhere).  The head size (128 or 64) follows from ``w``'s rows.
    ``row_sumsq`` / ``row_eps``: as in ``gemm_tc``."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(w, "w", torch.bfloat16); _need(out, "out", torch.bfloat16, contiguous=False)
    _need(positions, "positions", torch.int32); _need(slot_of_token, "slot_of_token", torch.int32)
    _need(page_table, "page_table", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    M, K = a.shape
    hd = w.shape[0] // (num_heads + 2 * num_kv_heads)
    assert hd in (64, 128) and w.shape == ((num_heads + 2 * num_kv_heads) * hd, K)
    assert out.shape == (M, w.shape[0]) and out.stride(1) == 1
    assert positions.numel() == M and slot_of_token.numel() == M and inv_freq.numel() == hd // 2
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == w.shape[0]
    if k_pool is not None:
        _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16)
        assert k_pool.shape[1:] == (num_kv_heads, PAGE_SIZE, hd) and v_pool.shape == k_pool.shape
    pieces = 0
    if row_sumsq is not None:
        _need(row_sumsq, "row_sumsq", torch.float32)
        assert row_sumsq.dim() == 2 and row_sumsq.shape[0] == M
        pieces = row_sumsq.shape[1]
    lda = a.stride(0) if M > 1 else K
    ldo = out.stride(0) if M > 1 else out.shape[1]
    _check(library().rl_gemm_tc_qkv_rope(
        a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, K, lda, ldo, _tc_error_word(a.device).data_ptr(),
        _ptr(row_sumsq), pieces, float(row_eps), positions.data_ptr(), slot_of_token.data_ptr(), page_table.data_ptr(),
        page_table.shape[1], inv_freq.data_ptr(), 1 if interleaved else 0, num_heads, num_kv_heads, hd,
        _ptr(k_pool), _ptr(v_pool), _stream()), "rl_gemm_tc_qkv_rope")
    _count()


def _gate_args(gate: Optional[torch.Tensor], rows: int, width: int, align: int):
    """Pointer and row stride of an output gate [rows, width] bf16 (a view is fine), or (None, 0)."""
    if gate is None:
        return None, 0
    _need(gate, "gate", torch.bfloat16, contiguous=False)
    assert gate.shape == (rows, width) and gate.stride(1) == 1
    ldg = gate.stride(0) if rows > 1 else max(gate.stride(0), width)
    if gate.data_ptr() % align or (ldg * 2) % align:
        raise KernelError(f"the gate must be {align}-byte aligned, rows included")
    return gate.data_ptr(), ldg


# ----------------------------------------------------------------------------- decode attention
_num_sms = {}


def num_sms() -> int:
    """SMs of the current device, asked from the device once."""
    dev = torch.cuda.current_device() if torch.cuda.is_available() else -1
    if dev not in _num_sms:
        lib = library()
        lib.rl_sm_count.restype = _c_int
        lib.rl_sm_count.argtypes = []
        _num_sms[dev] = int(lib.rl_sm_count())
    return _num_sms[dev]


def attention_decode_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and bool(library().rl_attention_decode_supported(num_heads, num_kv_heads, head_dim))


# One sequence alone: up to this many cached tokens its eight chunks run as one cluster that
# combines through shared memory (one kernel; 6.0 us against 7.9 us at 1,024 tokens, equal at
# 4,096); beyond, sixteen chunks and the combining kernel (32,768 tokens: 30 us against 52 us;
# 131,072: 95 us against 198 us - 64 CTAs cannot keep the memory busy).  A captured step keeps
# its grid, so the step carries on which side of this it lies (``StepState.long_context``).
LONG_CONTEXT = 6144


def decode_splits(num_seqs: int, num_kv_heads: int) -> int:
    """Splits of the context per (sequence, KV head): enough CTAs for about one and a
    half per SM, at most 8 for a batch and 16 for one sequence (measured best at 1 to 64
    sequences of 800 and 4,096 tokens), and at least 2 for a batch, so that its chunks are
    dealt by length: beside short sequences a long one is then cut in pieces (64 sequences of
    256 to 8,700 tokens: 115 us as one chunk each, 95 us dealt), and a sequence that remains
    one chunk costs nothing more for it.  Depends on the batch's size only, so that a
    captured step keeps its grid."""
    most = 16 if num_seqs == 1 else 8
    least = 1 if num_seqs == 1 else 2
    return max(least, min(most, -(-3 * num_sms() // (2 * num_seqs * num_kv_heads))))


# Several sequences: how far the longest lies above the mean of all decides whether equal chunks a
# sequence (a cluster, one kernel) or chunks dealt by length (and a second kernel that combines
# them) serve them better; a captured step keeps its launches, so the step carries the class
# (``StepState.length_spread``): 0 = within EVEN_SPREAD tokens, 1 = within NEAR_SPREAD, 2 = within
# FAR_SPREAD and the longest no more than one in LONGEST_SHARE of all tokens (63 sequences of 100
# tokens beside one of 4,000, whole: 50 us, dealt: 24 us), 3 = the rest.
EVEN_SPREAD = 16
NEAR_SPREAD = 768
FAR_SPREAD = 4096
LONGEST_SHARE = 20


def length_spread(kv_lens: Sequence[int]) -> int:
    """The class of a batch's lengths (see above); one sequence is class 0."""
    n = len(kv_lens)
    over = max(kv_lens) * n - sum(kv_lens)        # (longest - mean) * n, in integers
    if over <= NEAR_SPREAD * n:
        return 0 if over <= EVEN_SPREAD * n else 1
    return 2 if over <= FAR_SPREAD * n and max(kv_lens) * LONGEST_SHARE <= sum(kv_lens) else 3


def decode_places(head_dim: int) -> int:
    """CTAs of the decode kernel the GPU holds at once at this head size (296 at 128, 444 at 64)."""
    n = int(library().rl_attention_decode_places(int(head_dim)))
    if n <= 0:
        _check(n or -1, "rl_attention_decode_places")
    return n


def decode_order_wanted(num_seqs: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whole sequences that are more CTAs than the GPU holds at once (and keep 30 MB in flight
    among them) start in the order of their lengths, the longest first.  Sequences of 128 to 2,047
    tokens, in order against dealt chunks: head size 128, 40 sequences 36.4 / 38.6 us, 48: 39.1 /
    43.2, 56: 40.7 / 48.8, 64: 43.0 / 54.3 (6.45 TB/s; 53 us sorted but KV head by KV head, 52.7
    unsorted); head size 64, 96: 38.4 / 40.5, 128: 42.0 / 50.2, but 64 (24 MB in flight): 31.7 /
    30.4.  The order kernel takes up to 1,024 sequences."""
    ctas = num_seqs * num_kv_heads
    ring = int(library().rl_attention_decode_ring_bytes(int(head_dim)))
    return ctas > decode_places(head_dim) and ctas * ring >= 30_000_000 and num_seqs <= 1024


def decode_cluster_size(num_seqs: int, num_kv_heads: int, head_dim: int, long_context: bool, spread: int) -> int:
    """How the decode attention cuts the sequences of a step: 8, 4 or 2 = so many equal chunks a
    sequence as one cluster; 1 = every sequence whole in one CTA a KV head; 0 = chunks dealt by
    length and a combining kernel.  One sequence alone: eight chunks up to the long-context mark.
    Whole sequences in order (``decode_order_wanted``) serve every batch up to class 2.  Else,
    lengths that are equal (class 0) or near (class 1): where two chunks a sequence no longer fit
    the GPU at once, every sequence whole if that keeps 15 MB in flight (head size 64, 4,096
    tokens a sequence, whole against dealt: 32 sequences 59 / 49 us, 40: 61 / 73); else the largest
    power of two within ``decode_splits`` - for class 1 only if nothing is lost to the rounding.
    Whole decode steps of the 8B shape, 1,024 tokens a sequence, against dealt chunks: 2 sequences
    2.91 / 2.95 ms, 6: 3.04 / 3.12, 8: 3.10 / 3.18, 16: 3.30 / 3.38, 20: 3.57 / 3.84, 32: 3.81 / 4.05,
    64: 4.93 / 5.23; lengths 1,024 +- 30 %: 8: 3.13 / 3.19, 16: 3.36 / 3.42, 32: 3.84 / 4.06, 64: 5.05 /
    5.20, but 4 sequences (7 splits rounded to 4): 3.07 / 3.04, so those stay dealt; with the
    longest 80 % above the mean the two are about even, and beyond, the longest sequence's few
    CTAs would finish last.  (A cluster of two at 20 sequences, 320 CTAs for 296 places: 17.7 us
    against 10.9 us whole at 512 tokens.)"""
    splits = decode_splits(num_seqs, num_kv_heads)
    if num_seqs == 1:
        return 8 if splits >= 8 and not long_context else 0
    if splits < 2:
        return 0
    if decode_order_wanted(num_seqs, num_kv_heads, head_dim):
        return 1 if spread <= 2 else 0
    if spread > 1:
        return 0
    places, ctas = decode_places(head_dim), num_seqs * num_kv_heads
    if ctas * 2 > places:
        return 1 if ctas * int(library().rl_attention_decode_ring_bytes(int(head_dim))) >= 15_000_000 else 0
    size = 8 if splits >= 8 else 4 if splits >= 4 else 2
    if spread == 1 and size != splits:
        return 0
    return size if ctas * size <= places else 0


def decode_order(seq_slots: torch.Tensor, kv_lens: torch.Tensor, window: int) -> torch.Tensor:
    """A plan of whole sequences, the longest first (inside ``window`` if it is not 0), made on the
    device: for ``attention_decode`` with one split.  At most 1,024 sequences."""
    _need(seq_slots, "seq_slots", torch.int32); _need(kv_lens, "kv_lens", torch.int32)
    B = seq_slots.numel()
    assert kv_lens.numel() == B
    plan = torch.empty(6 * B, dtype=torch.int32, device=seq_slots.device)     # rl_attention_decode_order_ints
    _check(library().rl_attention_decode_order(seq_slots.data_ptr(), kv_lens.data_ptr(), B, int(window), plan.data_ptr(), _stream()),
           "rl_attention_decode_order")
    _count(1)
    return plan


def decode_scratch_floats(num_seqs: int, num_heads: int, head_dim: int, num_splits: int) -> int:
    if num_splits <= 1:
        return 0
    return num_seqs * num_heads * num_splits * (head_dim + 2)


def decode_plan(seq_slots: torch.Tensor, kv_lens: torch.Tensor, window: int, num_splits: int) -> Optional[torch.Tensor]:
    """Deals ``B * num_splits`` chunks to the sequences by their lengths, on the device.
    The plan serves every ``attention_decode`` call of the step with the same window and
    splits (``None`` with one split: every sequence is one chunk)."""
    _need(seq_slots, "seq_slots", torch.int32); _need(kv_lens, "kv_lens", torch.int32)
    B = seq_slots.numel()
    if num_splits <= 1 or B == 0:
        return None
    plan = torch.empty(4 * B * num_splits + 2 * B, dtype=torch.int32, device=seq_slots.device)
    _check(library().rl_attention_decode_plan(seq_slots.data_ptr(), kv_lens.data_ptr(), B, int(window), int(num_splits),
                                              plan.data_ptr(), _stream()), "rl_attention_decode_plan")
    _count(1)
    return plan


def attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                     seq_slots: torch.Tensor, kv_lens: torch.Tensor, out: torch.Tensor, num_heads: int,
                     num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                     num_splits: Optional[int] = None, scratch: Optional[torch.Tensor] = None,
                     plan: Optional[torch.Tensor] = None, cluster: bool = False, sink: bool = False,
                     gate: Optional[torch.Tensor] = None, softcap: float = 0.0, keep_first: int = 0,
                     gate_per_head: bool = False) -> None:
    """One token per sequence over the bf16 cache, split over the context (tensor cores).
    q: [B, >= H*hd] bf16 (a view into the qkv buffer is fine); out: [B, H*hd] bf16.
    ``num_splits``: chunks per sequence; with a ``plan`` (from ``decode_plan`` with the
    same sequences, window and splits) that many on average, dealt to the sequences by
    length; with one split a ``plan`` from ``decode_order`` starts the longest sequences first.
    ``cluster`` (2, 4 or 8 splits, no plan): the chunks of a sequence run as a
    thread-block cluster and combine through shared memory - no scratch, one kernel.
    ``softcap`` > 0: a score s (scale included) becomes softcap * tanh(s / softcap); ``keep_first``: with a
    window, positions [0, keep_first) stay visible."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(page_table, "page_table", torch.int32); _need(seq_slots, "seq_slots", torch.int32)
    _need(kv_lens, "kv_lens", torch.int32)
    B = q.shape[0]
    assert seq_slots.numel() == B and kv_lens.numel() == B and q.stride(1) == 1
    if num_splits is None:
        num_splits = decode_splits(B, num_kv_heads)
    if cluster:
        assert plan is None and scratch is None and num_splits in (2, 4, 8)
    need = 0 if cluster else decode_scratch_floats(B, num_heads, head_dim, num_splits)
    if num_splits > 1 and scratch is None and not cluster:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    if scratch is not None:
        _need(scratch, "scratch", torch.float32)
        assert scratch.numel() >= need
    if plan is not None:
        _need(plan, "plan", torch.int32)
        assert plan.numel() >= 4 * B * num_splits + 2 * B
    ldq = q.stride(0) if B > 1 else max(q.stride(0), num_heads * head_dim)
    gptr, ldg = _gate_args(gate, B, num_heads if gate_per_head else num_heads * head_dim, 2)
    _check(library().rl_attention_decode_headgate(
        q.data_ptr(), ldq, k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        seq_slots.data_ptr(), kv_lens.data_ptr(), out.data_ptr(), out.stride(0), _ptr(scratch), _ptr(plan), B,
        num_heads, num_kv_heads, head_dim, float(scale), int(window), int(num_splits), int(bool(sink)), gptr, ldg,
        float(softcap or 0.0), int(keep_first or 0), int(bool(gate_per_head and gate is not None)), _stream()), "rl_attention_decode")
    _count(2 if num_splits > 1 and not cluster else 1)


# ----------------------------------------------------------------------------- prefill attention
PREFILL_QTILE = 64


def attention_prefill_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and bool(library().rl_attention_prefill_supported(num_heads, num_kv_heads, head_dim))


def attention_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                      cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, kv_lens: torch.Tensor, q_lens,
                      out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                      window: int = 0, sink: bool = False, gate: Optional[torch.Tensor] = None) -> None:
    """Causal attention of packed query tokens over the bf16 cache (tensor cores).
    q: [M, >= H*hd] bf16; cu_seqlens [B+1], seq_slots [B], kv_lens [B] on the device;
    q_lens: host list of tokens per sequence; out: [M, H*hd] bf16."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(page_table, "page_table", torch.int32); _need(cu_seqlens, "cu_seqlens", torch.int32)
    _need(seq_slots, "seq_slots", torch.int32); _need(kv_lens, "kv_lens", torch.int32)
    B = len(q_lens)
    assert cu_seqlens.numel() == B + 1 and seq_slots.numel() == B and kv_lens.numel() == B
    assert q.shape[0] == sum(q_lens) and q.stride(1) == 1
    tiles = sum(-(-n // PREFILL_QTILE) for n in q_lens)
    ldq = q.stride(0) if q.shape[0] > 1 else max(q.stride(0), num_heads * head_dim)
    gptr, ldg = _gate_args(gate, q.shape[0], num_heads * head_dim, 4)
    _check(library().rl_attention_prefill_gated(
        q.data_ptr(), ldq, k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        cu_seqlens.data_ptr(), seq_slots.data_ptr(), kv_lens.data_ptr(), B, tiles, out.data_ptr(), out.stride(0),
        num_heads, num_kv_heads, head_dim, float(scale), int(window), int(bool(sink)), gptr, ldg, _stream()),
        "rl_attention_prefill")
    _count()


PREFILL_TC_QTILE = 128


def prefill_tile_order(q_lens, kv_lens, device) -> torch.Tensor:
    """For the tcgen05 prefill attention: the step's 128-query tiles as (sequence, tile of the
    sequence) pairs by falling number of keys (a tile attends to its sequence's cached prefix and
    to the step's tokens up to its own last one), int32 [tiles, 2] on the device.  Made once a
    step from the host's copies of the lengths and used by every layer."""
    items = []
    for b, (nq, nkv) in enumerate(zip(q_lens, kv_lens)):
        first = nkv - nq
        for t in range(-(-nq // PREFILL_TC_QTILE)):
            items.append((-(first + min(nq, (t + 1) * PREFILL_TC_QTILE)), b, t))
    items.sort()
    return torch.tensor([[b, t] for _, b, t in items], dtype=torch.int32).to(device, non_blocking=True)


def attention_prefill_tc_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and bool(library().rl_attention_prefill_tc_supported(num_heads, num_kv_heads, head_dim))


def attention_prefill_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                         cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, kv_lens: torch.Tensor, q_lens,
                         out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                         window: int = 0, tile_order: Optional[torch.Tensor] = None, sink: bool = False,
                         gate: Optional[torch.Tensor] = None, softcap: float = 0.0, keep_first: int = 0, chunk: int = 0,
                         gate_per_head: bool = False) -> None:
    """The same as ``attention_prefill`` on tcgen05 tensor cores (head size 64 or 128).  ``chunk`` > 0 (instead of a
    window): a query at position p sees positions [p - p % chunk, p].  The cache
    pools must hold finite values everywhere (the cache zero-fills them when it allocates them).
    ``tile_order``: what ``prefill_tile_order`` made for this step (the blocks then start heaviest first)."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(page_table, "page_table", torch.int32); _need(cu_seqlens, "cu_seqlens", torch.int32)
    _need(seq_slots, "seq_slots", torch.int32); _need(kv_lens, "kv_lens", torch.int32)
    B = len(q_lens)
    assert cu_seqlens.numel() == B + 1 and seq_slots.numel() == B and kv_lens.numel() == B
    assert q.shape[0] == sum(q_lens) and q.stride(1) == 1
    tiles = sum(-(-n // PREFILL_TC_QTILE) for n in q_lens)
    if tile_order is not None:
        _need(tile_order, "tile_order", torch.int32)
        assert tile_order.numel() == 2 * tiles
    ldq = q.stride(0) if q.shape[0] > 1 else max(q.stride(0), num_heads * head_dim)
    gptr, ldg = _gate_args(gate, q.shape[0], num_heads, 2) if gate_per_head else _gate_args(gate, q.shape[0], num_heads * head_dim, 16)
    _check(library().rl_attention_prefill_tc_headgate(
        q.data_ptr(), ldq, k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0], page_table.data_ptr(),
        page_table.shape[1], cu_seqlens.data_ptr(), seq_slots.data_ptr(), kv_lens.data_ptr(), B, tiles, q.shape[0],
        out.data_ptr(), out.stride(0), num_heads, num_kv_heads, head_dim, float(scale), int(window),
        _tc_error_word(q.device).data_ptr(), _ptr(tile_order), int(bool(sink)), gptr, ldg, float(softcap or 0.0),
        int(keep_first or 0), int(chunk or 0), int(bool(gate_per_head and gate is not None)), _stream()), "rl_attention_prefill_tc")
    _count()


def attention_shared_key_supported(dtype: torch.dtype, num_heads: int, key_dim: int, value_dim: int) -> bool:
    return dtype == torch.bfloat16 and bool(library().rl_attention_shared_key_supported(num_heads, key_dim, value_dim))


def attention_shared_key(q: torch.Tensor, k_pool: torch.Tensor, page_table: torch.Tensor, cu_seqlens: torch.Tensor,
                         seq_slots: torch.Tensor, kv_lens: torch.Tensor, q_lens, out: torch.Tensor, num_heads: int,
                         key_dim: int, value_dim: int, scale: float, window: int = 0,
                         gate: Optional[torch.Tensor] = None) -> None:
    """All query heads over ONE cached row a position whose first ``value_dim`` elements are the value (tensor cores,
    prompt portions and single tokens).  q: [M, >= H * key_dim] bf16; k_pool: [pages, 1, PAGE_SIZE, key_dim]; out:
    [M, H * value_dim]; ``gate`` [M, H]: head h's output is multiplied by sigmoid(gate[m, h])."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pool, "k_pool", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(page_table, "page_table", torch.int32); _need(cu_seqlens, "cu_seqlens", torch.int32)
    _need(seq_slots, "seq_slots", torch.int32); _need(kv_lens, "kv_lens", torch.int32)
    B, M = len(q_lens), q.shape[0]
    assert cu_seqlens.numel() == B + 1 and seq_slots.numel() == B and kv_lens.numel() == B
    assert M == sum(q_lens) and q.stride(1) == 1 and k_pool.shape[1:] == (1, PAGE_SIZE, key_dim), k_pool.shape
    assert out.shape == (M, num_heads * value_dim)
    one_each = all(n == 1 for n in q_lens)
    per_block = int(library().rl_attention_shared_key_block_tokens(num_heads, key_dim, int(one_each)))
    tiles = B if one_each else sum(-(-n // per_block) for n in q_lens)
    ldg = 0
    if gate is not None:
        _need(gate, "gate", torch.bfloat16, contiguous=False)
        assert gate.shape == (M, num_heads) and gate.stride(1) == 1
        ldg = gate.stride(0) if M > 1 else num_heads
    ldq = q.stride(0) if M > 1 else max(q.stride(0), num_heads * key_dim)
    # single tokens of few sequences: a sequence's key blocks in several runs, so that the step fills the GPU.  The
    # count depends on the batch's size and the window alone (a captured step keeps its grid).
    groups = -(-num_heads // 16)
    splits, part = 1, None
    if one_each:
        along_heads = int(library().rl_attention_shared_key_head_blocks(num_heads, key_dim, 1))
        splits = max(1, min(8, num_sms() // (B * along_heads)))
        if window:
            splits = min(splits, -(-int(window) // PAGE_SIZE) + 1)
        if splits > 1:
            part = torch.empty((B * groups * splits * 16 * (value_dim + 2),), dtype=torch.float32, device=q.device)
    _check(library().rl_attention_shared_key(
        q.data_ptr(), ldq, k_pool.data_ptr(), page_table.data_ptr(), page_table.shape[1], cu_seqlens.data_ptr(),
        seq_slots.data_ptr(), kv_lens.data_ptr(), B, tiles, int(one_each), out.data_ptr(), out.stride(0), _ptr(gate), ldg,
        num_heads, key_dim, value_dim, float(scale), int(window or 0), splits, _ptr(part), _stream()), "rl_attention_shared_key")
    _count()


# ----------------------------------------------------------------------------- attention dispatch
def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
              step, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
              window: int = 0, value_dim: Optional[int] = None, sink: bool = False,
              gate: Optional[torch.Tensor] = None, softcap: float = 0.0, keep_first: int = 0, chunk: int = 0,
              values_in_keys: bool = False, gate_per_head: bool = False) -> None:
    """Attention of the step's tokens over the cache; picks the kernel for the
    dtype and the shape of the step.  ``step`` carries positions, slots and
    sequence boundaries (engine.step.StepState).  Value heads of another width than the
    key heads (``value_dim``) run on the any-shape kernel; the tensor-core kernels take
    one width for both.  ``sink``: one more term of score 0 in the softmax's denominator.
    ``gate`` [M, H*vd]: the output is multiplied by sigmoid(gate) (``gate_per_head``: [M, H], one number a head).
    ``chunk`` > 0 instead of a window: a query sees the positions of its own block of ``chunk`` positions up to
    itself.  ``values_in_keys``: the values are the front part of the key rows (any-shape kernel)."""
    if chunk and window:
        raise KernelError("a chunked mask and a sliding window exclude one another")
    if (values_in_keys and num_kv_heads == 1 and (gate is None or gate_per_head) and not (sink or softcap or keep_first or chunk)
            and attention_shared_key_supported(q.dtype, num_heads, head_dim, head_dim if value_dim is None else value_dim)
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0):
        # all heads over one cached row whose front is the value: one kernel for prompt portions and single tokens
        attention_shared_key(q, k_pool, page_table, step.cu_seqlens, step.seq_slots, step.kv_lens, step.q_lens, out,
                             num_heads, head_dim, head_dim if value_dim is None else value_dim, scale, window, gate=gate)
        return
    vd_eff = head_dim if value_dim is None else value_dim
    tc_head_gate = (gate_per_head and gate is not None and not values_in_keys and vd_eff == head_dim and q.dtype == torch.bfloat16
                    and not chunk and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
                    and (attention_decode_supported(q.dtype, num_heads, num_kv_heads, head_dim) if step.is_decode else
                         attention_prefill_tc_supported(q.dtype, num_heads, num_kv_heads, head_dim)))
    if values_in_keys or (gate_per_head and not tc_head_gate):
        attention_simt(q, k_pool, v_pool, page_table, step.slot_of_token, step.positions, out,
                       num_heads, num_kv_heads, head_dim, scale, window, value_dim=value_dim, sink=sink, gate=gate,
                       softcap=softcap, keep_first=keep_first, chunk=chunk, values_in_keys=values_in_keys,
                       gate_per_head=gate_per_head)
        return
    # the decode kernel and its plans take a chunked mask as a negative window
    dec_window = -int(chunk) if chunk else int(window)
    masked = bool(softcap or (keep_first and window) or chunk)
    tc_prefill = (not step.is_decode and attention_prefill_tc_supported(q.dtype, num_heads, num_kv_heads, head_dim)
                  and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
                  and (gate is None or gate_per_head or (gate.data_ptr() % 16 == 0 and gate.stride(0) % 8 == 0)))
    if (value_dim is not None and value_dim != head_dim) or (masked and not tc_prefill and not (
            step.is_decode and attention_decode_supported(q.dtype, num_heads, num_kv_heads, head_dim))):
        # soft-capped scores, kept first tokens and chunked masks: the any-shape kernel, the decode kernel and the
        # tcgen05 prompt kernel have them (the mma.sync prompt kernel does not)
        attention_simt(q, k_pool, v_pool, page_table, step.slot_of_token, step.positions, out,
                       num_heads, num_kv_heads, head_dim, scale, window, value_dim=value_dim, sink=sink, gate=gate,
                       softcap=softcap, keep_first=keep_first, chunk=chunk)
        return
    if step.is_decode and attention_decode_supported(q.dtype, num_heads, num_kv_heads, head_dim):
        splits = decode_splits(q.shape[0], num_kv_heads)
        cluster = decode_cluster_size(q.shape[0], num_kv_heads, head_dim, getattr(step, "long_context", False),
                                      getattr(step, "length_spread", 3))
        if cluster:
            # nothing to deal: equal chunks a sequence as one cluster, combined through shared memory,
            # or every sequence whole
            order = None
            derived = getattr(step, "derived", None)
            if cluster == 1 and derived is not None and decode_order_wanted(q.shape[0], num_kv_heads, head_dim):
                order = derived.get(("decode_order", dec_window))
                if order is None:
                    order = derived[("decode_order", dec_window)] = decode_order(step.seq_slots, step.kv_lens, dec_window)
            attention_decode(q, k_pool, v_pool, page_table, step.seq_slots, step.kv_lens, out,
                             num_heads, num_kv_heads, head_dim, scale, dec_window, num_splits=cluster, plan=order,
                             cluster=cluster > 1, sink=sink, gate=gate, softcap=softcap, keep_first=keep_first,
                             gate_per_head=gate_per_head)
            return
        plan = None
        derived = getattr(step, "derived", None)     # what layers of one step share
        if splits > 1 and q.shape[0] > 1 and derived is not None:
            key = ("decode_plan", dec_window, splits)
            plan = derived.get(key)
            if plan is None:
                plan = derived[key] = decode_plan(step.seq_slots, step.kv_lens, dec_window, splits)
        attention_decode(q, k_pool, v_pool, page_table, step.seq_slots, step.kv_lens, out,
                         num_heads, num_kv_heads, head_dim, scale, dec_window, num_splits=splits, plan=plan, sink=sink, gate=gate,
                         softcap=softcap, keep_first=keep_first, gate_per_head=gate_per_head)
        return
    if tc_prefill:
        order = None
        derived = getattr(step, "derived", None)
        if derived is not None and len(step.q_lens) > 1:     # one sequence: the kernel's own reverse order is the heaviest first
            order = derived.get("prefill_tile_order")
            if order is None:
                order = derived["prefill_tile_order"] = prefill_tile_order(step.q_lens, step.kv_lens_host, q.device)
        attention_prefill_tc(q, k_pool, v_pool, page_table, step.cu_seqlens, step.seq_slots, step.kv_lens,
                             step.q_lens, out, num_heads, num_kv_heads, head_dim, scale, window, tile_order=order,
                             sink=sink, gate=gate, softcap=softcap, keep_first=keep_first, chunk=chunk, gate_per_head=gate_per_head)
        return
    if not chunk and not step.is_decode and attention_prefill_supported(q.dtype, num_heads, num_kv_heads, head_dim) \
            and (gate is None or (gate.data_ptr() % 4 == 0 and gate.stride(0) % 2 == 0)):
        attention_prefill(q, k_pool, v_pool, page_table, step.cu_seqlens, step.seq_slots, step.kv_lens,
                          step.q_lens, out, num_heads, num_kv_heads, head_dim, scale, window, sink=sink, gate=gate)
        return
    attention_simt(q, k_pool, v_pool, page_table, step.slot_of_token, step.positions, out,
                   num_heads, num_kv_heads, head_dim, scale, window, sink=sink, gate=gate, chunk=chunk)


from .sampling.config import MAX_TOP_K  # noqa: E402  (one definition, host side)


def sample_candidates(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
                      min_p: torch.Tensor, out: torch.Tensor,
                      topk_rows: Optional[torch.Tensor], topk_k: Optional[torch.Tensor], topk_p: Optional[torch.Tensor],
                      topp_rows: Optional[torch.Tensor], topp_p: Optional[torch.Tensor]) -> None:
    """Rows that sample from a candidate set.  ``topk_rows`` (int32 row indices, on the
    device) with their ``topk_k`` (int32, each at most ``MAX_TOP_K``) and ``topk_p`` (float32)
    take the top-k path; ``topp_rows`` with ``topp_p`` the top-p path over the whole
    vocabulary; ``None`` = no such rows.  temperature / uniform / min_p / out are indexed by
    logits row."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    _need(temperature, "temperature", torch.float32); _need(uniform, "uniform", torch.float32)
    _need(min_p, "min_p", torch.float32)
    n_k = n_p = 0
    if topk_rows is not None:
        _need(topk_rows, "topk_rows", torch.int32); _need(topk_k, "topk_k", torch.int32); _need(topk_p, "topk_p", torch.float32)
        n_k = topk_rows.numel()
        assert topk_k.numel() == n_k and topk_p.numel() == n_k
    if topp_rows is not None:
        _need(topp_rows, "topp_rows", torch.int32); _need(topp_p, "topp_p", torch.float32)
        n_p = topp_rows.numel()
        assert topp_p.numel() == n_p
    if n_k == 0 and n_p == 0:
        return
    _check(library().rl_sample_candidates(logits.data_ptr(), logits.shape[1], _ptr(topk_rows), _ptr(topk_k), _ptr(topk_p),
                                          n_k, _ptr(topp_rows), _ptr(topp_p), n_p,
                                          temperature.data_ptr(), uniform.data_ptr(), min_p.data_ptr(), out.data_ptr(),
                                          _stream()), "rl_sample_candidates")
    _count((1 if n_k else 0) + (1 if n_p else 0))
