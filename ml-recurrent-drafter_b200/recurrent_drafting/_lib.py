"""ctypes binding of libredrafter_b200.so (the C ABI declared in include/redrafter_b200.h).

There is no fallback: if the shared library is missing or a CUDA device is not available the
operators raise.  Build it with `python ml-recurrent-drafter_b200/build.py`.
"""

import ctypes
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libredrafter_b200.so")

F32, BF16 = 0, 1
EPI_NONE, EPI_BIAS, EPI_BIAS_SILU, EPI_BIAS_SILU_RES, EPI_RES, EPI_SWIGLU = range(6)
ATTN_CAUSAL, ATTN_TREE, ATTN_DENSE = 0, 1, 2
TOPK_MAX_KEPT = 64
STATIC_SCRATCH_BYTES = 16 << 20
MAX_BEAM_WIDTH = 64
MAX_BEAM_LENGTH = 8

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

# name -> (restype, argtypes); one entry per function declared in include/redrafter_b200.h
SIGNATURES = {
    "rd_strerror": (ctypes.c_char_p, [_I]),
    "rd_last_cuda_error": (_I, []),
    "rd_abi_version": (_I, []),
    "rd_tree_pack": (_I, [_P, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P]),
    "rd_tree_pack_reference_layout": (_I, [_I, _I, _I, _P, _P, _P, _P, _P, _I, _P, _I, _P, _P, _P, _P, _P, _P]),
    "rd_drafter_prepare": (_I, [_I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "rd_vocab_topk": (_I, [_I, _P, _L, _I, _P, _I, _I, _F, _I, _F, _P, _P, _P, _P, _P]),
    "rd_beam_select": (_I, [_I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "rd_drafter_dense_log_probs": (_I, [_I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P]),
    "rd_gemm": (_I, [_I, _I, _P, _L, _P, _L, _P, _L, _P, _P, _L, _I, _P, _I, _I, _I, _P]),
    "rd_gemm_plan_create": (_P, [_P, _L, _I, _P, _L, _I, _I]),
    "rd_gemm_plan_destroy": (None, [_P]),
    "rd_gemm_bf16_tc": (_I, [_P, _I, _P, _L, _P, _P, _L, _P, _I, _P, _P]),
    "rd_gemm_bf16_tc_qkv_rope": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P]),
    "rd_gemm_bf16_tc_res_norm": (_I, [_P, _P, _L, _P, _L, _P, _P, _P, _L, _P, _L, _P, _P]),
    "rd_gemm_bf16_tc_swiglu_normed": (_I, [_P, _P, _L, _P, _P, _L, _I, _I, _F, _P, _P]),
    "rd_gemm_bf16_tc_qkv_rope_normed": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _L, _I, _I, _F,
                                              _P, _P]),
    "rd_gemm_argmax_workspace_bytes": (_L, [_I, _I]),
    "rd_gemm_bf16_tc_argmax": (_I, [_P, _P, _P, _L, _P, _P, _P, _P]),
    "rd_gemm_bf16_tc_slicemax": (_I, [_P, _I, _P, _L, _P, _P, _L, _P, _P]),
    "rd_vocab_topk_sliced": (_I, [_I, _P, _L, _I, _P, _I, _I, _F, _I, _F, _P, _L, _P, _P, _P, _P, _P]),
    "rd_embed_gather": (_I, [_I, _P, _P, _P, _I, _P, _I, _P]),
    "rd_rmsnorm": (_I, [_I, _P, _P, _P, _I, _P, _I, _F, _P]),
    "rd_rope_kv_write": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P, _I, _I, _I, _I, _P]),
    "rd_attention": (_I, [_I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _L, _L, _P]),
    "rd_attention_plan_create": (_P, [_P, _I, _P, _P, _I, _I, _I, _I, _I]),
    "rd_attention_plan_destroy": (None, [_P]),
    "rd_attention_tc": (_I, [_P, _P, _P, _P, _P, _I, _I, _P, _I, _P, _P]),
    "rd_attention_split_workspace_bytes": (_L, [_I, _I, _I]),
    "rd_attention_tc_split": (_I, [_P, _P, _P, _P, _P, _I, _I, _P, _I, _I, _P, _L, _P, _P]),
    "rd_argmax_rows": (_I, [_P, _L, _I, _P, _I, _P, _P, _P]),
    "rd_accept_commit_greedy": (_I, [_I, _P, _I, _I, _I, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "rd_commit_reference_slots": (_I, [_I, _I, _I, _P, _P, _P, _I, _I, _P, _P]),
    "rd_accept_commit_sample": (
        _I,
        [_I, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P],
    ),
    "rd_sample_from_sparse": (_I, [_P, _P, _P, _I, _P, _P, _P]),
    "rd_emit_tokens": (_I, [_P, _I, _P, _P, _P, _L, _I, _I, _P, _P]),
    "rd_cache_unpack": (_I, [_I, _P, _I, _I, _I, _I, _I, _I, _P, _I, _P, _P]),
    "rd_cache_unpack_static": (_I, [_I, _P, _I, _I, _I, _I, _I, _I, _P, _I, _P]),
}

_lib = None


class RedrafterError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Loads the shared library (once) and declares every entry point."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RedrafterError(
                f"{LIB_PATH} not found: build the CUDA library first (python ml-recurrent-drafter_b200/build.py)"
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"unsupported dtype {dtype}: the kernels compute in float32 or bfloat16")


def ptr(t: Optional[torch.Tensor]):
    """Device pointer of a tensor (None -> NULL).  The tensor must live on a CUDA device."""
    if t is None:
        return None
    if not t.is_cuda:
        raise RedrafterError("operator called with a CPU tensor: this library has no CPU path")
    return ctypes.c_void_p(t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(rc: int, what: str) -> None:
    if rc != 0:
        lib = load()
        msg = lib.rd_strerror(rc).decode()
        extra = f" (cudaError {lib.rd_last_cuda_error()})" if rc == -4 else ""
        raise RedrafterError(f"{what}: {msg}{extra}")


# kernels enqueued per entry point where that is not one; `launches` counts the kernels this process has enqueued
# through call() (a replayed CUDA graph adds the number of kernels captured in it, see count_replay)
KERNELS_PER_CALL = {"rd_tree_pack": 2, "rd_gemm_bf16_tc_argmax": 2, "rd_attention_tc_split": 2, "rd_cache_unpack": 2,
                    "rd_cache_unpack_static": 2}
launches = 0


def call(name: str, *args) -> None:
    global launches
    launches += KERNELS_PER_CALL.get(name, 1)
    check(getattr(load(), name)(*args), name)


def count_replay(n_kernels: int) -> None:
    global launches
    launches += n_kernels


def ptr_array(tensors):
    """Host array of device pointers (for the `*_host` parameters)."""
    arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    return arr
