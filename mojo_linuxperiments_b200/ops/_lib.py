"""ctypes binding of the sm_100a kernel library (``_lib/libb200_kernels.so``).

The library is built in-tree by ``mojo_linuxperiments_b200._build``.  On a machine with a GPU a missing
library is an error (there is no PyTorch fallback for the hot ops); on a CPU-only machine importing this
module works and ``lib()`` raises only when a kernel is actually requested.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_void_p, c_size_t, c_float, c_longlong, c_uint64
from functools import lru_cache
from pathlib import Path

import torch

import os


def _variant() -> str:
    """Which build of the kernel library this process loads: B200RT_KERNELS=trace (in-kernel time stamps) or debug
    (range-checked peer / scratch accesses); B200RT_DEBUG=1 also selects the debug build.  Default: production."""
    v = os.environ.get("B200RT_KERNELS", "").strip().lower()
    if v in ("trace", "debug"):
        return v
    return "debug" if os.environ.get("B200RT_DEBUG", "0") not in ("", "0") else ""


_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / (
    "libb200_kernels.so" if not _variant() else f"libb200_kernels_{_variant()}.so")


class KernelError(RuntimeError):
    pass


@lru_cache(maxsize=None)
def lib() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        raise KernelError(
            f"{_LIB_PATH} is missing: run `python -m mojo_linuxperiments_b200._build --all` (needs nvcc, no GPU)")
    L = ctypes.CDLL(str(_LIB_PATH))
    for name in dir(_Sig):
        if name.startswith("b200_"):
            restype, argtypes = getattr(_Sig, name)
            try:
                fn = getattr(L, name)
            except AttributeError as e:  # stale library
                raise KernelError(f"{name} not found in {_LIB_PATH}; rebuild the kernel library") from e
            fn.restype = restype
            fn.argtypes = argtypes
    return L


P = c_void_p
I = c_int
LL = c_longlong
F = c_float


class _Sig:
    b200_w8a8_gemm_ws_bytes = (c_size_t, [I, I, I, I])
    b200_w8a8_gemm = (I, [P, P, P, P, P, P, I, I, I, I, I, P, c_size_t, P, I, P, I, I, P])
    b200_w8a8_gemm_decode = (I, [P, P, P, P, P, P, I, I, I, I, I, P, I, I, P])
    b200_w8a8_gemm_decode_resident_clusters = (I, [I, I])
    b200_w8a8_gemm_decode_p = (I, [P, P, P, P, P, I, I, I, I, I, P, I, P])
    b200_w8a8_gemm_decode_ar_p = (I, [P, P, P, P, P, I, I, I, I, P, I, P, P, P, I, I, c_size_t, c_size_t, P, I, I, c_size_t, c_size_t, c_size_t, I, c_size_t, c_size_t, c_size_t, P])
    b200_peer_allreduce = (I, [P, P, P, I, I, c_size_t, c_size_t, P, P, c_size_t, I, I, P, P, I, I, I, P])
    b200_peer_argmax = (I, [P, P, I, I, c_size_t, P, P, I, I, P, P, P, I, P])
    b200_w8a8_gemm_ag = (I, [P, P, P, P, P, I, I, I, I, I, P, P, I, I, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, I, I, P, P, I, I, P, I, I, P])
    b200_w8a8_gemm_rs = (I, [P, P, P, P, P, P, I, I, I, I, I, I, P, I, I, c_size_t, c_size_t, c_size_t, I, P, I, P, I, I, P])
    b200_ep_dispatch = (I, [P, P, P, P, I, I, I, I, I, P, I, I] + [c_size_t] * 10 + [I, P, P, P, I, P])
    b200_ep_wait = (I, [P, I, I] + [c_size_t] * 5 + [I, I, I, I, P, P, P, P, I, P])
    b200_ep_gather = (I, [P] + [c_size_t] * 4 + [P, I, P, P, I, P, P, P])
    b200_ep_combine_scatter = (I, [P, LL, P, P, I, I, I, I, P, I, I, c_size_t, c_size_t, c_size_t, I, P, P, I, P, I, P])
    b200_ep_combine_reduce = (I, [P, I, I, I, I, I, P, I, I, c_size_t, c_size_t, c_size_t, I, P, P, LL, P, I, I, P])
    b200_ag_sync = (I, [P, I, I, c_size_t, c_size_t, I, I, I, P, I, I, P, I, P])
    b200_w8a8_gemm_decode_ar = (I, [P, P, P, P, P, P, I, I, I, I, P, I, P, P, P, I, I, c_size_t, c_size_t, P, I, I, c_size_t, c_size_t, c_size_t, I, c_size_t, c_size_t, c_size_t, P])
    b200_where_am_i = (I, [P, I, I, P])
    b200_debug_compiled = (I, [])
    b200_debug_set_heap_extent = (I, [c_size_t])
    b200_trace_compiled = (I, [])
    b200_trace_set = (I, [P, ctypes.c_uint])
    b200_fill_uniform_reduce = (I, [P, c_uint64, c_uint64, c_uint64, P, I, P, P, P])
    b200_w8a8_gemm_decode_grouped = (I, [P, P, P, P, P, I, I, I, I, I, I, P, P, P, I, P])
    b200_w8a8_gemm_grouped = (I, [P, P, P, P, P, I, I, I, I, I, P, P, I, P, I, P])
    b200_router_topk = (I, [P, LL, I, I, I, I, P, P, P])
    b200_moe_align = (I, [P, I, I, I, I, P, P, P, P, P, P, P])
    b200_moe_gather = (I, [P, P, I, P, P, I, P, P, P])
    b200_moe_combine = (I, [P, LL, P, P, I, I, I, P, LL, P])
    b200_act_quant = (I, [P, LL, P, LL, P, F, P, LL, P, P, LL, I, I, I, P])
    b200_rope_kv_write = (I, [P, LL, P, P, P, P, P, P, F, P, P, P, P, P, I, I, I, I, I, I, I, P, P])
    b200_embed_gather = (I, [P, P, P, I, I, I, P])
    b200_argmax_rows = (I, [P, LL, I, I, I, I, P, P, P])
    b200_argmax_merge = (I, [P, P, I, I, P, P])
    b200_attn_decode_scratch_floats = (c_size_t, [I, I, I])
    b200_attn_decode = (I, [P, P, P, P, P, P, P, I, I, I, I, I, I, F, P, P])
    b200_attn_decode_noalloc = (I, [P, P, P, P, P, I, I, I, I, I, I, F, P])
    b200_attn_decode_tma = (I, [P, P, I, P, P, P, P, P, I, I, I, I, I, I, F, P, P])
    b200_attn_decode_tc = (I, [P, P, I, P, P, P, P, P, I, I, I, I, I, I, F, P, P])
    b200_attn_decode_tc_min_splits = (I, [I])
    b200_attn_decode_fused = (I, [P, LL, P, P, P, I, P, P, F, P, I, P, P, P, P, LL, P, P, P, P, P, P, I, I, I, I, I, I, F, P, P, c_uint64, P])
    b200_attn_decode_tcp = (I, [P, P, I, P, P, P, P, P, I, I, I, I, I, I, F, P, I, P])
    b200_attn_prefill = (I, [P, LL, P, LL, P, LL, P, P, I, I, I, I, I, F, P, P])
    b200_attn_prefill_split = (I, [P, LL, P, LL, P, LL, P, P, I, I, I, I, I, F, I, P, P, P])
    b200_attn_prefill_split_scratch_floats = (c_size_t, [I, I, I, I])


class QuantProlog(ctypes.Structure):
    """``b200_quant_prolog`` of csrc/kernels/api.h: the activation prologue a decode GEMM launch carries itself."""
    _fields_ = [("mode", c_int), ("x", c_void_p), ("ldx", c_longlong), ("residual", c_void_p), ("ldr", c_longlong),
                ("gamma", c_void_p), ("eps", c_float), ("q", c_void_p), ("scale", c_void_p), ("flags", c_void_p),
                ("step", c_void_p), ("residual_out", c_void_p), ("ldro", c_longlong), ("allow_inline", c_int)]


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = [0]     # kernels of this library launched (or captured into a CUDA graph) by this process


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")
    LAUNCHES[0] += 1


@lru_cache(maxsize=None)
def num_sms(device_index: int) -> int:
    return torch.cuda.get_device_properties(device_index).multi_processor_count
