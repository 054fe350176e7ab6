"""ctypes access to the sm_100a kernel library (``lib/libortb200_kernels.so``).

The session executor reaches the same symbols from C++; this module exists so
that tests, micro-benchmarks and Python-side tools can drive each kernel in
isolation with torch tensors.  Loading fails loudly when the library is
missing: there is no eager fallback behind these wrappers.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None

F16, BF16, F32 = 0, 1, 2
ACT = {"none": 0, "gelu": 1, "fastgelu": 2, "relu": 3, "silu": 4, "swiglu": 5, "quickgelu": 6}


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libortb200_kernels.so")


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run `python -m onnxruntime_b200.build` first")
        _LIB = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
        _LIB.ortb200_gemm.restype = ctypes.c_int
        _LIB.ortb200_gemm_workspace_bytes.restype = ctypes.c_int64
    return _LIB


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return F16
    if dt == torch.bfloat16:
        return BF16
    if dt == torch.float32:
        return F32
    raise TypeError(f"unsupported dtype {dt}")


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p), ("w", ctypes.c_void_p), ("out", ctypes.c_void_p), ("bias", ctypes.c_void_p),
        ("residual", ctypes.c_void_p), ("ldo", ctypes.c_int64), ("ldr", ctypes.c_int64),
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("w_rows", ctypes.c_int),
        ("dual_offset", ctypes.c_int), ("dtype", ctypes.c_int), ("act", ctypes.c_int), ("alpha", ctypes.c_float),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64), ("status", ctypes.c_void_p),
        ("force_splits", ctypes.c_int), ("force_bn", ctypes.c_int), ("use_pdl", ctypes.c_int),
    ]


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_WS = {}


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised split-K scratch, grown on demand, one per device."""
    key = (device.index if device.index is not None else torch.cuda.current_device())
    cur = _WS.get(key)
    if cur is None or cur.numel() < nbytes:
        cur = torch.zeros(max(nbytes, 32 << 20), dtype=torch.uint8, device=device)
        _WS[key] = cur
    return cur


def gemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, act: str = "none", alpha: float = 1.0,
         out: Optional[torch.Tensor] = None, n: Optional[int] = None, dual_offset: int = 0,
         force_splits: int = 0, force_bn: int = 0, status: Optional[torch.Tensor] = None,
         use_pdl: bool = False) -> torch.Tensor:
    """out[M, N] = act(alpha * x[M, K] @ w[N, K].T + bias) + residual  (tcgen05 kernel)."""
    assert x.is_cuda and w.is_cuda and x.dtype == w.dtype and x.dim() == 2 and w.dim() == 2
    assert x.is_contiguous() and w.is_contiguous()
    M, K = x.shape
    w_rows = w.shape[0]
    if n is None:
        n = w_rows // 2 if act == "swiglu" else w_rows
        if act == "swiglu" and dual_offset == 0:
            dual_offset = n
    if out is None:
        out = torch.empty((M, n), dtype=x.dtype, device=x.device)
    nbytes = lib().ortb200_gemm_workspace_bytes(M, n, K, ACT[act])
    ws = workspace(x.device, nbytes)
    a = GemmArgs(_ptr(x), _ptr(w), _ptr(out), _ptr(bias), _ptr(residual), out.stride(0),
                 residual.stride(0) if residual is not None else 0, M, n, K, w_rows, dual_offset,
                 dtype_code(x.dtype), ACT[act], alpha, _ptr(ws), ws.numel(), _ptr(status), force_splits, force_bn,
                 1 if use_pdl else 0)
    rc = lib().ortb200_gemm(ctypes.byref(a), ctypes.c_void_p(stream_ptr()))
    if rc != 0:
        raise RuntimeError(f"ortb200_gemm rejected its arguments (code {rc})")
    return out


def gemm_last_config():
    bn, sp, st = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib().ortb200_gemm_last_config(ctypes.byref(bn), ctypes.byref(sp), ctypes.byref(st))
    return bn.value, sp.value, st.value
