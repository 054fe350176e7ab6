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
        ("world", ctypes.c_int), ("rank", ctypes.c_int), ("peers", ctypes.c_void_p * 8), ("symm_bytes", ctypes.c_int64),
        ("in_dtype", ctypes.c_int), ("rms_eps", ctypes.c_float), ("force_tile_rows", ctypes.c_int), ("mc_ptr", ctypes.c_void_p),
        ("alpha_dev", ctypes.c_void_p),
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
         use_pdl: bool = False, peers=None, rank: int = 0, symm_bytes: int = 0,
         out_dtype: Optional[torch.dtype] = None, rms_eps: float = 0.0, force_tile_rows: int = 0,
         q4: bool = False, mc_ptr: int = 0) -> torch.Tensor:
    """out[M, N] = act(alpha * x[M, K] @ w[N, K].T + bias) + residual  (tcgen05 kernel).
    x / w of dtype float8_e4m3fn use the 8-bit tensor-core mode; out_dtype (fp16 / bf16) is then required."""
    assert x.is_cuda and w.is_cuda and (x.dtype == w.dtype or q4) and x.dim() == 2
    if q4:  # w is the tile-blob array from nbits_build_blobs: [tiles, K / 64, 4864] bytes; n must be given
        assert n is not None
        w = w.reshape(w.shape[0] * 128, -1)
    assert x.is_contiguous() and w.is_contiguous()
    M, K = x.shape
    w_rows = w.shape[0]
    if n is None:
        n = w_rows // 2 if act == "swiglu" else w_rows
        if act == "swiglu" and dual_offset == 0:
            dual_offset = n
    fp8 = x.dtype == torch.float8_e4m3fn
    odt = out_dtype if out_dtype is not None else (out.dtype if out is not None else x.dtype)
    if out is None:
        out = torch.empty((M, n), dtype=odt, device=x.device)
    nbytes = lib().ortb200_gemm_workspace_bytes(M, n, K, ACT[act])
    ws = workspace(x.device, nbytes)
    a = GemmArgs(_ptr(x), _ptr(w), _ptr(out), _ptr(bias), _ptr(residual), out.stride(0),
                 residual.stride(0) if residual is not None else 0, M, n, K, w_rows, dual_offset,
                 dtype_code(odt), ACT[act], alpha, _ptr(ws), ws.numel(), _ptr(status), force_splits, force_bn,
                 1 if use_pdl else 0, len(peers) if peers else 1, rank,
                 (ctypes.c_void_p * 8)(*(list(peers) + [None] * (8 - len(peers)))) if peers else (ctypes.c_void_p * 8)(),
                 symm_bytes, 4 if q4 else (3 if fp8 else 0), rms_eps, force_tile_rows, mc_ptr or None, None)
    rc = lib().ortb200_gemm(ctypes.byref(a), ctypes.c_void_p(stream_ptr()))
    if rc != 0:
        raise RuntimeError(f"ortb200_gemm rejected its arguments (code {rc})")
    return out


class ChainStage(ctypes.Structure):
    _fields_ = [("w", ctypes.c_void_p), ("out", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p),
                ("ldr", ctypes.c_int64), ("N", ctypes.c_int), ("K", ctypes.c_int), ("w_rows", ctypes.c_int),
                ("dual_offset", ctypes.c_int), ("act", ctypes.c_int), ("rms_eps", ctypes.c_float),
                ("residual_stage", ctypes.c_int), ("all_reduce", ctypes.c_int)]


class GemmChainArgs(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("M", ctypes.c_int), ("num_stages", ctypes.c_int), ("dtype", ctypes.c_int),
                ("stage", ChainStage * 4), ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64),
                ("status", ctypes.c_void_p), ("use_pdl", ctypes.c_int), ("prefetch_items", ctypes.c_int),
                ("max_ctas", ctypes.c_int), ("world", ctypes.c_int), ("rank", ctypes.c_int), ("peers", ctypes.c_void_p * 8),
                ("symm_bytes", ctypes.c_int64), ("trace", ctypes.c_void_p)]


_CHAIN_WS = {}


def gemm_chain(x: torch.Tensor, stages, status: Optional[torch.Tensor] = None, use_pdl: bool = False, prefetch_items: int = 0,
               max_ctas: int = 0, peers=None, rank: int = 0, symm_bytes: int = 0, trace: Optional[torch.Tensor] = None):
    """Runs up to four dependent decode-shaped GEMMs (x: [M <= 16, K0]) as one persistent launch.

    ``stages`` is a list of dicts: ``w`` [rows, K] (for ``act="swiglu"`` the gate rows followed by the up rows), optional
    ``bias`` [N], ``residual`` ([M, N] tensor, or an int = index of an earlier stage whose output is added), ``act``,
    ``rms_eps`` (the caller has folded gamma into ``w``), ``all_reduce``.  Returns the list of stage outputs."""
    assert x.is_cuda and x.dim() == 2 and x.is_contiguous() and 1 <= len(stages) <= 4
    M = x.shape[0]
    lib().ortb200_gemm_chain_workspace_bytes.restype = ctypes.c_int64
    need = lib().ortb200_gemm_chain_workspace_bytes()
    key = x.device.index if x.device.index is not None else torch.cuda.current_device()
    ws = _CHAIN_WS.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=x.device)
        _CHAIN_WS[key] = ws
    a = GemmChainArgs()
    a.x, a.M, a.num_stages, a.dtype = _ptr(x), M, len(stages), dtype_code(x.dtype)
    outs, keep = [], []
    for i, st in enumerate(stages):
        w = st["w"]
        assert w.is_contiguous() and w.dtype == x.dtype
        act = st.get("act", "none")
        n = st.get("n", w.shape[0] // 2 if act == "swiglu" else w.shape[0])
        out = torch.empty((M, n), dtype=x.dtype, device=x.device)
        outs.append(out)
        res = st.get("residual")
        c = a.stage[i]
        c.w, c.out, c.bias = _ptr(w), _ptr(out), _ptr(st.get("bias"))
        c.N, c.K, c.w_rows = n, w.shape[1], w.shape[0]
        c.dual_offset = st.get("dual_offset", n) if act == "swiglu" else 0
        c.act, c.rms_eps = ACT[act], float(st.get("rms_eps", 0.0))
        c.all_reduce = 1 if st.get("all_reduce") else 0
        if isinstance(res, int):
            c.residual_stage, c.residual, c.ldr = res, None, 0
        else:
            c.residual_stage, c.residual, c.ldr = -1, _ptr(res), (res.stride(0) if res is not None else 0)
            keep.append(res)
    a.workspace, a.workspace_bytes, a.status = _ptr(ws), ws.numel(), _ptr(status)
    a.use_pdl, a.prefetch_items, a.max_ctas = (1 if use_pdl else 0), prefetch_items, max_ctas
    a.world, a.rank, a.symm_bytes = (len(peers) if peers else 1), rank, symm_bytes
    a.trace = _ptr(trace)
    if peers:
        for i, pp in enumerate(peers):
            a.peers[i] = pp
    _check(lib().ortb200_gemm_chain(ctypes.byref(a), ctypes.c_void_p(stream_ptr())), "ortb200_gemm_chain")
    return outs


def gemm_last_config():
    bn, sp, st = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib().ortb200_gemm_last_config(ctypes.byref(bn), ctypes.byref(sp), ctypes.byref(st))
    return bn.value, sp.value, st.value


# ---------------------------------------------------------------------------- norm
class NormArgs(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("skip", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("gamma", ctypes.c_void_p),
                ("beta", ctypes.c_void_p), ("out", ctypes.c_void_p), ("sum_out", ctypes.c_void_p), ("rows", ctypes.c_int64),
                ("hidden", ctypes.c_int), ("epsilon", ctypes.c_float), ("simplified", ctypes.c_int), ("dtype", ctypes.c_int)]


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} rejected its arguments (code {rc})")


def norm(x, gamma, beta=None, skip=None, bias=None, eps=1e-5, simplified=False, want_sum=False):
    x = x.contiguous()
    H = x.shape[-1]
    out = torch.empty_like(x)
    s = torch.empty_like(x) if want_sum else None
    a = NormArgs(_ptr(x), _ptr(skip), _ptr(bias), _ptr(gamma), _ptr(beta), _ptr(out), _ptr(s), x.numel() // H, H, eps,
                 1 if simplified else 0, dtype_code(x.dtype))
    _check(lib().ortb200_norm(ctypes.byref(a), ctypes.c_void_p(stream_ptr())), "ortb200_norm")
    return (out, s) if want_sum else out


# ----------------------------------------------------------------------------- GQA
class GqaPrepArgs(ctypes.Structure):
    _fields_ = [("qkv", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("q_out", ctypes.c_void_p),
                ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p), ("seqlens_k", ctypes.c_void_p),
                ("cos_cache", ctypes.c_void_p), ("sin_cache", ctypes.c_void_p), ("position_ids", ctypes.c_void_p),
                ("B", ctypes.c_int), ("S", ctypes.c_int), ("N", ctypes.c_int), ("Nk", ctypes.c_int), ("H", ctypes.c_int),
                ("Smax", ctypes.c_int), ("rot_dim", ctypes.c_int), ("interleaved", ctypes.c_int),
                ("first_prompt", ctypes.c_int), ("do_rotary", ctypes.c_int), ("dtype", ctypes.c_int), ("use_pdl", ctypes.c_int),
                ("cos_rows", ctypes.c_int)]


def gqa_prep(qkv, k_cache, v_cache, seqlens_k, cos, sin, N, Nk, H, first_prompt, interleaved=False, position_ids=None):
    B, S = qkv.shape[0], qkv.shape[1]
    q_out = torch.empty(B, S, N, H, dtype=qkv.dtype, device=qkv.device)
    a = GqaPrepArgs(_ptr(qkv), None, None, _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(seqlens_k), _ptr(cos), _ptr(sin),
                    _ptr(position_ids), B, S, N, Nk, H, k_cache.shape[2], 0 if cos is None else cos.shape[1] * 2,
                    1 if interleaved else 0, 1 if first_prompt else 0, 0 if cos is None else 1, dtype_code(qkv.dtype), 0,
                    0 if cos is None else cos.shape[0])
    _check(lib().ortb200_gqa_prep(ctypes.byref(a), ctypes.c_void_p(stream_ptr())), "ortb200_gqa_prep")
    return q_out


class GqaDecodeArgs(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("seqlens_k", ctypes.c_void_p), ("head_sink", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64), ("B", ctypes.c_int), ("N", ctypes.c_int),
                ("Nk", ctypes.c_int), ("H", ctypes.c_int), ("Smax", ctypes.c_int), ("splits", ctypes.c_int),
                ("window", ctypes.c_int), ("scale", ctypes.c_float), ("softcap", ctypes.c_float), ("dtype", ctypes.c_int),
                ("use_pdl", ctypes.c_int), ("status", ctypes.c_void_p), ("block_table", ctypes.c_void_p),
                ("block_size", ctypes.c_int), ("max_blocks", ctypes.c_int), ("qkv", ctypes.c_void_p), ("cos_cache", ctypes.c_void_p),
                ("sin_cache", ctypes.c_void_p), ("do_rotary", ctypes.c_int), ("rotary_interleaved", ctypes.c_int),
                ("num_blocks", ctypes.c_int), ("algo", ctypes.c_int), ("prefetch", ctypes.c_void_p), ("prefetch_bytes", ctypes.c_int64),
                ("cos_rows", ctypes.c_int)]


_ATTN_WS = {}


def gqa_decode(q, k_cache, v_cache, seqlens_k, splits=0, window=-1, scale=0.0, softcap=0.0, head_sink=None, block_table=None,
               qkv=None, num_heads=0, cos=None, sin=None, interleaved=False, algo=0, prefetch=None):
    """Dense cache [B,Nk,Smax,H]; or, with block_table [B,max_blocks] int32, a paged cache [num_blocks,block_size,Nk,H].
    With ``qkv`` (packed [B,(N+2Nk)H], ``num_heads`` = N) the kernel also rotates q / k and appends k / v itself.
    ``algo``: 0 = pick, 1 = CUDA-core split-KV kernel, 2 = tcgen05 kernel (head size 128, 16-bit types)."""
    if qkv is not None:
        H = k_cache.shape[3]
        B, N = qkv.shape[0], num_heads
        q = qkv
    else:
        B, N, H = q.shape
    if block_table is None:
        Nk, Smax = k_cache.shape[1], k_cache.shape[2]
        block_size = max_blocks = num_blocks = 0
    else:
        num_blocks = k_cache.shape[0]
        Nk, block_size, max_blocks = k_cache.shape[2], k_cache.shape[1], block_table.shape[1]
        Smax = block_size * max_blocks
    out = torch.empty(B, N * H, dtype=q.dtype, device=q.device)
    lib().ortb200_gqa_decode_workspace_bytes.restype = ctypes.c_int64
    need = lib().ortb200_gqa_decode_workspace_bytes(B, N, H)
    key = q.device.index
    ws = _ATTN_WS.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=q.device)
        _ATTN_WS[key] = ws
    a = GqaDecodeArgs(None if qkv is not None else _ptr(q.contiguous()), _ptr(k_cache), _ptr(v_cache), _ptr(seqlens_k), _ptr(head_sink), _ptr(out), _ptr(ws),
                      ws.numel(), B, N, Nk, H, Smax, splits, window, scale, softcap, dtype_code(q.dtype), 0, None,
                      _ptr(block_table), block_size, max_blocks, _ptr(qkv), _ptr(cos), _ptr(sin), 0 if cos is None else 1,
                      1 if interleaved else 0, num_blocks, algo, _ptr(prefetch),
                      prefetch.numel() * prefetch.element_size() if prefetch is not None else 0,
                      0 if cos is None else cos.shape[0])
    _check(lib().ortb200_gqa_decode(ctypes.byref(a), ctypes.c_void_p(stream_ptr())), "ortb200_gqa_decode")
    return out


class AttnPrefillArgs(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("seqlens_k", ctypes.c_void_p),
                ("head_sink", ctypes.c_void_p), ("out", ctypes.c_void_p), ("B", ctypes.c_int), ("S", ctypes.c_int),
                ("N", ctypes.c_int), ("Nk", ctypes.c_int), ("H", ctypes.c_int), ("kv_len", ctypes.c_int),
                ("q_strides", ctypes.c_int64 * 3), ("o_strides", ctypes.c_int64 * 3), ("kv_strides", ctypes.c_int64 * 3),
                ("first_prompt", ctypes.c_int), ("causal", ctypes.c_int), ("window", ctypes.c_int), ("scale", ctypes.c_float),
                ("softcap", ctypes.c_float), ("dtype", ctypes.c_int), ("status", ctypes.c_void_p), ("key_mask", ctypes.c_void_p)]


def attn_prefill(q, k, v, seqlens_k=None, first_prompt=True, causal=True, window=-1, scale=0.0, softcap=0.0,
                 kv_layout="bnsh", status=None, key_mask=None):
    """q [B,S,N,H]; k/v [B,Nk,T,H] ("bnsh") or [B,T,Nk,H] ("bsnh"); key_mask int32 [B,T] (0 = padding).  Returns [B,S,N,H]."""
    B, S, N, H = q.shape
    if kv_layout == "bnsh":
        Nk, T = k.shape[1], k.shape[2]
        kvs = (k.stride(0), k.stride(1), k.stride(2))
    else:
        T, Nk = k.shape[1], k.shape[2]
        kvs = (k.stride(0), k.stride(2), k.stride(1))
    out = torch.empty_like(q)
    a = AttnPrefillArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(seqlens_k), None, _ptr(out), B, S, N, Nk, H, T,
                        (ctypes.c_int64 * 3)(q.stride(0), q.stride(1), q.stride(2)),
                        (ctypes.c_int64 * 3)(out.stride(0), out.stride(1), out.stride(2)), (ctypes.c_int64 * 3)(*kvs),
                        1 if first_prompt else 0, 1 if causal else 0, window, scale, softcap, dtype_code(q.dtype), _ptr(status),
                        _ptr(key_mask))
    _check(lib().ortb200_attn_prefill(ctypes.byref(a), ctypes.c_void_p(stream_ptr())), "ortb200_attn_prefill")
    return out


class PagedPrepArgs(ctypes.Structure):
    _fields_ = [("qkv", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("q_out", ctypes.c_void_p),
                ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p), ("cu_seqlens", ctypes.c_void_p),
                ("past_seqlens", ctypes.c_void_p), ("block_table", ctypes.c_void_p), ("slot_mapping", ctypes.c_void_p),
                ("cos_cache", ctypes.c_void_p), ("sin_cache", ctypes.c_void_p), ("T", ctypes.c_int), ("B", ctypes.c_int),
                ("N", ctypes.c_int), ("Nk", ctypes.c_int), ("H", ctypes.c_int), ("block_size", ctypes.c_int),
                ("max_blocks", ctypes.c_int), ("num_blocks", ctypes.c_int), ("rot_dim", ctypes.c_int), ("interleaved", ctypes.c_int),
                ("do_rotary", ctypes.c_int), ("dtype", ctypes.c_int), ("status", ctypes.c_void_p), ("cos_rows", ctypes.c_int)]


def paged_prep(qkv, k_cache, v_cache, cu_seqlens, past_seqlens, block_table, N, Nk, cos=None, sin=None, interleaved=False,
               slot_mapping=None, status=None):
    """Packed qkv [T,(N+2Nk)H]; caches [num_blocks,block_size,Nk,H] updated in place.  Returns rotated q [T,N,H]."""
    T = qkv.shape[0]
    H = k_cache.shape[3]
    q_out = torch.empty(T, N, H, dtype=qkv.dtype, device=qkv.device)
    a = PagedPrepArgs(_ptr(qkv.contiguous()), None, None, _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(cu_seqlens),
                      _ptr(past_seqlens), _ptr(block_table), _ptr(slot_mapping), _ptr(cos), _ptr(sin), T, past_seqlens.numel(), N, Nk, H,
                      k_cache.shape[1], block_table.shape[1], k_cache.shape[0], 0 if cos is None else cos.shape[1] * 2,
                      1 if interleaved else 0, 0 if cos is None else 1, dtype_code(qkv.dtype), _ptr(status),
                      0 if cos is None else cos.shape[0])
    _check(lib().ortb200_paged_prep(ctypes.byref(a), ctypes.c_void_p(stream_ptr())), "ortb200_paged_prep")
    return q_out


def nbits_prepack(B):
    """MatMulNBits 4-bit weights [N, n_blocks, block/2] -> [N, K/2] bytes in the nibble order the GEMM expands."""
    B = B.contiguous()
    out = torch.empty(B.shape[0], B.numel() // B.shape[0], dtype=torch.uint8, device=B.device)
    _check(lib().ortb200_nbits_prepack(ctypes.c_void_p(_ptr(B)), ctypes.c_void_p(_ptr(out)), ctypes.c_int64(B.numel()),
                                       ctypes.c_void_p(stream_ptr())), "ortb200_nbits_prepack")
    return out


def nbits_build_blobs(B, scales, zp_bytes, N, K, block_size=32):
    """MatMulNBits 4-bit weights -> the [tiles, K / 64, 4864] byte array ``gemm(..., q4=True)`` consumes."""
    from .. import _core
    return _core.nbits_build_blobs(B, scales, zp_bytes, N, K, block_size)


def nbits_dequant(B, scales, zero_points, N, K, bits=4, block_size=32):
    """MatMulNBits weights -> [N, K] rows of scales.dtype."""
    out = torch.empty(N, K, dtype=scales.dtype, device=scales.device)
    packed = zero_points is not None and zero_points.dtype == torch.uint8
    _check(lib().ortb200_nbits_dequant(ctypes.c_void_p(_ptr(B.contiguous())), ctypes.c_void_p(_ptr(scales.contiguous())),
                                       ctypes.c_void_p(_ptr(zero_points)), 1 if packed else 0, ctypes.c_void_p(_ptr(out)),
                                       ctypes.c_int64(N), K, bits, block_size, ctypes.c_int64(K), dtype_code(scales.dtype),
                                       ctypes.c_void_p(stream_ptr())), "ortb200_nbits_dequant")
    return out


class SymmCollectiveArgs(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int), ("inp", ctypes.c_void_p), ("out", ctypes.c_void_p), ("rows", ctypes.c_int64),
                ("row_bytes", ctypes.c_int64), ("dtype", ctypes.c_int), ("world", ctypes.c_int), ("rank", ctypes.c_int),
                ("peers", ctypes.c_void_p * 8), ("symm_bytes", ctypes.c_int64), ("status", ctypes.c_void_p), ("use_pdl", ctypes.c_int),
                ("mc_ptr", ctypes.c_void_p)]


def symm_collective(op, x, peers, rank, symm_bytes, axis=0, status=None, mc_ptr=0):
    """op in {"allreduce", "allgather", "alltoall"} over the peer-mapped workspace (parallel.symm); all ranks call it."""
    world = len(peers)
    x = x.contiguous()
    code = {"allreduce": 0, "allgather": 1, "alltoall": 2}[op]
    rows, row_bytes = 1, x.numel() * x.element_size()
    shape = list(x.shape)
    if op == "allgather":
        for d in range(axis):
            rows *= x.shape[d]
        row_bytes //= rows
        shape[axis] *= world
    elif op == "alltoall":
        row_bytes //= world
    out = torch.empty(shape, dtype=x.dtype, device=x.device)
    a = SymmCollectiveArgs(code, _ptr(x), _ptr(out), rows, row_bytes, dtype_code(x.dtype) if op == "allreduce" else 0, world, rank,
                           (ctypes.c_void_p * 8)(*(list(peers) + [None] * (8 - world))), symm_bytes, _ptr(status), 0, mc_ptr or None)
    _check(lib().ortb200_symm_collective(ctypes.byref(a), ctypes.c_void_p(stream_ptr())), "ortb200_symm_collective")
    return out


class AllGatherGemmArgs(ctypes.Structure):
    _fields_ = [("x_local", ctypes.c_void_p), ("w", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("rows_local", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("dtype", ctypes.c_int), ("act", ctypes.c_int),
                ("world", ctypes.c_int), ("rank", ctypes.c_int), ("peers", ctypes.c_void_p * 8), ("symm_bytes", ctypes.c_int64),
                ("status", ctypes.c_void_p), ("use_pdl", ctypes.c_int)]


def allgather_gemm_max_rows(world, K, symm_bytes):
    fn = lib().ortb200_allgather_gemm_max_rows
    fn.restype = ctypes.c_int64
    return int(fn(world, K, ctypes.c_int64(symm_bytes)))


def allgather_gemm_offsets(symm_bytes, parity, src):
    """(byte offset of the gather area of `parity`, byte offset of source rank `src`'s flag word) in a workspace."""
    area, flag = lib().ortb200_allgather_gemm_area_offset, lib().ortb200_allgather_gemm_flag_offset
    area.restype = flag.restype = ctypes.c_int64
    return int(area(ctypes.c_int64(symm_bytes), parity)), int(flag(src))


def allgather_gemm(x_local, w, peers, rank, symm_bytes, bias=None, act="none", status=None):
    """concat over ranks of x_local [rows, K], times w^T ([N, K]) -> [world * rows, N], as one kernel: the shard is
    pushed to the peers' workspaces by spare warps while the tensor-core warps start on the local rows.  All ranks call it."""
    world = len(peers)
    x_local, w = x_local.contiguous(), w.contiguous()
    rows, K = x_local.shape
    out = torch.empty(world * rows, w.shape[0], dtype=x_local.dtype, device=x_local.device)
    a = AllGatherGemmArgs(_ptr(x_local), _ptr(w), _ptr(bias), _ptr(out), rows, w.shape[0], K, dtype_code(x_local.dtype), ACT[act], world, rank,
                          (ctypes.c_void_p * 8)(*(list(peers) + [None] * (8 - world))), symm_bytes, _ptr(status), 0)
    _check(lib().ortb200_allgather_gemm(ctypes.byref(a), ctypes.c_void_p(stream_ptr())), "ortb200_allgather_gemm")
    return out


# ---------------------------------------------------------------------------- misc
def argmax(x):
    x = x.contiguous()
    rows, n = x.numel() // x.shape[-1], x.shape[-1]
    out = torch.empty(x.shape[:-1], dtype=torch.int64, device=x.device)
    ws = torch.zeros(rows * 16, dtype=torch.uint8, device=x.device)
    _check(lib().ortb200_argmax(ctypes.c_void_p(_ptr(x)), ctypes.c_void_p(_ptr(out)), ctypes.c_int64(rows), ctypes.c_int64(n),
                                dtype_code(x.dtype), ctypes.c_void_p(_ptr(ws)), ctypes.c_int64(ws.numel()),
                                ctypes.c_void_p(stream_ptr())), "ortb200_argmax")
    return out


def gather_rows(table, ids):
    ids = ids.contiguous()
    out = torch.empty(*ids.shape, table.shape[1], dtype=table.dtype, device=table.device)
    _check(lib().ortb200_gather_rows(ctypes.c_void_p(_ptr(table)), ctypes.c_void_p(_ptr(ids)), ctypes.c_void_p(_ptr(out)),
                                     ctypes.c_int64(ids.numel()), ctypes.c_int64(table.shape[0]), table.shape[1],
                                     table.element_size(), ctypes.c_void_p(stream_ptr())), "ortb200_gather_rows")
    return out
