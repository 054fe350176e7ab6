"""Library arm of the headline benchmark: the same Llama-shaped decoder written with vendor-library kernels only.

This is the op decomposition the reference's CUDA provider executes for this model on a B200, restated with
PyTorch: cuBLAS GEMMs (``torch.matmul``; reference: onnxruntime/core/providers/cuda/math/matmul.cc:180-419), a separate
RMS-norm kernel per norm (SkipSimplifiedLayerNormalization, onnxruntime/contrib_ops/cuda/bert/skip_layer_norm_impl.cu),
FlashAttention-2 with in-kernel rotary embedding and cache append for the attention
(``flash_attn_with_kvcache`` = mha_fwd_kvcache, onnxruntime/contrib_ops/cuda/bert/flash_attention/flash_api.cc:441;
PyTorch SDPA when flash_attn is missing), a separate SiLU * up kernel, and one ``ncclAllReduce`` after each row-parallel
GEMM (onnxruntime/contrib_ops/cuda/collective/nccl_kernels.cc:413-427).  The decode step is captured in a CUDA graph
like the session's.  None of this package's kernels or its engine are on this path: it exists to give the
hand-written kernels an honest number to beat on the same box.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn.functional as F

try:  # FlashAttention-2: the kernel family the reference ships for GroupQueryAttention
    from flash_attn import flash_attn_with_kvcache  # type: ignore
except Exception:  # pragma: no cover - depends on the image
    flash_attn_with_kvcache = None


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    if hasattr(F, "rms_norm"):
        return F.rms_norm(x, (x.shape[-1],), w, eps)
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class LibraryLlama:
    """Random-init Llama-shaped decoder, tensor-parallel over ``tp`` ranks (heads and FFN columns split, vocabulary
    replicated), with a static KV cache [B, Smax, kv_heads / tp, head]."""

    def __init__(self, cfg, batch: int, max_len: int, rank: int = 0, tp: int = 1, device="cuda", dtype=torch.bfloat16,
                 group=None, use_graph: bool = True, seed: int = 0):
        self.cfg, self.B, self.max_len, self.tp, self.group = cfg, batch, max_len, tp, group
        self.device, self.dtype, self.use_graph = torch.device(device), dtype, use_graph
        H, hd = cfg.hidden_size, cfg.head_dim
        self.nq, self.nkv, self.ffn = cfg.num_heads // tp, max(cfg.num_kv_heads // tp, 1), cfg.ffn_size // tp
        g = torch.Generator(device=self.device).manual_seed(seed + 17 * rank)

        def w(*shape):
            return (torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32) * 0.02).to(dtype)

        self.embed = w(cfg.vocab_size, H)
        self.layers = []
        for _ in range(cfg.num_layers):
            self.layers.append(dict(
                ln1=torch.ones(H, device=self.device, dtype=dtype), ln2=torch.ones(H, device=self.device, dtype=dtype),
                wqkv=w((self.nq + 2 * self.nkv) * hd, H), wo=w(H, self.nq * hd), wgu=w(2 * self.ffn, H), wd=w(H, self.ffn)))
        self.ln_f = torch.ones(H, device=self.device, dtype=dtype)
        self.lm_head = w(cfg.vocab_size, H)
        half = hd // 2
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, dtype=torch.float64) / half))
        fr = torch.outer(torch.arange(max_len, dtype=torch.float64), inv)
        self.cos, self.sin = fr.cos().to(dtype).to(self.device), fr.sin().to(dtype).to(self.device)
        self.kc = [torch.zeros(batch, max_len, self.nkv, hd, device=self.device, dtype=dtype) for _ in range(cfg.num_layers)]
        self.vc = [torch.zeros(batch, max_len, self.nkv, hd, device=self.device, dtype=dtype) for _ in range(cfg.num_layers)]
        self.step_ids = torch.zeros(batch, 1, dtype=torch.int64, device=self.device)
        self.step_lens = torch.zeros(batch, dtype=torch.int32, device=self.device)  # tokens already in the cache
        self.step_next = torch.zeros(batch, 1, dtype=torch.int64, device=self.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.cur_len = 0
        # FlashAttention-2 is used when its kernels run on this device; otherwise PyTorch SDPA (cuDNN / flash back-ends)
        self.use_fa = False
        if flash_attn_with_kvcache is not None:
            try:
                q = torch.zeros(1, 1, self.nq, hd, device=self.device, dtype=dtype)
                kc = torch.zeros(1, 16, self.nkv, hd, device=self.device, dtype=dtype)
                flash_attn_with_kvcache(q, kc, kc.clone(), cache_seqlens=torch.ones(1, dtype=torch.int32, device=self.device), causal=True)
                torch.cuda.synchronize()
                self.use_fa = True
            except Exception:
                self.use_fa = False

    # ------------------------------------------------------------------------------------------------------------
    def _allreduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp > 1:
            import torch.distributed as dist
            dist.all_reduce(x, group=self.group)
        return x

    def _rope(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        # x [B, S, n, hd]; pos [B, S]; half-rotated (non-interleaved) form
        c, s = self.cos[pos].unsqueeze(2), self.sin[pos].unsqueeze(2)
        x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    def _attention(self, li: int, qkv: torch.Tensor, lens: torch.Tensor, S: int) -> torch.Tensor:
        B, hd = qkv.shape[0], self.cfg.head_dim
        q, k, v = qkv.view(B, S, self.nq + 2 * self.nkv, hd).split([self.nq, self.nkv, self.nkv], dim=2)
        if self.use_fa:
            o = flash_attn_with_kvcache(q, self.kc[li], self.vc[li], k=k, v=v, rotary_cos=self.cos, rotary_sin=self.sin,
                                        cache_seqlens=lens, causal=True, rotary_interleaved=False)
            return o.reshape(B, S, self.nq * hd)
        pos = lens.long().unsqueeze(1) + torch.arange(S, device=qkv.device).unsqueeze(0)
        q, k = self._rope(q, pos), self._rope(k, pos)
        bi = torch.arange(B, device=qkv.device).unsqueeze(1)
        self.kc[li][bi, pos] = k
        self.vc[li][bi, pos] = v
        keys = torch.arange(self.max_len, device=qkv.device)
        mask = keys.view(1, 1, 1, -1) <= pos.view(B, 1, S, 1)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), self.kc[li].transpose(1, 2), self.vc[li].transpose(1, 2), attn_mask=mask,
                                           enable_gqa=True)
        return o.transpose(1, 2).reshape(B, S, self.nq * hd)

    def forward(self, ids: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
        """ids [B, S]; lens [B] int32 = tokens already cached.  Returns the arg-max token of the last position [B, 1]."""
        B, S = ids.shape
        eps = getattr(self.cfg, "rms_eps", 1e-5)
        h = self.embed[ids]
        for li, L in enumerate(self.layers):
            x = _rms(h, L["ln1"], eps)
            qkv = torch.matmul(x, L["wqkv"].t())
            a = self._attention(li, qkv, lens, S)
            h = h + self._allreduce(torch.matmul(a, L["wo"].t()))
            x = _rms(h, L["ln2"], eps)
            gu = torch.matmul(x, L["wgu"].t())
            act = F.silu(gu[..., : self.ffn]) * gu[..., self.ffn:]
            h = h + self._allreduce(torch.matmul(act, L["wd"].t()))
        x = _rms(h[:, -1:, :], self.ln_f, eps)
        logits = torch.matmul(x, self.lm_head.t())
        return logits.float().argmax(-1)

    # ------------------------------------------------------------------------------------------------------------
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        ids = ids.to(self.device, non_blocking=True)
        lens = torch.zeros(self.B, dtype=torch.int32, device=self.device)
        nxt = self.forward(ids, lens)
        self.cur_len = ids.shape[1]
        return nxt

    def _step_body(self) -> None:
        self.step_next.copy_(self.forward(self.step_ids, self.step_lens))

    def decode_step(self, tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        if tokens is not None:
            self.step_ids.copy_(tokens, non_blocking=True)
        else:
            self.step_ids.copy_(self.step_next)
        self.step_lens.fill_(self.cur_len)
        self._run_step()
        self.cur_len += 1
        return self.step_next

    def decode_step_host(self, ids_pinned: torch.Tensor, lens_pinned: torch.Tensor, out_pinned: torch.Tensor) -> None:
        lens_pinned.fill_(self.cur_len)
        self.step_ids.copy_(ids_pinned, non_blocking=True)
        self.step_lens.copy_(lens_pinned, non_blocking=True)
        self._run_step()
        self.cur_len += 1
        out_pinned.copy_(self.step_next, non_blocking=True)

    def _run_step(self) -> None:
        if not self.use_graph:
            self._step_body()
            return
        if self.graph is None:
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):  # lazy initialisation (cuBLAS handles, NCCL channels) stays outside the capture
                    self._step_body()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._step_body()
        self.graph.replay()


def count_kernels_of_one_step(model: LibraryLlama) -> int:
    """Kernel launches of one eager decode step, counted with the PyTorch profiler (CUPTI); 0 when unavailable."""
    try:
        from torch.profiler import ProfilerActivity, profile
        graph, model.use_graph = model.use_graph, False
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            model._step_body()
            torch.cuda.synchronize()
        model.use_graph = graph
        return sum(1 for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA)
    except Exception:
        return 0
