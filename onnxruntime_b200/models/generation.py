"""Greedy generation drivers for decoder graphs with GroupQueryAttention or PagedAttention.

Mirrors how the reference's tooling drives an exported LLM
(onnxruntime/python/tools/transformers/models/llama/benchmark_e2e.py:120-148,
435-512): inputs and outputs are bound once with ``IOBinding``; ``past`` and
``present`` of every layer are bound to the SAME pre-allocated cache buffer so
the KV cache never moves; the prompt runs once, then one token per step.  The
decode step has fixed shapes and addresses, so with ``enable_cuda_graph`` the
session captures it on the first step and replays it afterwards.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..capi import InferenceSession, RunOptions
from .llama import LlamaConfig, empty_kv_cache, empty_paged_cache


class DecoderRunner:
    """Owns the KV cache and the bindings of one (session, batch size, cache capacity)."""

    def __init__(self, session: InferenceSession, cfg: LlamaConfig, batch: int, max_len: int, tp_size: int = 1,
                 device: Optional[torch.device] = None):
        self.sess = session
        self.cfg = cfg
        self.batch = batch
        self.max_len = max_len
        self.device = device if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if "CUDAExecutionProvider" in session.get_providers() else torch.device("cpu"))
        self.cache = empty_kv_cache(cfg, batch, max_len, self.device, tp_size)
        self.out_names = [o.name for o in session.get_outputs()]
        self.has_argmax = "next_tokens" in self.out_names
        # static device buffers for the decode step (addresses must not change between graph replays)
        self.step_ids = torch.zeros(batch, 1, dtype=torch.int64, device=self.device)
        self.step_seqlens = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.step_next = torch.zeros(batch, 1, dtype=torch.int64, device=self.device)
        self.step_logits = torch.zeros(batch, 1, cfg.vocab_size, dtype=self.cache[0][0].dtype, device=self.device)
        self._decode_binding = None
        self._decode_total = None
        self._ro_decode = RunOptions()
        self._ro_decode.add_run_config_entry("gpu_graph_id", "1")
        self._ro_prefill = RunOptions()
        self._ro_prefill.add_run_config_entry("gpu_graph_id", "-1")

    def _bind_common(self, binding, ids: torch.Tensor, seqlens: torch.Tensor, total: torch.Tensor, logits, next_tokens) -> None:
        binding.bind_torch_input("input_ids", ids)
        binding.bind_torch_input("seqlens_k", seqlens)
        binding.bind_torch_input("total_sequence_length", total)
        for i, (k, v) in enumerate(self.cache):
            binding.bind_torch_input(f"past_key_values.{i}.key", k)
            binding.bind_torch_input(f"past_key_values.{i}.value", v)
            binding.bind_torch_output(f"present.{i}.key", k)
            binding.bind_torch_output(f"present.{i}.value", v)
        binding.bind_torch_output("logits", logits)
        if self.has_argmax:
            binding.bind_torch_output("next_tokens", next_tokens)

    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt [B, S]; returns the first generated token per sequence [B, 1] (device tensor)."""
        B, S = input_ids.shape
        assert B == self.batch and S <= self.max_len
        ids = input_ids.to(self.device)
        seqlens = torch.full((B,), S - 1, dtype=torch.int32, device=self.device)
        total = torch.tensor(S, dtype=torch.int32)
        logits = torch.empty(B, 1, self.cfg.vocab_size, dtype=self.cache[0][0].dtype, device=self.device)
        nxt = torch.empty(B, 1, dtype=torch.int64, device=self.device)
        binding = self.sess.io_binding()
        self._bind_common(binding, ids, seqlens, total, logits, nxt)
        self.sess.run_with_iobinding(binding, self._ro_prefill)
        self.cur_len = S
        if not self.has_argmax:
            nxt = logits.float().argmax(-1)
        return nxt

    def _ensure_decode_binding(self) -> None:
        if self._decode_binding is not None:
            return
        binding = self.sess.io_binding()
        # the capacity bound is a host scalar: the cache capacity, so the captured graph stays valid every step
        self._decode_total = torch.tensor(self.max_len, dtype=torch.int32)
        self._bind_common(binding, self.step_ids, self.step_seqlens, self._decode_total, self.step_logits, self.step_next)
        self._decode_binding = binding

    def decode_step(self, tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode step.  ``tokens`` [B, 1] (device or pinned host); None re-uses the previous step's output,
        which already sits in the bound input buffer."""
        self._ensure_decode_binding()
        if tokens is not None:
            self.step_ids.copy_(tokens, non_blocking=True)
        else:
            self.step_ids.copy_(self.step_next)
        self.step_seqlens.fill_(self.cur_len)  # total length - 1 after appending this token
        self.sess.run_with_iobinding(self._decode_binding, self._ro_decode)
        self.cur_len += 1
        if not self.has_argmax:
            self.step_next.copy_(self.step_logits.float().argmax(-1))
        return self.step_next

    def decode_step_host(self, ids_pinned: torch.Tensor, seqlens_pinned: torch.Tensor, out_pinned: torch.Tensor) -> None:
        """One decode step driven from the host: inputs come from pinned host memory, the sampled tokens are
        copied back to pinned host memory and the call returns after they have arrived."""
        self._ensure_decode_binding()
        seqlens_pinned.fill_(self.cur_len)
        self.step_ids.copy_(ids_pinned, non_blocking=True)
        self.step_seqlens.copy_(seqlens_pinned, non_blocking=True)
        self.sess.run_with_iobinding(self._decode_binding, self._ro_decode)
        self.cur_len += 1
        if not self.has_argmax:
            self.step_next.copy_(self.step_logits.float().argmax(-1))
        out_pinned.copy_(self.step_next, non_blocking=True)
        torch.cuda.current_stream().synchronize() if self.device.type == "cuda" else None

    def generate(self, input_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        out = [self.prefill(input_ids).clone()]
        for _ in range(max_new_tokens - 1):
            nxt = self.decode_step(out[-1])
            out.append(nxt.clone())
        return torch.cat(out, dim=1)


class PagedDecoderRunner:
    """Greedy decoding over a block (paged) KV cache: the serving form of the decoder, where all sequences share
    one pool of cache blocks and ``block_table[b, j]`` names the block that holds tokens [j * block_size,
    (j + 1) * block_size) of sequence b (the inputs of com.microsoft.PagedAttention,
    onnxruntime/contrib_ops/cuda/bert/paged_attention.cc).  Blocks are handed out round-robin over the sequences,
    so no sequence owns a contiguous range and every access goes through the table.  The decode step has fixed
    shapes and addresses and is captured as one CUDA graph."""

    def __init__(self, session: InferenceSession, cfg: LlamaConfig, batch: int, max_len: int, block_size: int = 256,
                 tp_size: int = 1, device: Optional[torch.device] = None):
        self.sess, self.cfg, self.batch, self.max_len, self.block_size = session, cfg, batch, max_len, block_size
        self.device = device if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if "CUDAExecutionProvider" in session.get_providers() else torch.device("cpu"))
        per_seq = (max_len + block_size - 1) // block_size
        self.cache = empty_paged_cache(cfg, batch * per_seq, block_size, self.device, tp_size)
        self.block_table = torch.arange(batch * per_seq, dtype=torch.int32).view(per_seq, batch).t().contiguous().to(self.device)
        dt = self.cache[0][0].dtype
        self.step_ids = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self.step_cum = torch.arange(batch + 1, dtype=torch.int32, device=self.device)
        self.step_past = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.step_rows = torch.arange(batch, dtype=torch.int64, device=self.device)
        self.step_logits = torch.zeros(batch, cfg.vocab_size, dtype=dt, device=self.device)
        self.step_next = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self.has_argmax = "next_tokens" in [o.name for o in session.get_outputs()]
        self._decode_binding = None
        self._ro_decode = RunOptions()
        self._ro_decode.add_run_config_entry("gpu_graph_id", "1")
        self._ro_prefill = RunOptions()
        self._ro_prefill.add_run_config_entry("gpu_graph_id", "-1")
        self.cur_len = 0

    def _bind(self, binding, ids, cum, past, rows, logits, nxt) -> None:
        binding.bind_torch_input("input_ids", ids)
        binding.bind_torch_input("cumulative_sequence_length", cum)
        binding.bind_torch_input("past_seqlens", past)
        binding.bind_torch_input("block_table", self.block_table)
        binding.bind_torch_input("logits_indices", rows)
        for i, (k, v) in enumerate(self.cache):
            binding.bind_torch_input(f"key_cache.{i}", k)
            binding.bind_torch_input(f"value_cache.{i}", v)
            binding.bind_torch_output(f"key_cache_out.{i}", k)
            binding.bind_torch_output(f"value_cache_out.{i}", v)
        binding.bind_torch_output("logits", logits)
        if self.has_argmax:
            binding.bind_torch_output("next_tokens", nxt)

    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Prompts [B, S] of equal length, packed to [B * S] tokens; returns the first generated token [B]."""
        B, S = input_ids.shape
        assert B == self.batch and S <= self.max_len
        ids = input_ids.reshape(-1).to(self.device)
        cum = (torch.arange(B + 1, dtype=torch.int32) * S).to(self.device)
        past = torch.zeros(B, dtype=torch.int32, device=self.device)
        rows = (torch.arange(1, B + 1, dtype=torch.int64) * S - 1).to(self.device)
        logits = torch.empty(B, self.cfg.vocab_size, dtype=self.step_logits.dtype, device=self.device)
        nxt = torch.empty(B, dtype=torch.int64, device=self.device)
        binding = self.sess.io_binding()
        self._bind(binding, ids, cum, past, rows, logits, nxt)
        self.sess.run_with_iobinding(binding, self._ro_prefill)
        self.cur_len = S
        if not self.has_argmax:
            nxt = logits.float().argmax(-1)
        return nxt

    def assume_context(self, length: int) -> None:
        """Treat the caches as holding ``length`` tokens per sequence (benchmarks that time decode over a cache
        filled with arbitrary values instead of running a prompt first)."""
        assert 0 <= length < self.max_len
        self.cur_len = length

    def decode_step(self, tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token per sequence; ``tokens`` [B] or None to feed back the previous step's output."""
        if self._decode_binding is None:
            self._decode_binding = self.sess.io_binding()
            self._bind(self._decode_binding, self.step_ids, self.step_cum, self.step_past, self.step_rows, self.step_logits,
                       self.step_next)
        self.step_ids.copy_(tokens.reshape(-1) if tokens is not None else self.step_next, non_blocking=True)
        self.step_past.fill_(self.cur_len)
        self.sess.run_with_iobinding(self._decode_binding, self._ro_decode)
        self.cur_len += 1
        if not self.has_argmax:
            self.step_next.copy_(self.step_logits.float().argmax(-1))
        return self.step_next

    def generate(self, input_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        out = [self.prefill(input_ids).clone()]
        for _ in range(max_new_tokens - 1):
            out.append(self.decode_step(out[-1]).clone())
        return torch.stack(out, dim=1)
