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
                 device: Optional[torch.device] = None, prefill_graph: bool = False):
        """``prefill_graph``: also capture the prompt run in a CUDA graph (one graph per prompt shape; worthwhile when the
        same prompt shape recurs, e.g. fixed-size prefill chunks).  Needs a session created with ``enable_cuda_graph``."""
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
        self._prefill_graph = prefill_graph
        self._prefill_graph_ids: Dict[Tuple[int, int], int] = {}

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
        ro = self._ro_prefill
        if self._prefill_graph:
            gid = self._prefill_graph_ids.setdefault((B, S), 2 + len(self._prefill_graph_ids))
            ro = RunOptions()
            ro.add_run_config_entry("gpu_graph_id", str(gid))
        try:
            self.sess.run_with_iobinding(binding, ro)
        except Exception:
            if ro is self._ro_prefill:
                raise
            # the prompt graph holds something that cannot be captured: run it eagerly from now on
            self._prefill_graph = False
            self.sess.run_with_iobinding(binding, self._ro_prefill)
        self.cur_len = S
        self.prefill_logits = logits
        if not self.has_argmax:
            nxt = logits.float().argmax(-1)
        return nxt

    def reorder_cache(self, rows: torch.Tensor) -> None:
        """Row i of every cache takes the content of row rows[i] (beam search: beams follow their parents)."""
        rows = rows.to(self.device)
        for k, v in self.cache:
            k.copy_(k.index_select(0, rows))
            v.copy_(v.index_select(0, rows))

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
                 tp_size: int = 1, device: Optional[torch.device] = None, graph_id: int = 1):
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
        self._ro_decode.add_run_config_entry("gpu_graph_id", str(graph_id))  # one captured graph per (session, shape)
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


# ----------------------------------------------------------------------------------------------------------------
# Logits processors, sampling and beam search on top of DecoderRunner.  The knobs are the attributes / inputs of the
# reference's generation operators (com.microsoft GreedySearch, Sampling, BeamSearch:
# onnxruntime/contrib_ops/cpu/transformers/{greedy_search.cc, sampling.cc, beam_search.cc, logits_processor.h});
# here the loop runs in Python over the session's bound decode step and all tensor work stays on the device.
class GenerationConfig:
    def __init__(self, max_new_tokens: int = 32, min_new_tokens: int = 0, eos_token_id: Optional[int] = None,
                 pad_token_id: int = 0, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
                 repetition_penalty: float = 1.0, no_repeat_ngram_size: int = 0, num_beams: int = 1,
                 length_penalty: float = 1.0, early_stopping: bool = False, num_return_sequences: int = 1,
                 vocab_mask: Optional[torch.Tensor] = None, seed: Optional[int] = None):
        self.__dict__.update(locals())
        del self.__dict__["self"]


def process_logits(logits: torch.Tensor, sequences: torch.Tensor, step: int, cfg: GenerationConfig) -> torch.Tensor:
    """logits [rows, vocab] (fp32), sequences [rows, len] = every token so far (prompt included).  Order of the
    reference's LogitsProcessorList: min length, repetition penalty, no-repeat n-gram, vocabulary mask, temperature."""
    logits = logits.float().clone()
    if cfg.eos_token_id is not None and step < cfg.min_new_tokens:
        logits[:, cfg.eos_token_id] = float("-inf")
    if cfg.repetition_penalty != 1.0:
        seen = torch.gather(logits, 1, sequences)
        seen = torch.where(seen < 0, seen * cfg.repetition_penalty, seen / cfg.repetition_penalty)
        logits.scatter_(1, sequences, seen)
    n = cfg.no_repeat_ngram_size
    if n > 0 and sequences.shape[1] + 1 >= n:
        L = sequences.shape[1]
        if n == 1:
            logits.scatter_(1, sequences, float("-inf"))
        else:
            grams = sequences.unfold(1, n, 1)                      # [rows, L - n + 1, n]
            tail = sequences[:, L - (n - 1):].unsqueeze(1)          # [rows, 1, n - 1]
            hit = (grams[:, :, : n - 1] == tail).all(-1)            # n-grams whose prefix equals the current tail
            banned = torch.where(hit, grams[:, :, n - 1], torch.full_like(grams[:, :, n - 1], -1))
            rows = torch.arange(logits.shape[0], device=logits.device).unsqueeze(1).expand_as(banned)
            keep = banned >= 0
            logits[rows[keep], banned[keep]] = float("-inf")
    if cfg.vocab_mask is not None:
        logits = logits.masked_fill(cfg.vocab_mask.to(logits.device).view(1, -1) == 0, float("-inf"))
    if cfg.temperature != 1.0 and cfg.temperature > 0:
        logits = logits / cfg.temperature
    return logits


def top_k_top_p_filter(logits: torch.Tensor, top_k: int, top_p: float) -> torch.Tensor:
    if top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.shape[-1]), dim=-1).values[:, -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:
        sorted_logits, idx = torch.sort(logits, descending=True, dim=-1)
        cum = torch.softmax(sorted_logits, -1).cumsum(-1)
        drop = cum - torch.softmax(sorted_logits, -1) > top_p       # keep the token that crosses the threshold
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(1, idx, sorted_logits)
    return logits


def generate(runner: DecoderRunner, input_ids: torch.Tensor, cfg: GenerationConfig) -> torch.Tensor:
    """Greedy (``num_beams == 1``, ``top_k == 0``, ``top_p == 1``, temperature 1), sampling or beam search.
    Returns [batch * num_return_sequences, prompt + generated] token ids, padded with ``pad_token_id`` after EOS.
    For beam search the runner must have been created with ``batch = prompts * num_beams``."""
    if cfg.num_beams > 1:
        return _beam_search(runner, input_ids, cfg)
    dev = runner.device
    sampling = cfg.top_k > 0 or cfg.top_p < 1.0 or cfg.seed is not None
    gen = torch.Generator(device=dev)
    if cfg.seed is not None:
        gen.manual_seed(cfg.seed)
    seqs = input_ids.to(dev)
    done = torch.zeros(seqs.shape[0], dtype=torch.bool, device=dev)
    runner.prefill(input_ids)
    logits = _last_logits(runner, prefill=True)
    for step in range(cfg.max_new_tokens):
        scores = process_logits(logits, seqs, step, cfg)
        if sampling:
            probs = torch.softmax(top_k_top_p_filter(scores, cfg.top_k, cfg.top_p), -1)
            nxt = torch.multinomial(probs, 1, generator=gen).squeeze(1)
        else:
            nxt = scores.argmax(-1)
        nxt = torch.where(done, torch.full_like(nxt, cfg.pad_token_id), nxt)
        seqs = torch.cat([seqs, nxt.unsqueeze(1)], 1)
        if cfg.eos_token_id is not None:
            done = done | (nxt == cfg.eos_token_id)
            if bool(done.all()):
                break
        if step + 1 < cfg.max_new_tokens:
            runner.decode_step(nxt.view(-1, 1))
            logits = _last_logits(runner, prefill=False)
    return seqs


def _last_logits(runner: DecoderRunner, prefill: bool) -> torch.Tensor:
    src = runner.prefill_logits if prefill else runner.step_logits
    return src.reshape(src.shape[0], -1).float()


def _beam_search(runner: DecoderRunner, input_ids: torch.Tensor, cfg: GenerationConfig) -> torch.Tensor:
    """Beam search with the scorer of the reference (beam_search_scorer.cc): hypotheses are ranked by
    sum(log p) / length ** length_penalty, 2 * num_beams candidates are examined per step so that finished beams
    can be replaced, and the KV cache rows follow their beams."""
    dev = runner.device
    B, K = input_ids.shape[0], cfg.num_beams
    assert runner.batch == B * K, "beam search needs a runner with batch = prompts * num_beams"
    seqs = input_ids.to(dev).repeat_interleave(K, 0)
    prompt_len = seqs.shape[1]
    runner.prefill(seqs)
    logits = _last_logits(runner, prefill=True)
    beam_scores = torch.zeros(B, K, device=dev)
    beam_scores[:, 1:] = -1e9                    # all beams of a prompt start identical: keep one alive
    finished: List[List[Tuple[float, torch.Tensor]]] = [[] for _ in range(B)]
    done = [False] * B
    V = logits.shape[-1]
    for step in range(cfg.max_new_tokens):
        logp = torch.log_softmax(process_logits(logits, seqs, step, cfg), -1)
        cand = (beam_scores.view(B * K, 1) + logp).view(B, K * V)
        top_scores, top_idx = torch.topk(cand, 2 * K, dim=1)
        src_beam, token = top_idx // V, top_idx % V
        new_scores = torch.full((B, K), -1e9, device=dev)
        new_src = torch.zeros(B, K, dtype=torch.long, device=dev)
        new_tok = torch.full((B, K), cfg.pad_token_id, dtype=torch.long, device=dev)
        ts, sb, tk = top_scores.tolist(), src_beam.tolist(), token.tolist()
        cur_len = seqs.shape[1] + 1 - prompt_len
        for b in range(B):
            if done[b]:
                continue
            filled = 0
            for rank in range(2 * K):
                if cfg.eos_token_id is not None and tk[b][rank] == cfg.eos_token_id:
                    if rank < K:   # only candidates that would have survived may finish
                        hyp = torch.cat([seqs[b * K + sb[b][rank]], torch.tensor([cfg.eos_token_id], device=dev)])
                        finished[b].append((ts[b][rank] / (cur_len ** cfg.length_penalty), hyp))
                    continue
                new_scores[b, filled], new_src[b, filled], new_tok[b, filled] = ts[b][rank], sb[b][rank], tk[b][rank]
                filled += 1
                if filled == K:
                    break
            if len(finished[b]) >= K:
                best_open = float(new_scores[b].max()) / (cur_len ** cfg.length_penalty)
                worst_kept = sorted(f[0] for f in finished[b])[-K]
                if cfg.early_stopping or worst_kept >= best_open:
                    done[b] = True
        rows = (torch.arange(B, device=dev).unsqueeze(1) * K + new_src).view(-1)
        seqs = torch.cat([seqs.index_select(0, rows), new_tok.view(-1, 1)], 1)
        beam_scores = new_scores
        if all(done):
            break
        if step + 1 < cfg.max_new_tokens:
            runner.reorder_cache(rows)
            runner.decode_step(new_tok.view(-1, 1))
            logits = _last_logits(runner, prefill=False)
    out = []
    gen_len = seqs.shape[1] - prompt_len
    for b in range(B):
        hyps = list(finished[b])
        for k in range(K):   # open beams count as hypotheses of the current length
            hyps.append((float(beam_scores[b, k]) / (max(gen_len, 1) ** cfg.length_penalty), seqs[b * K + k]))
        hyps.sort(key=lambda h: -h[0])
        out.extend(h[1] for h in hyps[: cfg.num_return_sequences])
    width = max(h.shape[0] for h in out)
    return torch.stack([torch.nn.functional.pad(h, (0, width - h.shape[0]), value=cfg.pad_token_id) for h in out])
