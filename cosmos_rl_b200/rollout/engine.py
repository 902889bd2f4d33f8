"""The built-in generation engine (replaces vLLM / TensorRT-LLM of the reference:
cosmos_rl/rollout/vllm_rollout/vllm_rollout.py:145-1128).

* Paged KV cache ``[layers, pages, 2, hkv, page_size, d]``; page 0 is a scratch page for padded slots.
* Each prompt is prefilled once; its ``n`` samples share the prompt's full pages and own the rest
  (pages for the whole response are reserved at admission, so a running sequence is never preempted).
* The decode step (embedding -> layers with paged attention -> lm_head -> fused sampler -> bookkeeping)
  runs entirely on the device and is replayed from a CUDA graph per batch-size bucket; the host looks at
  the produced tokens only every ``check_interval`` steps to retire finished sequences and admit new ones.
* The engine runs on the policy model's own parameter tensors when colocated, or on its own copy that the
  weight-sync kernel writes into.
On CPU the same code runs with the PyTorch statements of the ops (no graphs).
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Sequence, Tuple

import os

import torch

from ..ops import functional as F
from ..utils.logging import logger


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    repetition_penalty: float = 1.0
    n: int = 1
    max_tokens: int = 128
    stop_token_ids: Tuple[int, ...] = ()
    logprobs: bool = True
    seed: Optional[int] = None

    @classmethod
    def from_config(cls, config, validation: bool = False) -> "SamplingParams":
        r, s = config.rollout, config.rollout.sampling_config
        if validation:
            v = config.validation
            return cls(temperature=v.temperature, top_p=v.top_p if v.top_p is not None else s.top_p,
                       top_k=v.top_k if v.top_k is not None else s.top_k, repetition_penalty=v.repetition_penalty,
                       n=v.n_generation, max_tokens=v.max_response_length or r.max_response_length, seed=r.seed)
        return cls(temperature=s.temperature, top_p=s.top_p, top_k=s.top_k, repetition_penalty=s.repetition_penalty,
                   n=r.n_generation, max_tokens=r.max_response_length, seed=r.seed)


@dataclass
class Completion:
    token_ids: List[int]
    logprobs: List[float]
    finish_reason: str = "length"

    @property
    def cumulative_logprob(self) -> float:
        return float(sum(self.logprobs))


@dataclass
class _Seq:
    prompt_idx: int
    sample_idx: int
    slot: int
    pages: List[int]
    shared_pages: int
    start_step: int = 0
    n_generated: int = 0
    tokens: List[int] = field(default_factory=list)
    lps: List[float] = field(default_factory=list)
    done: bool = False
    finish_reason: str = "length"


class RolloutEngine:
    def __init__(self, model, *, max_num_seqs: int = 128, max_model_len: int = 2048, page_size: int = 128,
                 num_pages: Optional[int] = None, max_prefill_tokens: int = 16384, use_cuda_graph: bool = True,
                 gpu_memory_utilization: Optional[float] = None,
                 check_interval: int = 16, seed: int = 0, tp=None, shared_prefix_decode: bool = False):
        self.model = model
        self.args = model.args
        self.device = model.norm.device
        self.dtype = model.norm.dtype
        self.cuda = self.device.type == "cuda"
        self.S = max_num_seqs
        self.max_model_len = max_model_len
        self.P = page_size if self.cuda else min(page_size, 16)
        self.max_pages_per_seq = (max_model_len + check_interval + self.P - 1) // self.P + 1
        a = self.args
        self.hq = a.n_heads // a.tp_size
        self.hkv = max(1, a.n_kv_heads // a.tp_size)
        self.d = a.head_dim
        self.L = a.n_layers
        if num_pages is None:
            num_pages = 1 + self.S * self.max_pages_per_seq
            if gpu_memory_utilization is not None and self.device.type == "cuda":
                # rollout.gpu_memory_utilization: the KV pool takes what that share of the device leaves after the
                # weights (never less than one full-length sequence); sequences wait for pages at admission
                free, total = torch.cuda.mem_get_info(self.device)
                budget = int(total * float(gpu_memory_utilization)) - (total - free)
                page_bytes = self.L * 2 * self.hkv * self.P * self.d * torch.finfo(self.dtype).bits // 8
                num_pages = max(1 + self.max_pages_per_seq, min(num_pages, 1 + max(0, budget) // page_bytes))
        self.num_pages = num_pages
        self.kv = torch.zeros(self.L, num_pages, 2, self.hkv, self.P, self.d, dtype=self.dtype, device=self.device)
        # tensor-core decode kernel: V slabs are stored transposed
        self.kv_vt = self.cuda and F.tc_decode_supported(self.d, self.P, self.hq, self.hkv)
        self.free_pages: List[int] = list(range(num_pages - 1, 0, -1))
        self.page_refs: Dict[int, int] = {}
        self.max_prefill_tokens = max_prefill_tokens
        self.use_graph = use_cuda_graph and self.cuda
        self.check_interval = check_interval if self.cuda else 1
        self.seed = seed
        self.rep_penalty = 1.0
        self.seen: Optional[torch.Tensor] = None     # [slots, vocab] tokens already in prompt / output (repetition penalty)
        self.tp = tp if tp is not None else getattr(model, "tp", None)
        if (self.tp is not None and self.cuda and getattr(self.tp, "fused", None) is None
                and os.environ.get("COSMOS_B200_FUSED_TP", "1") != "0"):
            # row-parallel projections run as one GEMM + all-reduce kernel over peer memory
            self.tp.attach_fused(self.device, max(max_prefill_tokens, max_num_seqs), a.dim)
        self.weight_version = 0
        # ---- static decode state (device)
        S = self.S
        i32 = dict(dtype=torch.int32, device=self.device)
        self.block_table = torch.zeros(S, self.max_pages_per_seq, **i32)
        self.cur_len = torch.zeros(S, **i32)
        self.active = torch.zeros(S, **i32)
        self.last_tok = torch.zeros(S, dtype=torch.int64, device=self.device)
        self.temp = torch.ones(S, dtype=torch.float32, device=self.device)
        self.top_p = torch.ones(S, dtype=torch.float32, device=self.device)
        self.top_k = torch.full((S,), -1, **i32)
        self.step_counter = torch.zeros(1, dtype=torch.int64, device=self.device)
        # shared-prefix decode: the n samples of a prompt occupy consecutive slots and read the prompt's full pages
        # once per group (tcgen05 decode kernel only)
        self.prefix_pages = torch.zeros(S, **i32)
        self.group_n = 1
        self.shared_prefix_decode = shared_prefix_decode
        self.max_shared = max(1, min(16, max_model_len // self.P))
        self.ring = max(self.check_interval, 1)
        self.out_tok = torch.zeros(self.ring, S, dtype=torch.int64, device=self.device)
        self.out_lp = torch.zeros(self.ring, S, dtype=torch.float32, device=self.device)
        self.graphs: Dict[int, Any] = {}
        self.graph_launches: Dict[int, int] = {}
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "decode_steps": 0}

    # ------------------------------------------------------------------ pages
    def _alloc(self, n: int) -> List[int]:
        if len(self.free_pages) < n:
            raise RuntimeError("KV cache exhausted")
        out = [self.free_pages.pop() for _ in range(n)]
        for p in out:
            self.page_refs[p] = 1
        return out

    def _release(self, pages: Sequence[int]) -> None:
        for p in pages:
            self.page_refs[p] -= 1
            if self.page_refs[p] == 0:
                del self.page_refs[p]
                self.free_pages.append(p)

    def pages_needed(self, prompt_len: int, max_tokens: int, n: int) -> int:
        total = prompt_len + max_tokens + self.check_interval
        per_seq = (total + self.P - 1) // self.P
        shared = prompt_len // self.P
        return shared + n * (per_seq - shared)

    # ------------------------------------------------------------------ model pieces
    def _layers(self, h, positions, slot_mapping, attn):
        res = None
        m = self.model
        eps = self.args.norm_eps
        for li, layer in enumerate(m.layers):
            if res is None:
                x, _ = F.rms_norm(h, layer.input_layernorm, eps)
                res = h
            else:
                x, res = F.rms_norm(h, layer.input_layernorm, eps, residual=res)
            q, k, v = layer.self_attn.project_qkv(x, positions)
            F.kv_append(k, v, self.kv[li], slot_mapping, self.kv_vt)
            o = attn(li, q, k, v)
            o = o.reshape(o.shape[0], -1)
            if self.tp is not None:
                h = self.tp.row_linear(o, layer.self_attn.o_proj.weight)
            else:
                h = F.linear_maybe_fp8(o, layer.self_attn.o_proj.weight)
            x, res = F.rms_norm(h, layer.post_attention_layernorm, eps, residual=res)
            h = layer.mlp(x, self.tp)
        out, _ = F.rms_norm(h, m.norm, eps, residual=res)
        return out

    def _fused_decode_ok(self, B: int) -> bool:
        """The decode step can run on the weight-streaming GEMMs with fused reductions: bf16 weights on one GPU, no
        adapters, no per-head q/k norm, and a batch that fits the skinny kernel."""
        if not self.cuda or self.tp is not None or B > F._SKINNY_MAX_M or self.args.qk_norm or self.d % 8:
            return False
        if os.environ.get("COSMOS_B200_FUSED_DECODE", "1") == "0":
            return False
        ok = getattr(self, "_fused_ok", None)
        if ok is None:
            ok = True
            for layer in self.model.layers:
                for w in (layer.self_attn.qkv_proj.weight, layer.self_attn.o_proj.weight,
                          layer.mlp.gate_up_proj.weight, layer.mlp.down_proj.weight):
                    if (w.dtype != torch.bfloat16 or getattr(w, "_fp8", None) is not None
                            or getattr(w, "_lora", None) is not None or w.shape[0] % 8 or w.shape[1] % 8):
                        ok = False
            ok = ok and self.args.dim % 4 == 0 and self.args.dim <= 8192 and self.model.norm.dtype == torch.bfloat16
            self._fused_ok = ok
        return ok

    def _layers_decode_fused(self, h, positions, slot_mapping, attn):
        """One decode step through the blocks with four GEMM launches and three reductions per block: the qkv
        reduction applies bias and RoPE and appends K/V to the cache, the o_proj / down_proj reductions add the
        residual and apply the next RMSNorm, the gate/up GEMM multiplies SwiGLU in its epilogue."""
        m = self.model
        eps = self.args.norm_eps
        layers = list(m.layers)
        x, _ = F.rms_norm(h, layers[0].input_layernorm, eps)
        res = h
        for li, layer in enumerate(layers):
            at = layer.self_attn
            q = F.skinny_qkv_rope_append(x, at.qkv_proj.weight, at.qkv_proj.bias, positions, slot_mapping, at.theta,
                                         self.hq, self.hkv, self.d, self.kv[li], self.kv_vt)
            o = attn(li, q, None, None)
            x, res = F.skinny_linear_residual_rmsnorm(o.reshape(o.shape[0], -1), at.o_proj.weight, res,
                                                      layer.post_attention_layernorm, eps)
            act = F.skinny_gate_up_swiglu(x, layer.mlp.gate_up_proj.weight)
            nxt = layers[li + 1].input_layernorm if li + 1 < len(layers) else m.norm
            x, res = F.skinny_linear_residual_rmsnorm(act, layer.mlp.down_proj.weight, res, nxt, eps)
        return x

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def _prefill(self, prompts: List[List[int]], page_lists: List[List[int]]) -> torch.Tensor:
        """Run the prompts (packed), fill their pages, return last-position logits [n_prompts, V] fp32."""
        if torch.is_tensor(prompts[0]):
            ids = torch.cat([p.to(self.device, dtype=torch.long) for p in prompts])
        else:
            ids = torch.tensor([t for p in prompts for t in p], dtype=torch.long, device=self.device)
        lens = [len(p) for p in prompts]
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0).tolist()), dtype=torch.int32, device=self.device)
        pos = torch.cat([torch.arange(n, device=self.device) for n in lens])
        slots = []
        for n, pages in zip(lens, page_lists):
            t = torch.arange(n)
            slots.append(torch.tensor(pages, dtype=torch.long)[t // self.P] * self.P + t % self.P)
        slot_mapping = torch.cat(slots).to(torch.int32).to(self.device)
        max_len = max(lens)
        h = self.model.embed(ids)
        out = self._layers(h, pos, slot_mapping,
                           lambda li, q, k, v: F.varlen_attention(q, k, v, cu, max_len))
        last = (cu[1:] - 1).long()
        self.stats["prefill_tokens"] += int(ids.numel())
        return self.model.logits(out[last]).float()

    # ------------------------------------------------------------------ decode
    def _decode_body(self, B: int) -> None:
        """One decode step for slots [0, B): everything on the device, no host reads."""
        cur = self.cur_len[:B]
        act = self.active[:B]
        page_idx = (cur // self.P).long()
        page = self.block_table[:B].gather(1, page_idx[:, None]).squeeze(1)
        slot = torch.where(act > 0, page * self.P + cur % self.P, torch.full_like(cur, -1))
        seq_lens = torch.where(act > 0, cur + 1, torch.ones_like(cur))
        h = self.model.embed(self.last_tok[:B])
        bt = self.block_table[:B]
        prefix, scratch = {}, None
        if (self.shared_prefix_decode and self.kv_vt and self.group_n > 1
                and self.group_n * (self.hq // self.hkv) <= 128):
            prefix = dict(prefix_pages=self.prefix_pages[:B], group=self.group_n, max_shared=self.max_shared, nsplit=1)
            scratch = self._prefix_scratch(B)
        layers = self._layers_decode_fused if self._fused_decode_ok(B) else self._layers
        out = layers(h, cur.long(), slot,
                     lambda li, q, k, v: F.paged_decode(q, self.kv[li], bt, seq_lens, v_transposed=self.kv_vt,
                                                        scratch=scratch, **prefix))
        logits = self.model.logits(out)
        if self.rep_penalty != 1.0:
            logits = self._penalise(logits.float(), self.seen[:B])
        r = (self.step_counter % self.ring).long()
        if self.cuda:
            toks = torch.empty(B, dtype=torch.int64, device=self.device)
            lps = torch.empty(B, dtype=torch.float32, device=self.device)
            F.sample(logits, self.temp[:B], self.top_p[:B], self.top_k[:B], seed=self.seed, offset=1 << 20,
                     offset_dev=self.step_counter, out_tokens=toks, out_logprobs=lps)
        else:
            toks, lps = F.sample(logits.float(), self.temp[:B], self.top_p[:B], self.top_k[:B])
        self.out_tok.index_copy_(0, r, toks.unsqueeze(0) if B == self.S else
                                 torch.cat([toks, self.out_tok[0, B:]]).unsqueeze(0))
        self.out_lp.index_copy_(0, r, lps.unsqueeze(0) if B == self.S else
                                torch.cat([lps, self.out_lp[0, B:]]).unsqueeze(0))
        self.last_tok[:B] = torch.where(act > 0, toks, self.last_tok[:B])
        if self.rep_penalty != 1.0:
            self.seen[:B].scatter_(1, toks[:, None], True)      # rows of idle slots are reset when a sequence moves in
        self.cur_len[:B] += act
        self.step_counter += 1

    def _penalise(self, logits: torch.Tensor, seen: torch.Tensor) -> torch.Tensor:
        """Repetition penalty on tokens that already occur in the prompt or the output: positive logits are divided
        by the penalty, negative ones multiplied (the rule of the transformers / vLLM samplers)."""
        p = self.rep_penalty
        return torch.where(seen, torch.where(logits > 0, logits / p, logits * p), logits)

    def _prefix_scratch(self, B: int) -> torch.Tensor:
        need = B * self.hq * (self.max_shared + 1) * (self.d + 2)
        buf = getattr(self, "_pfx_scratch", None)
        if buf is None or buf.numel() < need:
            buf = self._pfx_scratch = torch.empty(self.S * self.hq * (self.max_shared + 1) * (self.d + 2),
                                                  dtype=torch.float32, device=self.device)
        return buf

    def _bucket(self, n: int) -> int:
        b = 8
        while b < n:
            b *= 2
        return min(b, self.S)

    @torch.no_grad()
    def _decode_step(self, n_slots: int) -> None:
        B = self._bucket(n_slots)
        if not self.use_graph:
            self._decode_body(B)
            return
        g = self.graphs.get(B)
        if g is None:
            # warm up outside capture (lazy initialisations, autotuned library GEMMs), then restore state
            saved = (self.cur_len.clone(), self.last_tok.clone(), self.step_counter.clone(),
                     self.out_tok.clone(), self.out_lp.clone(),
                     self.seen[:B].clone() if (self.rep_penalty != 1.0 and self.seen is not None) else None)
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):
                    self._decode_body(B)
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            from ..ops import native
            before = native.LAUNCHES[0]
            with torch.cuda.graph(g):
                self._decode_body(B)
            self.graph_launches[B] = native.LAUNCHES[0] - before
            self.cur_len.copy_(saved[0]); self.last_tok.copy_(saved[1]); self.step_counter.copy_(saved[2])
            self.out_tok.copy_(saved[3]); self.out_lp.copy_(saved[4])
            if saved[5] is not None:
                self.seen[:B].copy_(saved[5])     # the throw-away tokens of the warm-up must not count as "seen"
            self.graphs[B] = g
        g.replay()
        from ..ops import native
        native.add_launches(self.graph_launches.get(B, 0))

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sp: SamplingParams) -> List[List[Completion]]:
        """Generate ``sp.n`` completions for every prompt (token id lists)."""
        n = max(1, sp.n)
        results: List[List[Optional[Completion]]] = [[None] * n for _ in prompts]
        waiting: Deque[int] = deque(range(len(prompts)))
        running: Dict[int, _Seq] = {}
        if n > self.S:
            raise ValueError(f"{n} samples per prompt do not fit in {self.S} sequence slots")
        # a prompt's samples take one block of n consecutive slots; the block is reused when all of them finished
        free_groups = list(range(self.S // n - 1, -1, -1))
        group_live: Dict[int, int] = {}
        if n != self.group_n:
            self.group_n = n
            self.invalidate_graphs()        # the decode graphs bake the group size into the attention launch
        self.prefix_pages.zero_()
        if float(sp.repetition_penalty) != self.rep_penalty:
            self.rep_penalty = float(sp.repetition_penalty)
            self.invalidate_graphs()        # the penalty branch is part of the captured decode step
        if self.rep_penalty != 1.0 and self.seen is None:
            self.seen = torch.zeros(self.S, self.model.args.vocab_size, dtype=torch.bool, device=self.device)
        stop = set(sp.stop_token_ids)
        if sp.seed is not None:
            self.seed = sp.seed
        steps_since_check = 0
        host_step = 0

        def admit() -> None:
            nonlocal host_step
            batch, page_lists, tok_budget = [], [], self.max_prefill_tokens
            batch_groups: List[int] = []
            while waiting and free_groups:
                pi = waiting[0]
                p = prompts[pi] if torch.is_tensor(prompts[pi]) else list(prompts[pi])
                if len(p) + sp.max_tokens > self.max_model_len:
                    p = p[-(self.max_model_len - sp.max_tokens):]
                need = self.pages_needed(len(p), sp.max_tokens, n)
                if need > len(self.free_pages) or (batch and len(p) > tok_budget):
                    break
                waiting.popleft()
                n_prompt_pages = (len(p) + self.P - 1) // self.P
                pp = self._alloc(n_prompt_pages)
                batch.append((pi, p, pp))
                page_lists.append(pp)
                tok_budget -= len(p)
                batch_groups.append(free_groups.pop())
            if not batch:
                return
            logits = self._prefill([b[1] for b in batch], page_lists)
            # first token of each of the n samples comes from the prompt's last-position logits
            if self.rep_penalty != 1.0:
                pmask = torch.zeros(len(batch), logits.shape[1], dtype=torch.bool, device=self.device)
                for bi, (_, p, _) in enumerate(batch):
                    pmask[bi, torch.as_tensor(p, dtype=torch.long, device=self.device)] = True
                logits = self._penalise(logits, pmask)
            rep = logits.repeat_interleave(n, dim=0)
            B0 = rep.shape[0]
            t = torch.full((B0,), sp.temperature, dtype=torch.float32, device=self.device)
            tp_ = torch.full((B0,), sp.top_p, dtype=torch.float32, device=self.device)
            tk = torch.full((B0,), sp.top_k, dtype=torch.int32, device=self.device)
            first_tok, first_lp = F.sample(rep, t, tp_, tk, seed=self.seed, offset=host_step)
            first_tok_h, first_lp_h = first_tok.tolist(), first_lp.tolist()
            total_per_seq = lambda L: (L + sp.max_tokens + self.check_interval + self.P - 1) // self.P
            slots_taken = []
            for bi, (pi, p, pp) in enumerate(batch):
                shared = len(p) // self.P
                grp = batch_groups[bi]
                group_live[grp] = n
                for si in range(n):
                    slot = grp * n + si
                    own_n = total_per_seq(len(p)) - shared
                    own = self._alloc(own_n)
                    for q in pp[:shared]:
                        self.page_refs[q] += 1
                    pages = pp[:shared] + own
                    if shared < len(pp):
                        # the prompt's partial last page is private: copy it
                        self.kv[:, own[0]].copy_(self.kv[:, pp[shared]])
                    seq = _Seq(pi, si, slot, pages, shared, start_step=host_step)
                    k = bi * n + si
                    seq.tokens.append(first_tok_h[k])
                    seq.lps.append(first_lp_h[k])
                    seq.n_generated = 1
                    running[slot] = seq
                    slots_taken.append((slot, pages, len(p), first_tok_h[k], min(shared, self.max_shared)))
                self._release(pp)  # drop the prefill's own reference; children hold theirs
            # publish the new sequences' state to the device in one shot
            idx = torch.tensor([s[0] for s in slots_taken], dtype=torch.long, device=self.device)
            if self.rep_penalty != 1.0:
                rows = pmask.repeat_interleave(n, dim=0).clone()
                rows.scatter_(1, first_tok[:, None], True)
                order = {slot: k for k, slot in enumerate(grp * n + si for grp in batch_groups for si in range(n))}
                self.seen.index_copy_(0, idx, rows[torch.tensor([order[s_[0]] for s_ in slots_taken],
                                                               dtype=torch.long, device=self.device)])
            bt = torch.zeros(len(slots_taken), self.max_pages_per_seq, dtype=torch.int32)
            for i, (_, pages, _, _, _) in enumerate(slots_taken):
                bt[i, : len(pages)] = torch.tensor(pages, dtype=torch.int32)
            self.block_table.index_copy_(0, idx, bt.to(self.device))
            self.cur_len.index_copy_(0, idx, torch.tensor([s[2] for s in slots_taken], dtype=torch.int32, device=self.device))
            self.last_tok.index_copy_(0, idx, torch.tensor([s[3] for s in slots_taken], dtype=torch.int64, device=self.device))
            self.active.index_fill_(0, idx, 1)
            self.prefix_pages.index_copy_(0, idx, torch.tensor([s[4] for s in slots_taken], dtype=torch.int32,
                                                                device=self.device))
            self.temp.index_fill_(0, idx, sp.temperature)
            self.top_p.index_fill_(0, idx, sp.top_p)
            self.top_k.index_fill_(0, idx, sp.top_k)

        def retire(seq: _Seq, reason: str) -> None:
            seq.done, seq.finish_reason = True, reason
            results[seq.prompt_idx][seq.sample_idx] = Completion(seq.tokens, seq.lps, reason)
            self._release(seq.pages)
            del running[seq.slot]
            self.active[seq.slot] = 0
            self.prefix_pages[seq.slot] = 0
            grp = seq.slot // n
            group_live[grp] -= 1
            if group_live[grp] == 0:
                del group_live[grp]
                free_groups.append(grp)

        def harvest(n_steps: int) -> None:
            """Read the last ``n_steps`` rows of the token ring and retire finished sequences."""
            if n_steps == 0:
                return
            sc = int(self.step_counter.item())
            rows = [(sc - n_steps + i) % self.ring for i in range(n_steps)]
            toks = self.out_tok[rows].tolist()
            lps = self.out_lp[rows].tolist()
            for slot, seq in list(running.items()):
                first = max(0, seq.start_step - (host_step - n_steps))
                for i in range(first, n_steps):
                    if seq.done:
                        break
                    tok = toks[i][slot]
                    seq.tokens.append(tok)
                    seq.lps.append(lps[i][slot])
                    seq.n_generated += 1
                    if tok in stop:
                        retire(seq, "stop")
                    elif seq.n_generated >= sp.max_tokens:
                        retire(seq, "length")
            # sequences that finished on their very first token
            for slot, seq in list(running.items()):
                if not seq.done and (seq.tokens[-1] in stop or seq.n_generated >= sp.max_tokens):
                    retire(seq, "stop" if seq.tokens[-1] in stop else "length")

        admit()
        harvest(0)
        for slot, seq in list(running.items()):
            if seq.tokens[-1] in stop or seq.n_generated >= sp.max_tokens:
                retire(seq, "stop" if seq.tokens[-1] in stop else "length")
        while running or waiting:
            if not running:
                admit()
                if not running:
                    raise RuntimeError("a prompt does not fit in the KV cache")
                continue
            hi = max(running) + 1
            self._decode_step(hi)
            host_step += 1
            steps_since_check += 1
            self.stats["decode_steps"] += 1
            self.stats["decode_tokens"] += len(running)
            remaining = min(sp.max_tokens - s.n_generated - steps_since_check for s in running.values())
            if steps_since_check >= self.check_interval or remaining <= 0:
                harvest(steps_since_check)
                steps_since_check = 0
                if waiting:
                    admit()
        return [[c for c in row] for row in results]

    def release_cache(self) -> None:
        """Free the KV cache memory (colocated mode hands the memory to training)."""
        self.kv = None
        self.graphs.clear()
        if self.cuda:
            torch.cuda.empty_cache()

    def invalidate_graphs(self) -> None:
        self.graphs.clear()
        self._fused_ok = None       # adapters or quantised weights may have been attached since
