"""Generic wrapper that makes any ``transformers`` causal LM usable as a policy / teacher model
(cosmos_rl/policy/model/hf_models/__init__.py: the reference's ``hfmodel`` fallback, used for families without a
hand-written implementation: DeepSeek-V3, Gemma, Mistral, Phi, VLM text towers ...).

The framework's models take PACKED tokens; this wrapper re-pads them to ``[B, max_len]``, runs the HF decoder stack
with an attention mask and re-packs the hidden states, so everything downstream (fused log-prob kernel, GRPO loss,
flat optimizer, checkpointing) is shared with the native models. It is the compatibility path, not the fast path.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Any, Dict, List, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F
from .base import BaseModel, ModelRegistry, WeightMapper


class HFWeightMapper(WeightMapper):
    """Parameters keep their HF names (minus the wrapper prefix): no fusing, no renaming."""

    def hf_names(self, local: str) -> List[str]:
        return [local[len("inner."):] if local.startswith("inner.") else local]


@ModelRegistry.register(HFWeightMapper, default=True)
class HFModel(BaseModel):
    def __init__(self, hf_config: Dict[str, Any], attn_implementation: str = "sdpa"):
        super().__init__()
        from transformers import AutoConfig, AutoModelForCausalLM
        cfg = dict(hf_config) if isinstance(hf_config, dict) else hf_config.to_dict()
        mt = cfg.pop("model_type")
        cfg.pop("architectures", None)
        self.hf_config = AutoConfig.for_model(mt, **cfg)
        # vision-language families (a vision tower feeding image tokens into the decoder): same wrapper, the pixel
        # inputs of the current packed batch are handed over through ``mm_inputs``
        self.is_vlm = "vision_config" in cfg
        if self.is_vlm:
            from transformers import AutoModelForImageTextToText
            self.inner = AutoModelForImageTextToText.from_config(self.hf_config, attn_implementation=attn_implementation)
        else:
            self.inner = AutoModelForCausalLM.from_config(self.hf_config, attn_implementation=attn_implementation)
        self.mm_inputs: Dict[str, torch.Tensor] = {}
        c = self.hf_config.get_text_config() if self.is_vlm else self.hf_config
        self.args = SimpleNamespace(model_type=mt, vocab_size=c.vocab_size, dim=c.hidden_size,
                                    n_layers=c.num_hidden_layers, n_heads=c.num_attention_heads,
                                    norm_eps=getattr(c, "rms_norm_eps", 1e-6), tp_size=1, tp_rank=0,
                                    tie_word_embeddings=bool(getattr(c, "tie_word_embeddings", False)),
                                    to_hf_config=lambda: dict(self.hf_config.to_dict(), model_type=mt))
        self.gradient_checkpointing = False
        self.tp = None

    @staticmethod
    def supported_model_types():
        return ["hfmodel"]

    @classmethod
    def from_hf_config(cls, hf_config, **kw):
        if kw.get("tp_size", 1) != 1:
            raise ValueError("the generic HF wrapper has no tensor-parallel plan; use dp_shard / a native model")
        return cls(hf_config)

    # ------------------------------------------------------------------ materialisation helpers
    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        g = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.dim() == 1:         # biases start at zero, every other vector is a scale (norm weights, ln_q ...)
                    p.zero_() if name.endswith("bias") else p.fill_(1.0)
                else:
                    p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32).mul_(std).to(p.dtype))
        self.materialize_buffers()

    init_weights_on_device = init_weights

    def materialize_buffers(self) -> None:
        """Buffers built in ``__init__`` (rotary ``inv_freq``) are lost when the model is created on the meta
        device; rebuild them on the device the parameters live on."""
        dev = next(self.parameters()).device
        for mod in self.inner.modules():
            inv = getattr(mod, "inv_freq", None)
            if inv is None or not (inv.is_meta or inv.device != dev) or any(True for _ in mod.parameters()):
                continue
            # rotary-embedding modules own no parameters: building them again on the right device is exact
            if hasattr(mod, "config"):
                try:
                    type(mod).__init__(mod, mod.config, device=dev)
                except TypeError:
                    type(mod).__init__(mod, config=mod.config)
                    mod.to(dev)
            elif hasattr(mod, "dim") and hasattr(mod, "theta"):      # vision-tower rotary tables: (dim, theta)
                type(mod).__init__(mod, mod.dim, mod.theta)
                mod.to(dev)
        # any other buffer (router bias terms ...) is checkpoint state: zero until a checkpoint is loaded
        for mod in self.inner.modules():
            for name, buf in list(mod._buffers.items()):
                if buf is not None and buf.is_meta:
                    mod._buffers[name] = torch.zeros(buf.shape, dtype=buf.dtype, device=dev)

    # ------------------------------------------------------------------ forward
    @property
    def lm_head_weight(self) -> torch.Tensor:
        return self.inner.get_output_embeddings().weight

    def get_position_ids(self, cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
        pos = torch.arange(total, device=cu_seqlens.device)
        starts = torch.repeat_interleave(cu_seqlens[:-1].long(), (cu_seqlens[1:] - cu_seqlens[:-1]).long())
        return pos - starts

    def forward(self, input_ids, position_ids, cu_seqlens, max_seqlen: int):
        """Packed ``input_ids [T]`` -> final hidden states ``[T, H]``."""
        cu = cu_seqlens.long()
        lens = cu[1:] - cu[:-1]
        B, L = lens.numel(), int(max_seqlen)
        T = input_ids.numel()
        seq = torch.repeat_interleave(torch.arange(B, device=input_ids.device), lens)
        col = torch.arange(T, device=input_ids.device) - cu[:-1][seq]
        ids = torch.zeros(B, L, dtype=input_ids.dtype, device=input_ids.device)
        pos = torch.zeros(B, L, dtype=torch.long, device=input_ids.device)
        mask = torch.zeros(B, L, dtype=torch.long, device=input_ids.device)
        ids[seq, col], pos[seq, col], mask[seq, col] = input_ids, position_ids.long(), 1
        if self.gradient_checkpointing and torch.is_grad_enabled() and not self.inner.is_gradient_checkpointing:
            self.inner.gradient_checkpointing_enable()
        if self.is_vlm:
            # multimodal rotary positions depend on the image grids: the model derives them from ids + mask
            mm = {k: v.to(ids.device) for k, v in (self.mm_inputs or {}).items()}
            out = self.inner.model(input_ids=ids, attention_mask=mask, use_cache=False, **mm)
        else:
            out = self.inner.model(input_ids=ids, attention_mask=mask, position_ids=pos, use_cache=False)
        return out.last_hidden_state[seq, col]

    def logprobs(self, hidden, labels, temperature: float = 1.0):
        return F.fused_logprob(hidden, self.lm_head_weight, labels, temperature)

    def logits(self, hidden):
        return torch.nn.functional.linear(hidden, self.lm_head_weight)

    def get_nparams_and_flops(self, seq_len: int) -> Tuple[int, int]:
        n = sum(p.numel() for p in self.parameters())
        return n, 6 * n
