"""Data packers: model-specific conversion of dataset samples into rollout-engine inputs and of
(prompt, completion) pairs into policy training tensors
(contract of cosmos_rl/dispatcher/data/packer/base.py:54-266, decoder-only implementation
decoder_only_llm_data_packer.py:13-319).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Type, Union

import torch


class BaseDataPacker:
    _registry: Dict[str, Type["BaseDataPacker"]] = {}

    @classmethod
    def register(cls, model_types: Union[str, Sequence[str]], packer_cls: Optional[type] = None):
        if isinstance(model_types, str):
            model_types = [model_types]

        def deco(c):
            for mt in model_types:
                cls._registry[mt] = c
            return c
        return deco(packer_cls) if packer_cls is not None else deco

    @classmethod
    def get_default(cls, model_type: str) -> Type["BaseDataPacker"]:
        return cls._registry.get(model_type, DecoderOnlyLLMDataPacker)

    def setup(self, config, tokenizer=None, *a, **kw):
        self.config = config
        self.tokenizer = tokenizer

    # rollout side
    def get_rollout_input(self, item: Any) -> Any:
        raise NotImplementedError

    def rollout_collate_fn(self, items: List[Any]) -> Any:
        return items

    def get_rollout_output(self, items: List[Any], completed_conversations=None, logprobs=None, token_ids=None, **kw):
        return items

    # policy side
    def get_policy_input(self, sample: Any, rollout_output: Any, n_ignore_prefix_tokens: int = 0, **kw) -> Any:
        raise NotImplementedError

    def policy_compute_max_len(self, processed: List[Any]) -> int:
        raise NotImplementedError

    def policy_collate_fn(self, processed: List[Any], computed_max_len: int) -> Dict[str, Any]:
        raise NotImplementedError

    # sft
    def sft_process_sample(self, sample: Any) -> Any:
        raise NotImplementedError

    def sft_compute_max_len(self, processed: List[Any]) -> int:
        raise NotImplementedError

    def sft_collate_fn(self, processed: List[Any], computed_max_len: int, ignore_label_id: int = -100):
        raise NotImplementedError

    def batch_size(self, batch: Dict[str, Any]) -> int:
        return int(batch["input_ids"].shape[0])

    def slice_batch(self, batch: Dict[str, Any], start: int, end: int) -> Dict[str, Any]:
        return {k: (v[start:end] if torch.is_tensor(v) else v) for k, v in batch.items()}

    def save_state(self, path: str) -> None:
        pass


class DecoderOnlyLLMDataPacker(BaseDataPacker):
    """Text-only decoder LLMs. Prompts may be strings, chat conversations or already-tokenised id lists."""

    class PolicyInput:
        __slots__ = ("input_ids", "logprob_masks")

        def __init__(self, input_ids: List[int], logprob_masks: List[int]):
            self.input_ids = input_ids
            self.logprob_masks = logprob_masks

    def setup(self, config, tokenizer=None, *a, **kw):
        super().setup(config, tokenizer, *a, **kw)
        path = config.rollout.multi_turn_config.custom_chat_template_path
        if path and tokenizer is not None and hasattr(tokenizer, "chat_template"):
            with open(path) as f:
                tokenizer.chat_template = f.read()      # e.g. tools/chat_templates/tool_chat_template.jinja2
        # how a conversation becomes a generation prompt (multi-turn switches; defaults elsewhere)
        mt = config.rollout.multi_turn_config
        self.prompt_template_kwargs = {"add_generation_prompt": True}
        if mt.enable:
            self.prompt_template_kwargs["add_generation_prompt"] = bool(mt.add_generation_prompt
                                                                        and not mt.continue_final_message)
            if mt.continue_final_message:       # the model extends the last (assistant) message instead of opening one
                self.prompt_template_kwargs["continue_final_message"] = True
            if mt.enable_thinking:              # a variable of templates that gate a reasoning block on it
                self.prompt_template_kwargs["enable_thinking"] = True

    def _encode_prompt(self, prompt) -> List[int]:
        if isinstance(prompt, (list, tuple)) and (len(prompt) == 0 or isinstance(prompt[0], int)):
            return list(prompt)
        if self.tokenizer is None:
            raise RuntimeError("a tokenizer is required for text prompts")
        if isinstance(prompt, str):
            return self.tokenizer.encode(prompt, add_special_tokens=False)
        kw = getattr(self, "prompt_template_kwargs", {"add_generation_prompt": True})
        return self.tokenizer.apply_chat_template(prompt, tokenize=True, **kw)

    def _encode_completion(self, completion) -> List[int]:
        if isinstance(completion, (list, tuple)) and (len(completion) == 0 or isinstance(completion[0], int)):
            return list(completion)
        if self.tokenizer is None:
            raise RuntimeError("a tokenizer is required for text completions")
        ids = self.tokenizer.encode(completion, add_special_tokens=False)
        eos = getattr(self.tokenizer, "eos_token_id", None)
        return ids + ([eos] if eos is not None else [])

    def get_rollout_input(self, item):
        return self._encode_prompt(item)

    def extend_conversation(self, conversation, response: str, ground_truth=None):
        """Multi-turn rollouts: append the response (and the results of its tool calls). Returns (conversation,
        finished)."""
        from .multi_turn import extend_conversation
        mt = self.config.rollout.multi_turn_config
        return extend_conversation(conversation, response, mt.enable_tools)

    def get_policy_input(self, sample, rollout_output, n_ignore_prefix_tokens: int = 0, **kw):
        if isinstance(rollout_output, (list, tuple)) and rollout_output and isinstance(rollout_output[0], dict):
            # a completed multi-turn conversation: every assistant turn is scored, the rest is context
            from .multi_turn import ToolRegistry, assistant_token_mask
            tools = ToolRegistry.schemas() if self.config.rollout.multi_turn_config.enable_tools else None
            ids, m = assistant_token_mask(self.tokenizer, list(rollout_output), tools)
            return self.PolicyInput(ids, m[1:] + [0])       # mask[i] == 1 <=> token i + 1 is scored
        p = self._encode_prompt(sample)
        c = self._encode_completion(rollout_output)
        n_ign = min(n_ignore_prefix_tokens, len(c))
        # mask[i] == 1  <=>  token i+1 is a completion token whose log-prob is scored
        mask = [0] * (len(p) - 1 + n_ign) + [1] * (len(c) - n_ign) + [0]
        return self.PolicyInput(p + c, mask)

    def policy_compute_max_len(self, processed):
        return max(len(x.input_ids) for x in processed)

    def policy_collate_fn(self, processed, computed_max_len: int):
        pad = getattr(self.tokenizer, "pad_token_id", None) or 0
        ids = torch.full((len(processed), computed_max_len), pad, dtype=torch.long)
        masks = torch.zeros((len(processed), computed_max_len), dtype=torch.bool)
        for i, x in enumerate(processed):
            n = min(len(x.input_ids), computed_max_len)
            ids[i, :n] = torch.tensor(x.input_ids[:n], dtype=torch.long)
            masks[i, :n] = torch.tensor(x.logprob_masks[:n], dtype=torch.bool)
        return {"input_ids": ids, "logprob_masks": masks}

    # ---- SFT
    def sft_process_sample(self, sample):
        if isinstance(sample, dict) and "input_ids" in sample:
            return {"input_ids": list(sample["input_ids"]), "label_ids": list(sample.get("label_ids", sample["input_ids"]))}
        if isinstance(sample, (list, tuple)) and sample and isinstance(sample[0], int):
            return {"input_ids": list(sample), "label_ids": list(sample)}
        if self.tokenizer is None:
            raise RuntimeError("a tokenizer is required for conversation samples")
        conv = sample
        ids = self.tokenizer.apply_chat_template(conv, tokenize=True, add_generation_prompt=False)
        labels = list(ids)
        # score only assistant turns: mask the prefix up to the last assistant message
        prefix = self.tokenizer.apply_chat_template(conv[:-1], tokenize=True, add_generation_prompt=True)
        labels[: len(prefix)] = [-100] * min(len(prefix), len(labels))
        return {"input_ids": ids, "label_ids": labels}

    def sft_compute_max_len(self, processed):
        return max(len(x["input_ids"]) for x in processed)

    def sft_collate_fn(self, processed, computed_max_len: int, ignore_label_id: int = -100):
        pad = getattr(self.tokenizer, "pad_token_id", None) or 0
        ids = torch.full((len(processed), computed_max_len), pad, dtype=torch.long)
        labels = torch.full((len(processed), computed_max_len), ignore_label_id, dtype=torch.long)
        lens = torch.zeros(len(processed), dtype=torch.long)
        for i, x in enumerate(processed):
            n = min(len(x["input_ids"]), computed_max_len)
            ids[i, :n] = torch.tensor(x["input_ids"][:n])
            labels[i, :n] = torch.tensor(x["label_ids"][:n])
            lens[i] = n
        return {"input_ids": ids, "label_ids": labels, "seq_lens": lens}


BaseDataPacker.register(["llama", "qwen2", "qwen3", "qwen3_moe", "hfmodel"], DecoderOnlyLLMDataPacker)

MM_KEYS = ("pixel_values", "image_grid_thw", "pixel_values_videos", "video_grid_thw", "proprio")


def merge_mm(items: List[Optional[Dict[str, Any]]]) -> Dict[str, torch.Tensor]:
    """Concatenate the vision inputs of several samples in sample order (what HF vision-language models expect for a
    batch: all patches / grids of the batch stacked along dim 0)."""
    out: Dict[str, torch.Tensor] = {}
    for k in MM_KEYS:
        parts = [torch.as_tensor(it[k]) for it in items if it and it.get(k) is not None]
        if parts:
            out[k] = torch.cat(parts, dim=0)
    return out


class HFVLMDataPacker(DecoderOnlyLLMDataPacker):
    """Vision-language samples (cosmos_rl/dispatcher/data/packer/hf_vlm_data_packer.py). A sample is either already
    processed, ``{"input_ids": [...], "pixel_values": ..., "image_grid_thw": ...}`` (image placeholder tokens in
    place), or a conversation that the model's processor turns into that form (``setup(..., processor=...)`` or a
    processor loadable from the model folder)."""

    class PolicyInput(DecoderOnlyLLMDataPacker.PolicyInput):
        __slots__ = ("mm",)

        def __init__(self, input_ids, logprob_masks, mm=None):
            super().__init__(input_ids, logprob_masks)
            self.mm = mm

    def setup(self, config, tokenizer=None, processor=None, *a, **kw):
        super().setup(config, tokenizer)
        self.processor = processor
        path = getattr(config.policy, "model_name_or_path", "")
        if self.processor is None and path and __import__("os").path.isdir(path):
            try:
                from transformers import AutoProcessor
                self.processor = AutoProcessor.from_pretrained(path)
            except Exception:  # noqa: BLE001  (pre-processed samples need no processor)
                self.processor = None

    def _process(self, sample) -> Dict[str, Any]:
        if isinstance(sample, dict) and "prompt" in sample and "input_ids" not in sample:
            sample = sample["prompt"]
        if isinstance(sample, dict) and "input_ids" in sample:
            return {"input_ids": list(sample["input_ids"]), "mm": {k: sample[k] for k in MM_KEYS if sample.get(k) is not None}}
        if self.processor is None:
            raise RuntimeError("conversation samples of a vision-language model need its processor")
        enc = self.processor.apply_chat_template(sample, tokenize=True, add_generation_prompt=True, return_dict=True,
                                                 return_tensors="pt")
        return {"input_ids": enc["input_ids"][0].tolist(), "mm": {k: enc[k] for k in MM_KEYS if k in enc}}

    def get_rollout_input(self, item):
        return self._process(item)

    def get_policy_input(self, sample, rollout_output, n_ignore_prefix_tokens: int = 0, **kw):
        pr = self._process(sample)
        p, c = pr["input_ids"], self._encode_completion(rollout_output)
        n_ign = min(n_ignore_prefix_tokens, len(c))
        mask = [0] * (len(p) - 1 + n_ign) + [1] * (len(c) - n_ign) + [0]
        return self.PolicyInput(p + c, mask, pr["mm"])

    def sft_process_sample(self, sample):
        if isinstance(sample, dict) and "input_ids" in sample:
            out = {"input_ids": list(sample["input_ids"]), "label_ids": list(sample.get("label_ids", sample["input_ids"]))}
            out["mm"] = {k: sample[k] for k in MM_KEYS if sample.get(k) is not None}
            return out
        pr = self._process(sample)
        return {"input_ids": pr["input_ids"], "label_ids": list(pr["input_ids"]), "mm": pr["mm"]}


BaseDataPacker.register(["qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe", "internvl", "llava", "gemma3"],
                        HFVLMDataPacker)


class OpenVLADataPacker(HFVLMDataPacker):
    """Robot-manipulation records for the OpenVLA family (the role of
    cosmos_rl/policy/model/vla/processing_utils.py and the prismatic processors). A record is
    ``{"instruction_ids": [...], "image": [3 * featurizers, S, S], "actions": [[...] * action_dim] * chunk,
    "proprio": [...] (optional), "unnorm_key": name (optional)}``; already processed samples (``input_ids`` with the
    placeholders in place) pass through. The prompt is ``bos + placeholders for the patches (+ state) + instruction``;
    for supervised training the actions follow as tokens of the last ``n_action_bins`` vocabulary ids and only they
    carry labels."""

    def setup(self, config, tokenizer=None, processor=None, *a, **kw):
        super().setup(config, tokenizer, processor)
        from ..models import hf_io
        from ..models.openvla import ActionBins, OpenVLAArgs
        args = OpenVLAArgs.from_hf_config(hf_io.load_hf_config(config.policy.model_name_or_path,
                                                               config.custom.get("model_config")))
        self.vla_args = args
        g = args.towers[0].image_size // args.towers[0].patch_size
        self.n_patches = g * g
        self.bins = ActionBins(args.vocab_size - args.pad_to_multiple_of, args.n_action_bins, args.norm_stats)

    def _process(self, sample) -> Dict[str, Any]:
        if isinstance(sample, dict) and "prompt" in sample and "input_ids" not in sample and "instruction_ids" not in sample:
            sample = sample["prompt"]
        if isinstance(sample, dict) and "instruction_ids" in sample:
            from ..models.openvla import build_prompt
            a = self.vla_args
            has_state = bool(a.proprio_dim) and sample.get("proprio") is not None
            ids = build_prompt(sample["instruction_ids"], self.n_patches, a.image_token_id, extra=int(has_state))
            mm = {"pixel_values": torch.as_tensor(sample["image"], dtype=torch.float32)[None]}
            if has_state:
                mm["proprio"] = torch.as_tensor(sample["proprio"], dtype=torch.float32)[None]
            return {"input_ids": ids, "mm": mm}
        return super()._process(sample)

    def action_tokens(self, sample) -> List[int]:
        acts = torch.as_tensor(sample["actions"], dtype=torch.float32)
        return self.bins.encode(acts, sample.get("unnorm_key")).reshape(-1).tolist()

    def sft_process_sample(self, sample):
        if isinstance(sample, dict) and "instruction_ids" in sample:
            pr = self._process(sample)
            act = self.action_tokens(sample)
            return {"input_ids": pr["input_ids"] + act, "label_ids": [-100] * len(pr["input_ids"]) + act, "mm": pr["mm"]}
        return super().sft_process_sample(sample)


BaseDataPacker.register(["openvla"], OpenVLADataPacker)


DataPacker = BaseDataPacker       # the name language-model packers of user scripts derive from


class TensorDataPacker(BaseDataPacker):
    """Packer for rollouts that are tensor trajectories instead of text (control tasks, simulators; the reference's
    cosmos_rl/dispatcher/data/packer/tensor_data_packer.py:69). Everything passes through: the data set's sample is the
    rollout engine's input, the engine's trajectory dict is the trainer's per-episode payload, and a batch is the list
    of those dicts (episodes have different lengths; the trainer knows how to pad or pack for its algorithm). No
    tokenizer is needed. Subclasses override single hooks, e.g. ``get_rollout_input`` to parse initial conditions, or
    ``get_rollout_output`` / ``get_policy_input`` to swap tensors for references to a transport."""

    def get_rollout_input(self, item: Any, **kw) -> Any:
        return item

    def get_rollout_output(self, items: List[Any], completed_conversations=None, logprobs=None, token_ids=None, **kw):
        return items

    def get_policy_input(self, sample: Any, rollout_output: Any, n_ignore_prefix_tokens: int = 0, **kw) -> Any:
        return rollout_output

    def policy_compute_max_len(self, processed: List[Any]) -> int:
        return max((int(p.get("episode_length", 0)) if isinstance(p, dict) else 0 for p in processed), default=0)

    def policy_collate_fn(self, processed: List[Any], computed_max_len: int = 0) -> List[Any]:
        return list(processed)

    def batch_size(self, batch) -> int:
        return len(batch)

    def slice_batch(self, batch, start: int, end: int):
        return batch[start:end]


class TrajectoryPacker:
    """Contract of packers whose rollouts hold several trainable transitions under one envelope (one prompt index, one
    group-relative advantage): ``num_transitions`` and ``iter_transitions`` are the packer's to write; chunks and
    batches of rollouts have defaults. The methods describe STRUCTURE only: they never scale advantages or weights
    (loss aggregation is the trainer's), and ``num_transitions(r) == len(list(iter_transitions(r)))``
    (cosmos_rl/dispatcher/data/packer/trajectory_packer.py:37; ``policy/trainer/trajectory_mixin.py`` consumes it)."""

    def num_transitions(self, rollout) -> int:
        raise NotImplementedError

    def iter_transitions(self, rollout):
        raise NotImplementedError

    def iter_chunks(self, rollout, chunk_size: int):
        """Consecutive runs of at most ``chunk_size`` transitions, in order."""
        chunk: List[Any] = []
        for t in self.iter_transitions(rollout):
            chunk.append(t)
            if len(chunk) == chunk_size:
                yield chunk
                chunk = []
        if chunk:
            yield chunk

    def iter_rollouts(self, rollouts):
        """Batches of rollouts in the order the trainer should walk them (default: one batch with all)."""
        yield list(rollouts)
