"""A tokenizer-shaped object for workloads without text (control tasks, simulators, tensor trajectories): data packers
and config checks that expect a tokenizer get the few attributes and methods they touch
(cosmos_rl/utils/no_op_tokenizer.py:60-165). This package runs such workloads with ``tokenizer=None``; the class exists
for entry scripts that register it as their tokenizer loader:

    register_tokenizer_loader(lambda path: path.endswith(".toml"), lambda path: NoOpTokenizer())
"""
from __future__ import annotations

from typing import Any, List

import torch


def _length_of(item: Any) -> int:
    """Number of "tokens" an item stands for: the episode length of a trajectory dict, else 1."""
    if isinstance(item, dict) and "episode_length" in item:
        v = item["episode_length"]
        try:
            return max(1, int(v.item() if hasattr(v, "item") else v))
        except (TypeError, ValueError):
            return 1
    return 1


class _Encoding(dict):
    def __init__(self, n: int):
        super().__init__(input_ids=torch.zeros((1, n), dtype=torch.long), attention_mask=torch.ones((1, n), dtype=torch.long))
        self.input_ids, self.attention_mask = self["input_ids"], self["attention_mask"]


class NoOpTokenizer:
    eos_token, bos_token, pad_token, unk_token = "<eos>", "<bos>", "<pad>", "<unk>"

    def __init__(self, vocab_size: int = 4, model_max_length: int = 1 << 30):
        self.eos_token_id, self.bos_token_id, self.pad_token_id, self.unk_token_id = 0, 1, 2, 3
        self.vocab_size, self.model_max_length = vocab_size, model_max_length
        self.chat_template = None

    def __len__(self) -> int:
        return self.vocab_size

    def encode(self, item: Any, **kw) -> List[int]:
        return [0] * _length_of(item)

    def decode(self, token_ids, **kw) -> str:
        return ""

    def batch_decode(self, batches, **kw) -> List[str]:
        try:
            return [""] * len(batches)
        except TypeError:
            return [""]

    def __call__(self, item: Any, **kw) -> _Encoding:
        return _Encoding(_length_of(item))

    def convert_tokens_to_ids(self, tokens) -> List[int]:
        return []

    def convert_ids_to_tokens(self, ids) -> List[str]:
        return []

    def apply_chat_template(self, conversation, tokenize: bool = False, **kw):
        return [0] if tokenize else ""
