"""DPO on vision-language preference data in the layout of MMPR (the reference trains Nemotron-VL on MMPR-v1.2 with a
``DPODataset`` of this shape, tests/test_mmpr_dpo_dataset.py): rows (jsonl / parquet, local) of
``{"image": "relative/path.jpg" | [...], "question": ..., "chosen": ..., "rejected": ...}``.

Each row becomes ``{"prompt": <conversation with the images>, "chosen": text, "rejected": text}``, which is what the
DPO trainer takes: the vision-language data packer turns the prompt into tokens plus pixel inputs once, and both
answers of the pair are scored against the same images. Rows whose answers are identical carry no preference and are
skipped; ``max_pairs`` bounds the set.

`cosmos-rl --config <toml> cosmos_rl_b200/tools/dataset/vlm_dpo.py` with ``train_policy.type = "sft"`` and
``trainer_type = "dpo"``."""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional

from cosmos_rl_b200.tools.dataset.common import load_rows
from cosmos_rl_b200.tools.dataset.hf_vlm import to_conversation


def to_pair(row: Dict[str, Any], root: str) -> Optional[Dict[str, Any]]:
    chosen, rejected = row.get("chosen"), row.get("rejected")
    if isinstance(chosen, list):                      # conversation-form answers: the assistant text
        chosen = " ".join(str(m.get("content", "")) for m in chosen if m.get("role", "assistant") == "assistant")
    if isinstance(rejected, list):
        rejected = " ".join(str(m.get("content", "")) for m in rejected if m.get("role", "assistant") == "assistant")
    if not chosen or not rejected or str(chosen).strip() == str(rejected).strip():
        return None
    return {"prompt": to_conversation(row, root, with_answer=False), "chosen": str(chosen), "rejected": str(rejected)}


class VLMPreferenceDataset:
    def __init__(self, rows: Optional[List[Dict[str, Any]]] = None, root: str = "", max_pairs: int = 0):
        self.rows, self.root, self.max_pairs = rows, root, max_pairs
        self.pairs: List[Dict[str, Any]] = []
        self.n_skipped = 0
        if rows is not None:
            self._build()

    def _build(self) -> None:
        self.pairs, self.n_skipped = [], 0
        for r in self.rows or []:
            p = to_pair(r, self.root)
            if p is None:
                self.n_skipped += 1
                continue
            self.pairs.append(p)
            if self.max_pairs and len(self.pairs) >= self.max_pairs:
                break

    def setup(self, config, tokenizer=None, *a, **kw):
        if self.rows is None:
            d = config.train.train_policy.dataset
            self.rows = load_rows(d.name, d.subset, d.split)
            self.root = d.name if os.path.isdir(d.name) else os.path.dirname(d.name)
            self._build()

    def __len__(self) -> int:
        return len(self.pairs)

    def __getitem__(self, i: int) -> Dict[str, Any]:
        return self.pairs[i]


if __name__ == "__main__":
    from cosmos_rl_b200.launcher.worker_entry import main
    main(dataset=VLMPreferenceDataset())
