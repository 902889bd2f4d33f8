"""SFT / GRPO on vision-language data (cosmos_rl/tools/dataset/hf_vlm_sft.py, hf_vlm_grpo.py).

Rows (jsonl / parquet, local): ``{"image": "relative/path.jpg" | ["a.jpg", ...], "question": ..., "answer": ...}`` or a
ready ``"conversation"`` in the processor's chat format. Images are opened with PIL relative to the data folder and
handed to the model's processor by the vision-language data packer; the policy model is any family the transformers
wrapper serves (``policy.model_name_or_path`` = a local HF folder that contains the processor files).

`cosmos-rl --config <toml> cosmos_rl_b200/tools/dataset/hf_vlm.py` launches SFT or GRPO by ``train.train_policy.type``."""
from __future__ import annotations

import os
from typing import Any, Dict, List

from cosmos_rl_b200.dispatcher.algo.reward import boxed_math_reward, single_choice_reward
from cosmos_rl_b200.tools.dataset.common import load_rows


def to_conversation(row: Dict[str, Any], root: str, with_answer: bool) -> List[Dict[str, Any]]:
    if "conversation" in row:
        conv = list(row["conversation"])
        return conv if with_answer else [m for m in conv if m.get("role") != "assistant"]
    images = row.get("image") or row.get("images") or []
    images = [images] if isinstance(images, str) else list(images)
    content: List[Dict[str, Any]] = [{"type": "image", "image": os.path.join(root, p)} for p in images]
    content.append({"type": "text", "text": str(row.get("question") or row.get("prompt") or "")})
    conv = [{"role": "user", "content": content}]
    if with_answer:
        conv.append({"role": "assistant", "content": [{"type": "text", "text": str(row.get("answer", ""))}]})
    return conv


class VLMDataset:
    def __init__(self, sft: bool, rows=None, root: str = ""):
        self.sft, self.rows, self.root = sft, rows, root

    def setup(self, config, tokenizer=None, *a, **kw):
        d = config.train.train_policy.dataset
        if self.rows is None:
            self.rows = load_rows(d.name, d.subset, d.split)
            self.root = d.name if os.path.isdir(d.name) else os.path.dirname(d.name)

    def __len__(self) -> int:
        return len(self.rows or [])

    def __getitem__(self, i: int):
        return to_conversation(self.rows[i], self.root, with_answer=self.sft)

    def get_reference_answer(self, i: int):
        return str(self.rows[i].get("answer", ""))


def vlm_reward(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    """Multiple-choice letters or boxed numbers, whichever the reference looks like."""
    ref = str(reference or "").strip()
    if len(ref) == 1 and ref.isalpha():
        return single_choice_reward(to_be_evaluated, ref)
    return boxed_math_reward(to_be_evaluated, ref)


if __name__ == "__main__":
    from cosmos_rl_b200.config import Config, load_toml
    from cosmos_rl_b200.launcher.worker_entry import main
    cfg_path = os.environ.get("COSMOS_CONFIG")
    sft = bool(cfg_path) and Config.from_dict(load_toml(cfg_path)).train.train_policy.type == "sft"
    if sft:
        main(dataset=VLMDataset(True))
    else:
        main(dataset=VLMDataset(False), reward_fns=[vlm_reward])
