"""Shared pieces of the dataset entry scripts: loading rows from local files (there is no hub access inside a
job: ``train.train_policy.dataset.name`` is a local folder or file of parquet / jsonl / json, or anything the
``datasets`` library can open offline) and a prompt dataset with the ``setup / __getitem__ / get_reference_answer``
contract."""
from __future__ import annotations

import glob
import json
import os
from typing import Any, Callable, Dict, List, Optional, Sequence, Union


def load_rows(name: str, subset: Optional[str] = None, split: Union[str, Sequence[str], None] = None) -> List[Dict[str, Any]]:
    splits = [split] if isinstance(split, str) else list(split or [])
    if os.path.isfile(name):
        files = [name]
    elif os.path.isdir(name):
        root = os.path.join(name, subset) if subset and os.path.isdir(os.path.join(name, subset)) else name
        files = sorted(f for ext in ("parquet", "jsonl", "json") for f in glob.glob(os.path.join(root, "**", f"*.{ext}"),
                                                                                     recursive=True))
        if splits:
            picked = [f for f in files if any(s in os.path.basename(f) or os.sep + s + os.sep in f for s in splits)]
            files = picked or files
    else:
        files = []
    rows: List[Dict[str, Any]] = []
    for f in files:
        if f.endswith(".parquet"):
            import pyarrow.parquet as pq
            rows.extend(pq.read_table(f).to_pylist())
        elif f.endswith(".jsonl"):
            with open(f) as fh:
                rows.extend(json.loads(ln) for ln in fh if ln.strip())
        else:
            with open(f) as fh:
                data = json.load(fh)
            rows.extend(data if isinstance(data, list) else data.get("data", []))
    if rows:
        return rows
    from datasets import load_dataset          # offline cache or a dataset script on disk
    ds = load_dataset(name, subset)
    for s in (splits or list(ds.keys())):
        rows.extend(dict(r) for r in ds[s])
    return rows


class PromptDataset:
    """Rows -> (conversation or prompt string, reference answer)."""

    def __init__(self, to_prompt: Callable[[Dict[str, Any]], Any], to_answer: Callable[[Dict[str, Any]], Any],
                 rows: Optional[List[Dict[str, Any]]] = None, validation: bool = False):
        self.to_prompt, self.to_answer, self.rows, self.validation = to_prompt, to_answer, rows, validation

    def setup(self, config, tokenizer=None, *a, **kw):
        self.config, self.tokenizer = config, tokenizer
        if self.rows is None:
            d = config.validation.dataset if self.validation else config.train.train_policy.dataset
            self.rows = load_rows(d.name, d.subset, d.split)
            if self.validation and getattr(d, "test_size", None):
                n = d.test_size if isinstance(d.test_size, int) else int(len(self.rows) * d.test_size)
                self.rows = self.rows[-n:]

    def __len__(self) -> int:
        return len(self.rows or [])

    def __getitem__(self, idx: int):
        return self.to_prompt(self.rows[idx])

    def get_reference_answer(self, idx: int):
        return self.to_answer(self.rows[idx])


def chat(system: Optional[str], user: str) -> List[Dict[str, str]]:
    msgs = [{"role": "system", "content": system}] if system else []
    return msgs + [{"role": "user", "content": user}]


def config_dataset(config, validation: bool = False) -> Optional["PromptDataset"]:
    """The dataset a job gets when its entry script passes none: rows of ``dataset.name`` read through the column
    names of the training policy (cosmos_rl/dispatcher/data/__init__.py:83-170 builds the same from
    ``prompt_column_name`` / ``response_column_name``; the SFT workers read ``conversation_column_name``,
    cosmos_rl/policy/worker/sft_worker.py:60-110). ``system_prompt`` is put in front of string prompts and of
    conversations that do not start with a system turn. Returns None when the config names no dataset."""
    tp = config.train.train_policy
    d = config.validation.dataset if validation else tp.dataset
    if not getattr(d, "name", ""):
        return None
    system = getattr(tp, "system_prompt", "") or ""

    def with_system(conv):
        if system and not (conv and isinstance(conv[0], dict) and conv[0].get("role") == "system"):
            return [{"role": "system", "content": system}] + list(conv)
        return list(conv)

    if tp.type == "sft":
        col = tp.conversation_column_name

        def to_prompt(row):
            v = row[col]
            return with_system(v) if isinstance(v, list) and v and isinstance(v[0], dict) else v

        return PromptDataset(to_prompt, lambda row: None, validation=validation)
    pcol, rcol = tp.prompt_column_name, tp.response_column_name
    if not pcol:
        raise ValueError("train.train_policy.prompt_column_name is needed to read prompts from dataset.name")

    def to_prompt(row):
        v = row[pcol]
        if isinstance(v, list) and v and isinstance(v[0], dict):
            return with_system(v)
        return chat(system, v) if system else v

    return PromptDataset(to_prompt, lambda row: row.get(rcol) if rcol else None, validation=validation)
