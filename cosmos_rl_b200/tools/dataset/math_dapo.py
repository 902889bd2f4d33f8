"""DAPO on DAPO-Math-17k style rows: ``prompt`` is already a conversation, the ground truth sits in
``reward_model.ground_truth``; reward +1 / -1 on the graded final answer, the soft overlong penalty is added by the
reward calculator when ``train.train_policy.overlong_reward`` is enabled, and groups whose rewards are all equal
are dropped by dynamic sampling (``variant = "dapo"``) (cosmos_rl/tools/dataset/math_dapo.py)."""
from __future__ import annotations

import re

from cosmos_rl_b200.dispatcher.algo.reward import _text
from cosmos_rl_b200.tools.dataset.common import PromptDataset
from cosmos_rl_b200.tools.eval_utils import extract_boxed, math_equal


def final_answer(text: str):
    m = re.findall(r"Answer:\s*([^\n]+)", text)
    return m[-1].strip() if m else extract_boxed(text)


def dapo_reward(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    pred = final_answer(_text(to_be_evaluated))
    return 1.0 if pred is not None and reference not in (None, "") and math_equal(pred, str(reference)) else -1.0


def dapo_dataset(rows=None, validation: bool = False) -> PromptDataset:
    return PromptDataset(lambda r: list(r["prompt"]), lambda r: str(r["reward_model"]["ground_truth"]), rows, validation)


if __name__ == "__main__":
    from cosmos_rl_b200.launcher.worker_entry import main
    main(dataset=dapo_dataset(), reward_fns=[dapo_reward], filter_reward_fns=[dapo_reward])
