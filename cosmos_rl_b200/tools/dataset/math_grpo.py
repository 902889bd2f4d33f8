"""GRPO on competition-math style data (rows with ``problem`` and ``solution`` or ``answer``): the final
``\\boxed{}`` answer is graded for mathematical equality, not string equality (cosmos_rl/tools/dataset/math_grpo.py)."""
from __future__ import annotations

from cosmos_rl_b200.dispatcher.algo.reward import _text, register_reward_fn
from cosmos_rl_b200.tools.dataset.common import PromptDataset, chat
from cosmos_rl_b200.tools.eval_utils import extract_boxed, math_equal

SYSTEM = "Solve the problem. Put the final answer in \\boxed{}."


def reference_of(row) -> str:
    if row.get("answer") not in (None, ""):
        return str(row["answer"])
    return extract_boxed(str(row.get("solution", ""))) or ""


@register_reward_fn("direct_math")
def direct_math_reward(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    pred = extract_boxed(_text(to_be_evaluated))
    if pred is None or reference in (None, ""):
        return 0.0
    return 1.0 if math_equal(pred, str(reference)) else 0.0


def math_dataset(rows=None, validation: bool = False) -> PromptDataset:
    return PromptDataset(lambda r: chat(SYSTEM, r.get("problem") or r.get("question")), reference_of, rows, validation)


if __name__ == "__main__":
    from cosmos_rl_b200.launcher.worker_entry import main
    main(dataset=math_dataset(), val_dataset=math_dataset(validation=True), reward_fns=[direct_math_reward])
