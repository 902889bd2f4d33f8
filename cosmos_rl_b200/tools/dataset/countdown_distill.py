"""On-policy distillation on the Countdown task: reach ``target`` from ``nums`` with + - * /, each number used once
(cosmos_rl/tools/dataset/countdown_distill.py). Rows may come from files or are generated from a seed, so the job
runs without any download. The reward checks the equation in <answer></answer> with an arithmetic-only parser."""
from __future__ import annotations

import ast
import operator
import random
import re
from typing import List

from cosmos_rl_b200.dispatcher.algo.reward import _text
from cosmos_rl_b200.tools.dataset.common import PromptDataset, chat

_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv}


def synth_rows(n: int, seed: int = 0, k: int = 4) -> List[dict]:
    rng = random.Random(seed)
    rows = []
    for _ in range(n):
        nums = [rng.randint(1, 25) for _ in range(k)]
        val, order = float(nums[0]), list(nums)
        for x in nums[1:]:
            val = rng.choice([operator.add, operator.sub, operator.mul])(val, x)
        rows.append({"nums": order, "target": int(val)})
    return rows


def _eval(node, used: List[int]) -> float:
    if isinstance(node, ast.Expression):
        return _eval(node.body, used)
    if isinstance(node, ast.BinOp) and type(node.op) in _OPS:
        return _OPS[type(node.op)](_eval(node.left, used), _eval(node.right, used))
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
        return -_eval(node.operand, used)
    if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)):
        used.append(int(node.value))
        return float(node.value)
    raise ValueError("only numbers and + - * / are allowed")


def countdown_reward(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    """1.0 for a correct equation using exactly the given numbers, 0.1 for a well-formed but wrong one."""
    m = re.findall(r"<answer>(.*?)</answer>", _text(to_be_evaluated), re.DOTALL)
    if not m or not reference:
        return 0.0
    nums, target = reference["nums"], reference["target"]
    expr = m[-1].split("=")[0].strip()
    try:
        used: List[int] = []
        val = _eval(ast.parse(expr, mode="eval"), used)
    except (SyntaxError, ValueError, ZeroDivisionError):
        return 0.0
    return 1.0 if sorted(used) == sorted(nums) and abs(val - target) < 1e-6 else 0.1


def countdown_dataset(rows=None, n_synth: int = 4096, seed: int = 0) -> PromptDataset:
    rows = rows if rows is not None else synth_rows(n_synth, seed)
    ask = lambda r: chat(None, f"Using the numbers {r['nums']}, each exactly once, and + - * /, write an equation equal "
                               f"to {r['target']}. Think in <think></think>, answer in <answer></answer>.")
    return PromptDataset(ask, lambda r: {"nums": r["nums"], "target": r["target"]}, rows)


if __name__ == "__main__":
    from cosmos_rl_b200.launcher.worker_entry import main
    main(dataset=countdown_dataset(), val_dataset=countdown_dataset(n_synth=256, seed=1), reward_fns=[countdown_reward])
