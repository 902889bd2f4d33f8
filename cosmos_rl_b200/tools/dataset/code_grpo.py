"""GRPO on programming problems: rows with ``prompt`` (or ``question``) and ``tests`` (stdin/stdout pairs or
assert statements, as a list or a JSON string); the reward is the fraction of tests the last fenced code block of
the response passes in a sandboxed child interpreter (uses cosmos_rl/tools/eval_utils/code_verifier_utils.py's
counterpart)."""
from __future__ import annotations

import json

from cosmos_rl_b200.dispatcher.algo.reward import _text
from cosmos_rl_b200.tools.dataset.common import PromptDataset, chat
from cosmos_rl_b200.tools.eval_utils.code_verifier import extract_code, run_code_tests

SYSTEM = "Write a Python 3 solution. Reply with one fenced code block."


def code_reward(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    tests = json.loads(reference) if isinstance(reference, str) else (reference or [])
    if not tests:
        return 0.0
    return float(run_code_tests(extract_code(_text(to_be_evaluated)), tests, stop_on_first_failure=False)["pass_rate"])


def code_dataset(rows=None, validation: bool = False) -> PromptDataset:
    tests_of = lambda r: r["tests"] if isinstance(r["tests"], str) else json.dumps(r["tests"])
    return PromptDataset(lambda r: chat(SYSTEM, r.get("prompt") or r.get("question")), tests_of, rows, validation)


if __name__ == "__main__":
    from cosmos_rl_b200.launcher.worker_entry import main
    main(dataset=code_dataset(), reward_fns=[code_reward])
