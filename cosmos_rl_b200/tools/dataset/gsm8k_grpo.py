"""GRPO on GSM8K: `cosmos-rl --config <toml> cosmos_rl_b200/tools/dataset/gsm8k_grpo.py`
(cosmos_rl/tools/dataset/gsm8k_grpo.py). Rows have ``question`` and ``answer`` (worked solution ending in
``#### <number>``); the reward is 1 for the right final number plus a small bonus for the think/answer format."""
from __future__ import annotations

from cosmos_rl_b200.dispatcher.algo.reward import format_reward, gsm8k_reward
from cosmos_rl_b200.tools.dataset.common import PromptDataset, chat

SYSTEM = ("You are a careful math tutor. Think step by step inside <think></think>, then give the final number "
          "inside <answer></answer>.")


def reference_of(row) -> str:
    return str(row["answer"]).split("####")[-1].strip()


def gsm8k_dataset(rows=None, validation: bool = False) -> PromptDataset:
    return PromptDataset(lambda r: chat(SYSTEM, r["question"]), reference_of, rows, validation)


def reward_fn(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    return gsm8k_reward(to_be_evaluated, reference) + 0.1 * format_reward(to_be_evaluated)


if __name__ == "__main__":
    from cosmos_rl_b200.launcher.worker_entry import main
    main(dataset=gsm8k_dataset(), val_dataset=gsm8k_dataset(validation=True), reward_fns=[reward_fn],
         val_reward_fns=[gsm8k_reward])
