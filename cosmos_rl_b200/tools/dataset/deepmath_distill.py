"""On-policy distillation on DeepMath-style rows (``question`` / ``final_answer``; cosmos_rl/tools/dataset/deepmath_distill.py):
the student generates, a teacher replica scores every completion token (``[distillation]`` of the job file) and the
trainer minimises the reverse KL against it; the math grader only reports accuracy alongside.

Prompts are rendered by hand in the ChatML wording of the Qwen3 family with the assistant turn opened on ``<think>``,
as the paper's recipe does (a tokenizer's chat template would close the turn or add an empty think block): the string
goes to the rollout engine as it is."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

from cosmos_rl_b200.dispatcher.algo.reward import _text
from cosmos_rl_b200.tools.dataset.common import PromptDataset
from cosmos_rl_b200.tools.eval_utils import extract_boxed, math_equal


def render_chatml(messages: List[Dict[str, str]], open_thinking: bool = True) -> str:
    """``<|im_start|>role\\ncontent<|im_end|>`` per message; earlier assistant turns lose their thinking section (the
    family only ever saw its own current-turn thinking); the LAST message, when it is an empty assistant message,
    becomes the open generation prompt (``<|im_start|>assistant\\n<think>\\n``)."""
    out = []
    for i, m in enumerate(messages):
        role, content = m["role"], str(m.get("content", ""))
        last = i == len(messages) - 1
        if role == "assistant" and last and content == "":
            out.append("<|im_start|>assistant\n" + ("<think>\n" if open_thinking else ""))
            continue
        if role == "assistant" and "</think>" in content:
            content = content.split("</think>", 1)[1].lstrip()
        out.append(f"<|im_start|>{role}\n{content}<|im_end|>")
    return "\n".join(out)


def deepmath_prompt(row: Dict[str, Any]) -> str:
    return render_chatml([{"role": "user", "content": row.get("question") or row.get("problem")},
                          {"role": "assistant", "content": ""}])


def deepmath_reference(row: Dict[str, Any]) -> str:
    for k in ("final_answer", "answer"):
        if row.get(k) not in (None, ""):
            return str(row[k])
    return extract_boxed(str(row.get("solution", ""))) or ""


def deepmath_accuracy(to_be_evaluated, reference=None, prompt=None, **kw) -> float:
    """1.0 when the last ``\\boxed{}`` of the completion equals the reference mathematically (reported, not optimised:
    the distillation objective comes from the teacher's log-probs)."""
    pred = extract_boxed(_text(to_be_evaluated))
    if pred is None or reference in (None, ""):
        return 0.0
    return 1.0 if math_equal(pred, str(reference)) else 0.0


def deepmath_dataset(rows: Optional[List[Dict[str, Any]]] = None, validation: bool = False) -> PromptDataset:
    return PromptDataset(deepmath_prompt, deepmath_reference, rows, validation)


if __name__ == "__main__":
    from cosmos_rl_b200.launcher.worker_entry import main
    main(dataset=deepmath_dataset(), val_dataset=deepmath_dataset(validation=True), reward_fns=[deepmath_accuracy])
