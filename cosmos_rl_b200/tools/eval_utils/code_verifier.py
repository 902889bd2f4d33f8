"""Runs candidate programs against test cases in a child interpreter with CPU, memory and wall-clock limits
(cosmos_rl/tools/eval_utils/code_verifier_utils.py). Two test styles: stdin/stdout pairs and assert-style call
tests appended to the candidate."""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile
from typing import Dict, List, Optional, Sequence

_PRELUDE = """
import resource, sys
resource.setrlimit(resource.RLIMIT_AS, ({mem}, {mem}))
resource.setrlimit(resource.RLIMIT_CPU, ({cpu}, {cpu}))
sys.setrecursionlimit(10000)
"""


def extract_code(text: str) -> str:
    """Last fenced code block of a model response, or the text itself."""
    import re
    blocks = re.findall(r"```(?:python|py)?\n(.*?)```", text, re.DOTALL)
    return blocks[-1] if blocks else text


def _run(source: str, stdin: str, timeout_s: float, mem_mb: int) -> subprocess.CompletedProcess:
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "candidate.py")
        with open(path, "w") as f:
            f.write(_PRELUDE.format(mem=mem_mb << 20, cpu=int(timeout_s) + 1) + source)
        env = {"PATH": os.environ.get("PATH", ""), "PYTHONHASHSEED": "0"}
        return subprocess.run([sys.executable, "-I", path], input=stdin, capture_output=True, text=True,
                              timeout=timeout_s, cwd=d, env=env)


def run_code_tests(code: str, tests: Sequence[Dict[str, str]], timeout_s: float = 5.0, mem_mb: int = 1024,
                   stop_on_first_failure: bool = True) -> Dict[str, object]:
    """``tests``: ``{"input": ..., "output": ...}`` (program reads stdin, stdout is compared line-wise ignoring
    trailing blanks) or ``{"assert": "assert f(2) == 4"}`` (statement appended to the candidate). Returns pass
    fraction and per-test status (``pass`` / ``wrong`` / ``error`` / ``timeout``)."""
    status: List[str] = []
    for t in tests:
        try:
            if "assert" in t:
                r = _run(code + "\n" + t["assert"] + "\n", "", timeout_s, mem_mb)
                status.append("pass" if r.returncode == 0 else "error")
            else:
                r = _run(code, t.get("input", ""), timeout_s, mem_mb)
                if r.returncode != 0:
                    status.append("error")
                else:
                    norm = lambda s: [ln.rstrip() for ln in s.strip().splitlines()]
                    status.append("pass" if norm(r.stdout) == norm(t.get("output", "")) else "wrong")
        except subprocess.TimeoutExpired:
            status.append("timeout")
        if stop_on_first_failure and status[-1] != "pass":
            break
    n_pass = sum(s == "pass" for s in status)
    return {"pass_rate": n_pass / max(1, len(tests)), "all_passed": n_pass == len(tests), "status": status}
