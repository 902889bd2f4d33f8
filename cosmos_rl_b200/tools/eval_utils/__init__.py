"""Answer graders used by reward functions and offline evaluation (cosmos_rl/tools/eval_utils/)."""
from .code_verifier import run_code_tests  # noqa: F401
from .grader import extract_boxed, math_equal, normalize_answer  # noqa: F401
