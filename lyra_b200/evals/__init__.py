from functools import partial

from lyra_b200.evals import tasks
from lyra_b200.evals.common import Doc, EvalResult, Scorer, evaluate

TASKS = {
    "mmlu": tasks.load_mmlu,
    "arc-challenge": partial(tasks.load_arc, subset="ARC-Challenge"),
    "arc-easy": partial(tasks.load_arc, subset="ARC-Easy"),
    "hellaswag": tasks.load_hellaswag,
}

__all__ = ["TASKS", "Doc", "EvalResult", "Scorer", "evaluate"]
