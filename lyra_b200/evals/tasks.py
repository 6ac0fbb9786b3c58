"""Task loaders with the reference's prompts and pinned dataset revisions (lyra/evals/{arc,hellaswag,mmlu}.py)."""

from __future__ import annotations

import random
import re
from collections import defaultdict

from lyra_b200.evals.common import Doc, few_shot_prefix, select_limit

ARC = ("allenai/ai2_arc", "210d026faf9955653af8916fad021475a3f00453")
HELLASWAG = ("Rowan/hellaswag", "218ec52e09a7e7462a5400043bb9a69a41d06b76")
MMLU = ("cais/mmlu", "c30699e8356da336a370243923dbaf21066bb9fe")
LETTERS = ("A", "B", "C", "D")


def _load(name, *args, **kw):
    from datasets import load_dataset

    return load_dataset(name, *args, **kw)


# ---- ARC: "Question: ...\nAnswer:" --------------------------------------------------------------------
def arc_doc(row: dict, prefix: str = "") -> Doc:
    gold = row["choices"]["label"].index(row["answerKey"])
    return Doc(context=f"{prefix}Question: {row['question'].strip()}\nAnswer:", choices=tuple(row["choices"]["text"]), gold=gold,
               normalize_choices=True)


def load_arc(*, subset: str, limit: int | None = None, num_fewshot: int = 0, fewshot_seed: int = 1234) -> list[Doc]:
    train = _load(ARC[0], subset, split="train", revision=ARC[1]) if num_fewshot else []
    rng = random.Random(fewshot_seed)
    docs = []
    for row in select_limit(_load(ARC[0], subset, split="test", revision=ARC[1]), limit):
        shots = [arc_doc(train[i]) for i in rng.sample(range(len(train)), num_fewshot)]
        docs.append(arc_doc(row, few_shot_prefix(shots)))
    return docs


# ---- HellaSwag ----------------------------------------------------------------------------------------
def hellaswag_clean(text: str) -> str:
    text = re.sub(r"\[.*?\]", "", text.strip().replace(" [title]", ". "))
    return text.replace("  ", " ")


def hellaswag_doc(row: dict, prefix: str = "") -> Doc:
    context = hellaswag_clean(f"{row['activity_label']}: {row['ctx_a']} {row['ctx_b'].capitalize()}")
    return Doc(context=f"{prefix}{context}", choices=tuple(hellaswag_clean(e) for e in row["endings"]), gold=int(row["label"]),
               normalize_choices=True)


def load_hellaswag(*, limit: int | None = None, num_fewshot: int = 0, fewshot_seed: int = 1234) -> list[Doc]:
    train = _load(HELLASWAG[0], split="train", revision=HELLASWAG[1]) if num_fewshot else []
    rng = random.Random(fewshot_seed)
    docs = []
    for row in select_limit(_load(HELLASWAG[0], split="validation", revision=HELLASWAG[1]), limit):
        shots = [hellaswag_doc(train[i]) for i in rng.sample(range(len(train)), num_fewshot)]
        docs.append(hellaswag_doc(row, few_shot_prefix(shots)))
    return docs


# ---- MMLU: header + lettered choices + "Answer:"; few-shots are the first dev rows of the subject -------
def mmlu_question(row: dict) -> str:
    choices = "".join(f"{letter}. {choice}\n" for letter, choice in zip(LETTERS, row["choices"]))
    return f"{row['question'].strip()}\n{choices}Answer:"


def load_mmlu(*, limit: int | None = None, num_fewshot: int = 0, fewshot_seed: int = 1234) -> list[Doc]:
    shots: dict[str, str] = defaultdict(str)
    if num_fewshot:
        counts: dict[str, int] = defaultdict(int)
        for row in _load(MMLU[0], "all", split="dev", revision=MMLU[1]):
            if counts[row["subject"]] < num_fewshot:
                counts[row["subject"]] += 1
                shots[row["subject"]] += f"{mmlu_question(row)} {LETTERS[int(row['answer'])]}\n\n"
    docs = []
    for row in select_limit(_load(MMLU[0], "all", split="test", revision=MMLU[1]), limit):
        header = f"The following are multiple choice questions (with answers) about {row['subject'].replace('_', ' ')}.\n\n"
        docs.append(Doc(context=header + shots[row["subject"]] + mmlu_question(row), choices=LETTERS, gold=int(row["answer"])))
    return docs
