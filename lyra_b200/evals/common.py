"""Loglikelihood multiple-choice harness (lyra/evals/common.py): one request per (document, choice), the context is
left-truncated so context + continuation fits ``seq_len``, requests are padded to one width and scored in fixed-size
batches; ``acc`` = argmax of summed continuation log-probabilities, ``acc_norm`` = argmax after dividing by the
choice's character length. Log-probabilities are taken over the real vocabulary in fp32; full ``[B, T, V]`` logits are
never materialised - the hidden states go through the output head a block of rows at a time."""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from lyra_b200.config import ModelConfig
from lyra_b200.model import ModelWeights, lm_head_weight, model_apply
from lyra_b200.tokenizer import LyraTokenizer


@dataclass(frozen=True)
class Doc:
    """One multiple-choice question: the text shown to the model, the candidate continuations, the index of the right one, and
    whether the task also reports length-normalised accuracy (field names as in lyra/evals/common.py)."""

    context: str
    choices: tuple[str, ...]
    gold: int
    normalize_choices: bool = False


@dataclass
class EvalResult:
    """Accuracy of one task; ``acc_norm`` only for tasks whose documents ask for it."""

    task: str
    num_docs: int
    acc: float
    acc_norm: float | None = None

    def __str__(self) -> str:
        parts = [f"acc={self.acc:.4f}"]
        if self.acc_norm is not None:
            parts.append(f"acc_norm={self.acc_norm:.4f}")
        return f"{self.task}: {' '.join(parts)} (n={self.num_docs})"


@torch.no_grad()
def continuation_logprob(model: ModelWeights, config: ModelConfig, tokens: torch.Tensor, targets: torch.Tensor, mask: torch.Tensor,
                         rt=None, row_block: int = 2048) -> torch.Tensor:
    """Sum over masked positions of ``log p(target | prefix)`` per row; ``tokens, targets, mask [B, T]``."""
    h, _, _ = model_apply(tokens, model, None, config, return_hidden_states=True, rt=rt)
    w = lm_head_weight(model.tok, config)
    if rt is not None:
        w = rt.materialize(w)
    w = w[: config.vocab_size].to(h.dtype)
    B, T, C = h.shape
    flat_h, flat_t = h.reshape(B * T, C), targets.reshape(B * T).long()
    out = torch.empty(B * T, dtype=torch.float32, device=h.device)
    for s in range(0, B * T, row_block):
        logits = (flat_h[s:s + row_block] @ w.t()).float()
        out[s:s + row_block] = logits.gather(1, flat_t[s:s + row_block, None])[:, 0] - torch.logsumexp(logits, dim=-1)
    return (out.view(B, T) * mask).sum(-1)


class Scorer:
    def __init__(self, model: ModelWeights, config: ModelConfig, *, batch_size: int = 8, harmony: bool = False, device="cpu", rt=None) -> None:
        self.model, self.config, self.batch_size, self.device, self.rt = model, config, batch_size, device, rt
        self.tokenizer = LyraTokenizer()
        self.harmony = self._harmony_encoding() if harmony else None

    @staticmethod
    def _harmony_encoding():
        import openai_harmony as oh

        return oh.load_harmony_encoding(oh.HarmonyEncodingName.HARMONY_GPT_OSS)

    def _encode(self, context: str, continuation: str) -> tuple[list[int], list[int]]:
        """Token ids of the context and of the continuation. Plain models see ``<eos> context``; GPT-OSS models see the context
        as a user message and answer in the ``final`` channel of an assistant message (lyra/evals/common.py:52-63)."""
        if self.harmony is not None:
            return self._encode_chat(context, continuation)
        tok = self.tokenizer
        return [tok.eos_token] + list(tok.encode_ordinary(context)), list(tok.encode_ordinary(continuation))

    def _encode_chat(self, context: str, continuation: str) -> tuple[list[int], list[int]]:
        import openai_harmony as oh

        enc = self.harmony
        asked = oh.Conversation.from_messages([oh.Message.from_role_and_content(oh.Role.USER, context)])
        opening = list(enc.render_conversation_for_completion(asked, oh.Role.ASSISTANT))
        opening += enc.encode("<|channel|>final<|message|>", allowed_special="all")
        return opening, list(enc.encode(continuation))

    def requests(self, docs: list[Doc]) -> list["Request"]:
        """One request per (document, choice). The continuation is the choice joined to the context by a single space (trailing
        whitespace of the context moves to the continuation side); the context loses tokens from the left until context +
        continuation fit the model's window."""
        window = self.config.seq_len
        reqs: list[Request] = []
        for d, doc in enumerate(docs):
            stem = doc.context.rstrip()
            tail = doc.context[len(stem):]
            for c, choice in enumerate(doc.choices):
                context_ids, continuation_ids = self._encode(stem, f"{tail} {choice}")
                keep = max(window - len(continuation_ids), 0)
                context_ids = context_ids[len(context_ids) - keep:] if keep else []
                reqs.append(Request(doc=d, choice=c, ids=context_ids + continuation_ids, scored_from=len(context_ids)))
        return reqs

    def score(self, docs: list[Doc]) -> list[list[float]]:
        """``scores[d][c]`` = summed log-probability of choice ``c``'s continuation tokens. There is no compiled step whose
        shape must stay fixed, so requests are visited longest first and every batch is padded only to its own longest row
        (rounded up to a multiple of 64); a short last batch is filled with padding rows."""
        reqs = sorted(self.requests(docs), key=lambda r: -len(r.ids))
        scores = [[0.0] * len(doc.choices) for doc in docs]
        rows = self.batch_size
        for first in range(0, len(reqs), rows):
            group = reqs[first:first + rows]
            width = min(-(-len(group[0].ids) // 64) * 64, max(self.config.seq_len, len(group[0].ids)))
            tokens = np.full((rows, width), self.tokenizer.pad_token, dtype=np.int64)
            targets = np.zeros((rows, width), dtype=np.int64)
            scored = np.zeros((rows, width), dtype=np.float32)
            for row, r in enumerate(group):
                n = len(r.ids)
                tokens[row, :n] = r.ids
                targets[row, :n - 1] = r.ids[1:]                     # position t predicts token t + 1
                scored[row, r.scored_from - 1:n - 1] = 1.0           # ... and only the continuation's tokens count
            on_device = [torch.from_numpy(a).to(self.device) for a in (tokens, targets, scored)]
            sums = continuation_logprob(self.model, self.config, *on_device, self.rt).tolist()
            for r, total in zip(group, sums):
                scores[r.doc][r.choice] = float(total)
        return scores


@dataclass(frozen=True)
class Request:
    doc: int
    choice: int
    ids: list[int]
    scored_from: int
    """Index in ``ids`` of the first continuation token."""


def evaluate(task: str, docs: list[Doc], scorer: Scorer) -> EvalResult:
    """``acc``: share of documents whose highest-scoring choice is the gold one; ``acc_norm`` (when the task's documents ask for
    it): the same after dividing every score by its choice's length in characters."""
    scores = scorer.score(docs)
    gold = np.array([doc.gold for doc in docs])

    def accuracy(per_doc) -> float:
        picked = np.array([int(np.argmax(row)) for row in per_doc])
        return float((picked == gold).mean())

    by_length = None
    if docs and docs[0].normalize_choices:
        by_length = accuracy([np.asarray(row) / np.array([len(choice) for choice in doc.choices]) for doc, row in zip(docs, scores)])
    return EvalResult(task=task, num_docs=len(docs), acc=accuracy(scores), acc_norm=by_length)


def few_shot_prefix(docs: list[Doc]) -> str:
    """The in-context examples in front of a question: each example's context, a space, its right answer, a blank line."""
    shown = [doc.context + " " + doc.choices[doc.gold] for doc in docs]
    return "\n\n".join(shown) + "\n\n" if shown else ""


def select_limit(data, limit: int | None):
    """The first ``limit`` rows of a Hugging Face dataset (all of them for None)."""
    if limit is None or limit >= len(data):
        return data
    return data.select(range(limit))
