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
    context: str
    choices: tuple[str, ...]
    gold: int
    normalize_choices: bool = False


@dataclass
class EvalResult:
    task: str
    num_docs: int
    acc: float
    acc_norm: float | None = None

    def __str__(self) -> str:
        norm = "" if self.acc_norm is None else f" acc_norm={self.acc_norm:.4f}"
        return f"{self.task}: acc={self.acc:.4f}{norm} (n={self.num_docs})"


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
        self.harmony = None
        if harmony:
            from openai_harmony import HarmonyEncodingName, load_harmony_encoding

            self.harmony = load_harmony_encoding(HarmonyEncodingName.HARMONY_GPT_OSS)

    def _encode(self, context: str, continuation: str) -> tuple[list[int], list[int]]:
        if self.harmony is None:
            return [self.tokenizer.eos_token, *self.tokenizer.encode_ordinary(context)], self.tokenizer.encode_ordinary(continuation)
        from openai_harmony import Conversation, Message, Role

        conversation = Conversation.from_messages([Message.from_role_and_content(Role.USER, context)])
        prompt = self.harmony.render_conversation_for_completion(conversation, Role.ASSISTANT)
        prompt += self.harmony.encode("<|channel|>final<|message|>", allowed_special="all")
        return prompt, self.harmony.encode(continuation)

    def requests(self, docs: list[Doc]) -> list[tuple[int, int, list[int], int]]:
        out = []
        for d, doc in enumerate(docs):
            context = doc.context.rstrip()
            for c, choice in enumerate(doc.choices):
                ctx, cont = self._encode(context, doc.context[len(context):] + " " + choice)
                ctx = ctx[-(self.config.seq_len - len(cont)):]
                out.append((d, c, ctx + cont, len(ctx)))
        return out

    def score(self, docs: list[Doc]) -> list[list[float]]:
        reqs = self.requests(docs)
        width = max(len(ids) for _, _, ids, _ in reqs)
        scores = [[0.0] * len(doc.choices) for doc in docs]
        for start in range(0, len(reqs), self.batch_size):
            batch = reqs[start:start + self.batch_size]
            tokens = np.full((self.batch_size, width), self.tokenizer.pad_token, dtype=np.int64)
            targets = np.zeros((self.batch_size, width), dtype=np.int64)
            mask = np.zeros((self.batch_size, width), dtype=np.float32)
            for row, (_, _, ids, cont_start) in enumerate(batch):
                tokens[row, :len(ids)] = ids
                targets[row, :len(ids) - 1] = ids[1:]
                mask[row, cont_start - 1:len(ids) - 1] = 1.0   # continuation tokens only
            to = lambda a: torch.from_numpy(a).to(self.device)
            sums = continuation_logprob(self.model, self.config, to(tokens), to(targets), to(mask), self.rt).cpu().numpy()
            for row, (d, c, _, _) in enumerate(batch):
                scores[d][c] = float(sums[row])
        return scores


def evaluate(task: str, docs: list[Doc], scorer: Scorer) -> EvalResult:
    scores = scorer.score(docs)
    correct = [int(np.argmax(s)) == doc.gold for doc, s in zip(docs, scores)]
    acc_norm = None
    if docs[0].normalize_choices:
        normalized = [[s / len(choice) for s, choice in zip(ss, doc.choices)] for doc, ss in zip(docs, scores)]
        acc_norm = float(np.mean([int(np.argmax(s)) == doc.gold for doc, s in zip(docs, normalized)]))
    return EvalResult(task=task, num_docs=len(docs), acc=float(np.mean(correct)), acc_norm=acc_norm)


def few_shot_prefix(docs: list[Doc]) -> str:
    return "".join(f"{doc.context} {doc.choices[doc.gold]}\n\n" for doc in docs)


def select_limit(data, limit: int | None):
    return data if limit is None else data.select(range(min(limit, len(data))))
