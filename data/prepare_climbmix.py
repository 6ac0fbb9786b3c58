"""Tokenize ClimbMix (or any Hugging Face dataset with a ``text`` column) into ArrayRecord shards in the format the
loader reads: one record per document of little-endian int32 tokens ending in eos, ``tokens_per_shard`` tokens per shard,
and a ``<shard>.lengths.npy`` sidecar."""

from __future__ import annotations

import os
import sys
from collections.abc import Iterator
from dataclasses import dataclass
from pathlib import Path

import tyro

DATA_DIR = Path(__file__).resolve().parent
sys.path.insert(0, str(DATA_DIR.parent))

from lyra_b200.data import ShardWriter  # noqa: E402
from lyra_b200.tokenizer import LyraTokenizer  # noqa: E402


@dataclass(frozen=True)
class Args:
    output: Path = DATA_DIR / "train"
    """Shard directory."""
    max_tokens: int = 30_000_000_000
    """Tokens to write."""
    dataset: str = "karpathy/climbmix-400b-shuffle"
    """Hugging Face dataset with a text column."""
    tokens_per_shard: int = 300_000_000
    """Tokens per shard."""
    num_threads: int = os.cpu_count() or 1
    """Tokenizer threads."""


def documents(dataset: str, tokenizer: LyraTokenizer, num_threads: int) -> Iterator[list[int]]:
    from datasets import load_dataset

    for batch in load_dataset(dataset, split="train", streaming=True).iter(batch_size=4096):
        for tokens in tokenizer.encode_ordinary_batch(batch["text"], num_threads=num_threads):
            yield [*tokens, tokenizer.eos_token]


def main(argv: list[str] | None = None) -> int:
    args = tyro.cli(Args, args=argv)
    args.output.mkdir(parents=True, exist_ok=True)
    tokenizer = LyraTokenizer()
    writer = ShardWriter(args.output, args.tokens_per_shard)
    remaining = args.max_tokens
    for tokens in documents(args.dataset, tokenizer, args.num_threads):
        tokens = tokens[:remaining]
        writer.write(tokens)
        remaining -= len(tokens)
        if not remaining:
            break
    writer.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
