"""Turns a text corpus into the token shards the loader reads.

Output format (the reference's, data/prepare_climbmix.py:34-63): ArrayRecord files of one record per document, each record
the document's little-endian int32 token ids followed by eos; a shard is cut after exactly ``tokens_per_shard`` tokens (a
document may straddle two shards); beside every shard a ``<shard>.lengths.npy`` with its record lengths.

The corpus is ClimbMix streamed from the Hugging Face hub by default (any dataset with a ``text`` column works); without
network access, ``--text-files`` tokenizes local ``.txt`` (one document per file) or ``.jsonl`` (one ``{"text": ...}`` object
per line) files instead.

    python data/prepare_climbmix.py --max-tokens 1000000000
    python data/prepare_climbmix.py --text-files corpus/*.jsonl --output data/train
"""

from __future__ import annotations

import json
import os
import sys
from collections.abc import Iterable, Iterator
from dataclasses import dataclass
from pathlib import Path

import tyro

DATA_DIR = Path(__file__).resolve().parent
sys.path.insert(0, str(DATA_DIR.parent))

from lyra_b200.data import ShardWriter  # noqa: E402
from lyra_b200.tokenizer import LyraTokenizer  # noqa: E402

TEXTS_PER_CALL = 4096   # documents handed to the tokenizer's thread pool at a time


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
    text_files: tuple[Path, ...] = ()
    """Local .txt / .jsonl files to tokenize instead of the hub dataset."""


def hub_texts(dataset: str) -> Iterator[list[str]]:
    from datasets import load_dataset

    stream = load_dataset(dataset, split="train", streaming=True)
    for rows in stream.iter(batch_size=TEXTS_PER_CALL):
        yield rows["text"]


def local_texts(files: Iterable[Path]) -> Iterator[list[str]]:
    pending: list[str] = []
    for path in files:
        if path.suffix == ".jsonl":
            with path.open() as lines:
                pending.extend(json.loads(line)["text"] for line in lines if line.strip())
        else:
            pending.append(path.read_text())
        while len(pending) >= TEXTS_PER_CALL:
            yield pending[:TEXTS_PER_CALL]
            del pending[:TEXTS_PER_CALL]
    if pending:
        yield pending


def tokenize_corpus(texts: Iterable[list[str]], tokenizer: LyraTokenizer, writer: ShardWriter, limit: int, num_threads: int) -> int:
    """Writes documents until ``limit`` tokens are on disk (the last document is cut to fit); returns the tokens written."""
    written = 0
    for group in texts:
        for ids in tokenizer.encode_ordinary_batch(group, num_threads=num_threads):
            ids.append(tokenizer.eos_token)
            if written + len(ids) > limit:
                del ids[limit - written:]
            writer.write(ids)
            written += len(ids)
            if written >= limit:
                return written
    return written


def main(argv: list[str] | None = None) -> int:
    args = tyro.cli(Args, args=argv)
    args.output.mkdir(parents=True, exist_ok=True)
    writer = ShardWriter(args.output, args.tokens_per_shard)
    source = local_texts(args.text_files) if args.text_files else hub_texts(args.dataset)
    try:
        total = tokenize_corpus(source, LyraTokenizer(), writer, args.max_tokens, args.num_threads)
    finally:
        writer.close()
    print(f"{total:,} tokens in {args.output}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
