"""Fetches the pre-tokenized ClimbMix token shards this framework trains on, or writes synthetic ones.

The published dataset (the one the reference's ``data/dataset.py`` downloads) is a Hugging Face dataset repository of 100
ArrayRecord shards of 300 M tokens each, every shard with a ``.lengths.npy`` sidecar; shards 0..98 are training data and
shard 99 is the held-out validation shard. This script resolves how many shards a token budget needs, asks the hub for
exactly those files at a pinned revision, and lays them out as ``data/train`` and ``data/val``, which is where
``scripts/train.py`` looks by default.

    python data/dataset.py --max-tokens 3000000000          # ten training shards + the validation shard
    python data/dataset.py --no-val --max-tokens None        # all 99 training shards, no validation shard
    python data/dataset.py --synthetic 50000000              # no network: iid-uniform tokens in the same on-disk format
"""

from __future__ import annotations

import sys
from dataclasses import dataclass
from pathlib import Path

import tyro

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

from lyra_b200.data import LENGTHS_SUFFIX, ShardWriter  # noqa: E402

HUB_DATASET = "Ibbyml/lyra-climbmix-30b"
HUB_REVISION = "346a345f0a0e2671da6ed8112b45f1197598ebb1"
N_SHARDS = 100                       # the last one is the validation shard
SHARD_TOKENS = 300_000_000


@dataclass(frozen=True)
class Args:
    max_tokens: int | None = 21_000_000_000
    """Training tokens wanted; whole shards are fetched, so the amount is rounded up. None: every training shard."""
    val: bool = True
    """Fetch the validation shard as well."""
    synthetic: int | None = None
    """Skip the hub: write this many uniform random tokens to data/train and a tenth as many to data/val."""


@dataclass(frozen=True)
class ShardSelection:
    """Which shard numbers go where."""

    train: tuple[int, ...]
    val: tuple[int, ...]

    @staticmethod
    def for_budget(max_tokens: int | None, with_val: bool) -> "ShardSelection":
        available = N_SHARDS - 1
        wanted = available if max_tokens is None else -(-int(max_tokens) // SHARD_TOKENS)
        if wanted > available:
            raise SystemExit(f"error: {max_tokens:,} tokens asked for, the dataset has {available * SHARD_TOKENS:,} training tokens")
        return ShardSelection(train=tuple(range(wanted)), val=(N_SHARDS - 1,) if with_val else ())


def shard_files(numbers) -> list[str]:
    """File names of the shards and of their length sidecars."""
    files = []
    for n in numbers:
        record = f"shard-{n:05d}.array_record"
        files += [record, record + LENGTHS_SUFFIX]
    return files


def fetch(numbers, target: Path) -> None:
    if not numbers:
        return
    from huggingface_hub import snapshot_download

    print(f"{target}: fetching shards {numbers[0]}..{numbers[-1]} ({len(numbers)} x {SHARD_TOKENS:,} tokens) of {HUB_DATASET}@{HUB_REVISION[:8]}")
    snapshot_download(HUB_DATASET, repo_type="dataset", revision=HUB_REVISION, local_dir=target, allow_patterns=shard_files(numbers))


def write_synthetic(tokens: int, target: Path, seed: int, vocab: int = 201088, doc_len: int = 1024) -> None:
    """``tokens`` iid-uniform token ids as documents of ``doc_len`` tokens, in the shard format the loader reads."""
    import numpy as np

    target.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    writer = ShardWriter(target, min(tokens, SHARD_TOKENS))
    try:
        for start in range(0, tokens, doc_len):
            writer.write(rng.integers(0, vocab, size=min(doc_len, tokens - start)).tolist())
    finally:
        writer.close()


def main(argv: list[str] | None = None) -> int:
    args = tyro.cli(Args, args=argv)
    train_dir, val_dir = HERE / "train", HERE / "val"
    if args.synthetic is not None:
        write_synthetic(args.synthetic, train_dir, seed=0)
        if args.val:
            write_synthetic(max(args.synthetic // 10, 1), val_dir, seed=1)
        return 0
    chosen = ShardSelection.for_budget(args.max_tokens, args.val)
    fetch(chosen.train, train_dir)
    fetch(chosen.val, val_dir)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
