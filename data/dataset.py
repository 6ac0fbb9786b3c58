"""Download pre-tokenized ClimbMix shards (ArrayRecord + ``.lengths.npy`` sidecars). The last shard is held out for validation.
``--synthetic N`` instead writes N iid-uniform tokens as local shards (for machines without network access)."""

from __future__ import annotations

import math
import sys
from dataclasses import dataclass
from pathlib import Path

import tyro

DATA_DIR = Path(__file__).resolve().parent
sys.path.insert(0, str(DATA_DIR.parent))

from lyra_b200.data import LENGTHS_SUFFIX  # noqa: E402

REPO = "Ibbyml/lyra-climbmix-30b"
REVISION = "346a345f0a0e2671da6ed8112b45f1197598ebb1"
SHARDS = 100
TOKENS_PER_SHARD = 300_000_000


@dataclass(frozen=True)
class Args:
    max_tokens: int | None = 21_000_000_000
    """Training tokens to download, rounded up to whole shards; None downloads every training shard."""
    val: bool = True
    """Also download the held-out validation shard."""
    synthetic: int | None = None
    """Write this many uniform random tokens to data/train (and a tenth as many to data/val) instead of downloading."""


def training_shards(max_tokens: int | None) -> range:
    count = SHARDS - 1 if max_tokens is None else math.ceil(max_tokens / TOKENS_PER_SHARD)
    if count >= SHARDS:
        raise SystemExit(f"error: the dataset has {(SHARDS - 1) * TOKENS_PER_SHARD:,} training tokens")
    return range(count)


def download(shards, directory: Path) -> None:
    from huggingface_hub import snapshot_download

    names = [f"shard-{index:05d}.array_record" for index in shards]
    patterns = names + [name + LENGTHS_SUFFIX for name in names]
    print(f"Downloading {len(names)} shard(s) to {directory}")
    snapshot_download(REPO, repo_type="dataset", revision=REVISION, local_dir=directory, allow_patterns=patterns)


def write_synthetic(tokens: int, directory: Path, seed: int = 0, vocab: int = 201088, doc_len: int = 1024) -> None:
    import numpy as np

    from lyra_b200.data import ShardWriter

    directory.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    writer = ShardWriter(directory, min(tokens, TOKENS_PER_SHARD))
    left = tokens
    while left > 0:
        n = min(doc_len, left)
        writer.write(rng.integers(0, vocab, size=n).tolist())
        left -= n
    writer.close()


def main(argv: list[str] | None = None) -> int:
    args = tyro.cli(Args, args=argv)
    if args.synthetic is not None:
        write_synthetic(args.synthetic, DATA_DIR / "train", seed=0)
        if args.val:
            write_synthetic(max(args.synthetic // 10, 1), DATA_DIR / "val", seed=1)
        return 0
    download(training_shards(args.max_tokens), DATA_DIR / "train")
    if args.val:
        download([SHARDS - 1], DATA_DIR / "val")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
