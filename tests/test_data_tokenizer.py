import numpy as np
import pytest

from lyra_b200.data import DataLoader, DataLoaderConfig, IndexSampler, ShardWriter, TokenBlocks
from lyra_b200.tokenizer import PADDED_VOCAB_SIZE, LyraTokenizer


def _write(tmp_path, docs, per_shard):
    w = ShardWriter(tmp_path, per_shard)
    for d in docs:
        w.write(list(d))
    w.close()


def test_shards_read_back_as_one_token_stream_with_shifted_labels(tmp_path):
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, 200000, size=rng.integers(1, 90)).tolist() for _ in range(40)]
    stream = np.concatenate([np.asarray(d) for d in docs])
    _write(tmp_path, docs, 700)
    shards = sorted(tmp_path.glob("*.array_record"))
    assert len(shards) == -(-len(stream) // 700)
    assert sum(int(np.load(str(s) + ".lengths.npy").sum()) for s in shards) == len(stream)
    loader = DataLoader(tmp_path, 2, 16, config=DataLoaderConfig(worker_count=2), quiet=True)
    assert loader.token_count == len(stream) and loader.block_count == (len(stream) - 1) // 32
    for i, (x, y) in enumerate(loader):
        assert np.array_equal(x.reshape(-1), stream[i * 32:(i + 1) * 32]) and np.array_equal(y.reshape(-1), stream[i * 32 + 1:(i + 1) * 32 + 1])
    assert i == loader.block_count - 1
    with pytest.raises(ValueError, match="Download more data"):
        loader.check_steps(loader.block_count + 1, 1)


def test_records_larger_than_a_container_block_survive(tmp_path):
    big = np.random.default_rng(1).integers(0, 200000, size=50000)
    _write(tmp_path, [big, [1, 2, 3]], 10**9)
    t = TokenBlocks(tmp_path, 1, 8)
    assert np.array_equal(t.read(0, 50003), np.concatenate([big, [1, 2, 3]]))


def test_loader_state_resumes_and_shuffle_is_seeded(tmp_path):
    np.save(tmp_path / "t.npy", np.arange(5000, dtype="<i4"))
    cfg = DataLoaderConfig(shuffle=True, seed=3, num_epochs=2, worker_count=1)
    a = DataLoader(tmp_path / "t.npy", 2, 16, config=cfg, quiet=True)
    first = [next(a)[0].copy() for _ in range(5)]
    state = a.get_state()
    rest = [next(a)[0].copy() for _ in range(4)]
    b = DataLoader(tmp_path / "t.npy", 2, 16, config=cfg, quiet=True)
    b.set_state(state)
    assert all(np.array_equal(x, next(b)[0]) for x in rest)
    c = DataLoader(tmp_path / "t.npy", 2, 16, config=cfg, quiet=True)
    assert all(np.array_equal(x, next(c)[0]) for x in first)
    assert not np.array_equal(first[0].reshape(-1), np.arange(32))  # shuffled


def test_sampler_shards_blocks_across_ranks_without_overlap():
    parts = [IndexSampler(103, shuffle=True, seed=1, num_epochs=1, shard_index=r, shard_count=4) for r in range(4)]
    seen = [[s.index_at(p) for p in range(s.per_epoch)] for s in parts]
    flat = [i for part in seen for i in part]
    assert len(flat) == len(set(flat)) == 100 and parts[0].index_at(25) is None


@pytest.fixture(scope="module")
def tokenizer():
    return LyraTokenizer()


@pytest.mark.parametrize("text", ["hello world", "def f(x): return x * 2  # code-ish\n", "unicode: café — naïve — 日本語"])
def test_encode_decode_roundtrip(tokenizer, text):
    assert tokenizer.decode(tokenizer.encode_ordinary(text)) == text


def test_special_tokens_and_batch(tokenizer):
    assert tokenizer.eos_token == 199999 and tokenizer.pad_token == 200004 and tokenizer.pad_token < PADDED_VOCAB_SIZE
    assert "<|reserved_200018|>" not in tokenizer._special_tokens
    assert tokenizer.decode([200018]) == "<|endofprompt|>"
    texts = ["alpha", "beta gamma", "delta"]
    assert tokenizer.encode_ordinary_batch(texts) == [tokenizer.encode_ordinary(t) for t in texts]
    ids = tokenizer.encode_ordinary("tokenization")
    assert b"".join(tokenizer.decode_single_token_bytes(i) for i in ids).decode() == "tokenization"


def test_prepare_script_tokenizes_local_files_up_to_the_limit(tmp_path):
    import importlib.util
    import json
    import sys
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("prepare_climbmix", Path(__file__).resolve().parents[1] / "data" / "prepare_climbmix.py")
    prep = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = prep
    spec.loader.exec_module(prep)
    (tmp_path / "a.txt").write_text("the quick brown fox jumps over the lazy dog " * 4)
    (tmp_path / "b.jsonl").write_text("\n".join(json.dumps({"text": f"document number {i} " * 30}) for i in range(5)))
    out = tmp_path / "shards"
    assert prep.main(["--text-files", str(tmp_path / "a.txt"), str(tmp_path / "b.jsonl"), "--output", str(out), "--max-tokens", "700",
                      "--tokens-per-shard", "256", "--num-threads", "1"]) == 0
    shards = sorted(out.glob("*.array_record"))
    lengths = [np.load(str(s) + ".lengths.npy") for s in shards]
    assert sum(int(n.sum()) for n in lengths) == 700 and [int(n.sum()) for n in lengths] == [256, 256, 188]
    tok = LyraTokenizer()
    stream = TokenBlocks(out, 1, 8).read(0, 700)
    first = tok.encode_ordinary("the quick brown fox jumps over the lazy dog " * 4)
    assert stream[:len(first)].tolist() == first and stream[len(first)] == tok.eos_token


def test_dataset_script_selects_whole_shards_and_writes_synthetic_ones_the_loader_reads(tmp_path):
    import importlib.util
    import sys
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("dataset_script", Path(__file__).resolve().parents[1] / "data" / "dataset.py")
    ds = importlib.util.module_from_spec(spec)
    sys.modules["dataset_script"] = ds                   # dataclasses look their module up while the class is built
    spec.loader.exec_module(ds)

    few = ds.ShardSelection.for_budget(2 * ds.SHARD_TOKENS + 1, with_val=True)        # budgets round up to whole shards
    assert few.train == (0, 1, 2) and few.val == (ds.N_SHARDS - 1,)
    everything = ds.ShardSelection.for_budget(None, with_val=False)
    assert everything.train == tuple(range(ds.N_SHARDS - 1)) and everything.val == ()
    with pytest.raises(SystemExit):
        ds.ShardSelection.for_budget(ds.N_SHARDS * ds.SHARD_TOKENS, with_val=True)    # more than the training shards hold
    assert ds.shard_files((7,)) == ["shard-00007.array_record", "shard-00007.array_record" + ds.LENGTHS_SUFFIX]

    ds.write_synthetic(4000, tmp_path / "train", seed=3, vocab=97, doc_len=300)
    blocks = TokenBlocks(tmp_path / "train", 2, 16)
    assert len(blocks) == (4000 - 1) // 32
    first = blocks[0]
    assert first["input_ids"].shape == (2, 16) and int(first["input_ids"].max()) < 97
    assert np.array_equal(first["input_ids"].reshape(-1)[1:], first["labels"].reshape(-1)[:-1])
