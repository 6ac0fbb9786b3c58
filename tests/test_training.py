"""Train loop, checkpoints, resume, schedule, optimizer (CPU)."""

import json
from dataclasses import replace

import numpy as np
import pytest
import torch

from lyra_b200.data import DataLoaderConfig
from lyra_b200.model import ModelWeights
from lyra_b200.nn.checkpoints import checkpoint_run_config, checkpoint_steps, resolve_checkpoint
from lyra_b200.nn.params import tree_dict
from lyra_b200.training.optimizer import OptimizerState, newtonschulz, optimizer_step, wsd_lr
from lyra_b200.training.presets import TRAINING_PRESETS
from lyra_b200.training.state import init_train_state, load_train_state, save_checkpoint
from lyra_b200.training.train import TrainHooks, TrainingConfig, train
from tests.helpers import small_config, token_file


def _tcfg(tmp_path, **kw):
    base = dict(steps=6, batch_size=2, accumulation_steps=1, data_path=token_file(tmp_path / "tok.npy"), eval_data_path=tmp_path / "tok.npy",
                eval_every=3, eval_batches=1, checkpoint_every=3, checkpoint_path=tmp_path / "run", log_every=1, numerics_every=3,
                data_loader=DataLoaderConfig(worker_count=1))
    base.update(kw)
    return TrainingConfig(**base)


def _scales(config):
    return [wsd_lr(s, config)[2] for s in range(config.steps)]


def test_default_schedule_warms_up_then_cosine_decays():
    config = replace(TRAINING_PRESETS["train-dev"], steps=48)
    s = _scales(config)
    assert (config.warmup_steps, config.stable_steps, config.decay_steps) == (2, 0, 46)
    assert np.allclose(s[:3], [0.5, 1.0, 1.0]) and s[3] < 1.0 and abs(s[-1]) < 1e-6
    assert all(b <= a for a, b in zip(s[1:], s[2:]))
    assert replace(config, steps=954).warmup_steps == 29


def test_linear_wsd_schedule_from_cli():
    from scripts.train import Args, training_config

    config = training_config(Args(run="train-dev", steps=20, warmup_fraction=0.1, stable_fraction=0.8, decay_type="linear"))
    assert (config.warmup_steps, config.stable_steps, config.decay_steps) == (2, 16, 2)
    assert np.allclose(_scales(config), [0.5] + [1.0] * 18 + [0.0])
    one = replace(TRAINING_PRESETS["train-dev"], steps=1)
    assert np.isclose(wsd_lr(0, one)[2], 1.0) and np.isclose(wsd_lr(0, one)[0], one.adam_max_lr)


def test_cli_paths_expand_home_and_presets_save_where_serve_looks():
    from pathlib import Path

    from scripts.train import ROOT, Args, training_config

    config = training_config(Args(data="~/data", eval_data="~/val", out="~/checkpoints", resume="~/previous"))
    assert [str(p) for p in (config.data_path, config.eval_data_path, config.checkpoint_path, config.resume_from)] == [
        str(Path.home() / n) for n in ("data", "val", "checkpoints", "previous")]
    for variant in ("lyra-small", "lyra-medium", "lyra-large", "lyra-max"):
        assert training_config(Args(variant=variant)).checkpoint_path == ROOT / "chkpt" / variant


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    for shape in ((24, 64), (64, 24)):
        o = newtonschulz(torch.randn(*shape)).float()
        s = torch.linalg.svdvals(o)
        assert s.max() < 1.6 and s.min() > 0.3


def test_non_finite_gradient_skips_the_step():
    c = small_config()
    tcfg = TrainingConfig(steps=4, batch_size=2, accumulation_steps=1)
    w = ModelWeights.init(0, c)
    params = tree_dict(w)
    state = OptimizerState.init(w, ModelWeights.spec(c), tcfg)
    grads = {p: torch.randn_like(t) * 0.01 for p, t in params.items()}
    optimizer_step(params, grads, state, 0, tcfg)
    before = {p: t.clone() for p, t in params.items()}
    mom = {p: t.clone() for p, t in state.muon_moment.items()}
    grads["tok/emb"][0, 0] = float("inf")
    m = optimizer_step(params, grads, state, 1, tcfg)
    assert not bool(m["grad_is_finite"]) and int(state.adam_count) == 1
    assert all(torch.equal(before[p], params[p]) for p in params)
    assert all(torch.equal(mom[p], state.muon_moment[p]) for p in mom)


def test_checkpoint_round_trip_and_variant_mismatch(tmp_path):
    c = small_config()
    tcfg = TrainingConfig(steps=4, batch_size=2, accumulation_steps=1)
    state = init_train_state(ModelWeights.init(0, c), c, tcfg)
    for t in state.optimizer.muon_moment.values():
        t.copy_(torch.randn(t.shape).to(t.dtype))
    state.optimizer.adam_count += 3
    save_checkpoint(tmp_path, 7, state, b'{"position": 5}', {"resume_signature": {}}, keep=2)
    restored = load_train_state(tmp_path, c, tcfg)
    assert restored.step == 7 and restored.loader_state == b'{"position": 5}'
    a, b = tree_dict(state.params), tree_dict(restored.state.params)
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) and a[k].dtype == b[k].dtype for k in a)
    for name in ("muon_moment", "adam_mu", "adam_nu"):
        x, y = getattr(state.optimizer, name), getattr(restored.state.optimizer, name)
        assert x.keys() == y.keys() and all(torch.equal(x[k], y[k]) for k in x)
    assert int(restored.state.optimizer.adam_count) == 3
    with pytest.raises(ValueError, match="does not match the model config"):
        load_train_state(tmp_path, replace(c, use_sdpa_output_gate=True), tcfg)


def test_resolve_checkpoint_ignores_incomplete_directories(tmp_path):
    (tmp_path / "step_00000002").mkdir()
    (tmp_path / "step_00000002" / "_CHECKPOINT_METADATA").write_text("{}")
    (tmp_path / "step_00000005").mkdir()                                        # no metadata: unfinished
    (tmp_path / "step_00000009.orbax-checkpoint-tmp-0").mkdir()
    (tmp_path / "step_00000009.orbax-checkpoint-tmp-0" / "_CHECKPOINT_METADATA").write_text("{}")
    assert [p.name for p in checkpoint_steps(tmp_path)] == ["step_00000002"]
    assert resolve_checkpoint(tmp_path).name == "step_00000002"
    with pytest.raises(FileNotFoundError):
        resolve_checkpoint(tmp_path / "nothing")


def test_train_refuses_a_directory_with_checkpoints_and_rejects_changed_settings(tmp_path):
    c = small_config()
    tcfg = _tcfg(tmp_path, steps=3, eval_data_path=None, numerics_every=None)
    train(ModelWeights.init(0, c), c, tcfg, device="cpu")
    with pytest.raises(FileExistsError):
        train(ModelWeights.init(0, c), c, tcfg, device="cpu")
    with pytest.raises(ValueError, match="training settings differ"):
        train(None, c, replace(tcfg, resume_from=tmp_path / "run", muon_max_lr=1.0), device="cpu")
    with pytest.raises(ValueError, match="model settings differ"):
        train(None, replace(c, swiglu_limit=3.0), replace(tcfg, resume_from=tmp_path / "run"), device="cpu")


def test_interrupted_run_resumes_bit_exactly(tmp_path):
    c = small_config()
    full = train(ModelWeights.init(0, c), c, _tcfg(tmp_path), device="cpu")

    class Boom(TrainHooks):
        def before_step(self, step, *a):
            if step == 4:
                raise RuntimeError("interrupted")

    tcfg = _tcfg(tmp_path, checkpoint_path=tmp_path / "run2")
    with pytest.raises(RuntimeError, match="interrupted"):
        train(ModelWeights.init(0, c), c, tcfg, device="cpu", hooks=Boom())
    resumed = train(None, c, replace(tcfg, resume_from=tmp_path / "run2"), device="cpu")
    a, b = tree_dict(full.params), tree_dict(resumed.params)
    assert all(torch.equal(a[k], b[k]) for k in a)
    for name in ("muon_moment", "adam_mu", "adam_nu"):
        x, y = getattr(full.optimizer, name), getattr(resumed.optimizer, name)
        assert all(torch.equal(x[k], y[k]) for k in x)
    rows = [json.loads(l) for l in (tmp_path / "run2" / "metrics.jsonl").read_text().splitlines()]
    assert [r["step"] for r in rows if r["kind"] == "train"] == [1, 2, 3, 4, 5, 6]
    assert [r["step"] for r in rows if r["kind"] == "eval"] == [0, 3, 6]
    meta = checkpoint_run_config(resolve_checkpoint(tmp_path / "run2"))
    assert set(meta["run_artifacts"]) >= {"metrics.jsonl", "numerics.jsonl"}
    assert (tmp_path / "run2" / "metrics.png").exists() and (tmp_path / "run2" / "config.json").exists()
    numerics = [json.loads(l) for l in (tmp_path / "run2" / "numerics.jsonl").read_text().splitlines()]
    assert any("load_max_ratio" in s for s in numerics[0]["records"].values())


def test_tiny_moe_twenty_steps_checkpoint_at_twenty_and_resume(tmp_path):
    """The plumbing configuration: the `tiny` variant (d_model 256, one sliding + one global layer, 4 query / 2 kv heads of
    64, gated attention with sinks, 4 routed top-2 + 1 shared expert, hidden 512, full 201,088-token vocabulary), sequence
    256, batch 2, iid-uniform tokens from torch seed 0, fp32 weights with bf16 compute, Muon + Adam; 20 steps, the
    checkpoint of step 20, and a resumed run that continues from it."""
    from lyra_b200.variants import model_variant

    c = model_variant("tiny")
    assert (c.n_embd, c.n_layers, c.n_attn_heads, c.n_kv_heads, c.head_dim, c.vocab_size) == (256, 2, 4, 2, 64, 201088)
    assert c.param_dtype == torch.float32 and c.compute_dtype == torch.bfloat16
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, c.vocab_size, (64 * (c.seq_len + 1),), generator=g, dtype=torch.int32).numpy()
    np.save(tmp_path / "tok.npy", tokens)
    tcfg = TrainingConfig(steps=22, batch_size=2, accumulation_steps=1, data_path=tmp_path / "tok.npy", eval_data_path=tmp_path / "tok.npy",
                          eval_every=None, checkpoint_every=20, checkpoint_path=tmp_path / "run", log_every=5,
                          data_loader=DataLoaderConfig(worker_count=1))

    class StopAfterTwenty(TrainHooks):
        def before_step(self, step, *a):
            if step == 21:
                raise RuntimeError("stopped after the step-20 checkpoint")

    with pytest.raises(RuntimeError, match="step-20 checkpoint"):
        train(ModelWeights.init(0, c), c, tcfg, device="cpu", hooks=StopAfterTwenty())
    assert [p.name for p in checkpoint_steps(tmp_path / "run")] == ["step_00000020"]
    rows = [json.loads(l) for l in (tmp_path / "run" / "metrics.jsonl").read_text().splitlines() if json.loads(l)["kind"] == "train"]
    assert rows[-1]["step"] == 20 and all(np.isfinite(r["loss"]) for r in rows)
    assert rows[-1]["loss"] < rows[0]["loss"]                     # 64 sequences seen many times: the loss moves down
    at_twenty = load_train_state(tmp_path / "run", c, tcfg)
    assert at_twenty.step == 20
    resumed = train(None, c, replace(tcfg, resume_from=tmp_path / "run"), device="cpu")
    a, b = tree_dict(at_twenty.state.params), tree_dict(resumed.params)
    assert any(not torch.equal(a[k], b[k]) for k in a)            # two more optimizer steps were taken
    rows = [json.loads(l) for l in (tmp_path / "run" / "metrics.jsonl").read_text().splitlines() if json.loads(l)["kind"] == "train"]
    assert [r["step"] for r in rows][-1] == 22 and np.isfinite(rows[-1]["loss"])


def test_resume_auto_restarts_an_interrupted_run_with_the_same_command_line(tmp_path):
    """What a supervisor that restarts failed jobs needs (``torch.distributed.run --max-restarts``): the first launch starts a
    run, a launch after a failure continues from the newest finished checkpoint, both with the same arguments."""
    from scripts.train import Args, main, training_config

    data = token_file(tmp_path / "tok.npy", n=40000, vocab=256)
    argv = ["--variant", "dev", "--run", "train-dev", "--device", "cpu", "--implementation", "torch", "--steps", "4", "--batch-size", "2",
            "--acc-steps", "1", "--data", str(data), "--out", str(tmp_path / "run"), "--chkpt-every", "2", "--resume", "auto"]
    args = Args(variant="dev", run="train-dev", steps=4, batch_size=2, acc_steps=1, data=str(data), out=str(tmp_path / "run"), chkpt_every=2, resume="auto")
    first = training_config(args)
    assert first.resume_from is None                               # nothing there yet: a new run

    class FailAtThree(TrainHooks):
        def before_step(self, step, *a):
            if step == 3:
                raise RuntimeError("lost a peer")

    from lyra_b200.variants import model_variant

    c = replace(model_variant("dev"), implementation="torch")
    with pytest.raises(RuntimeError, match="lost a peer"):
        train(ModelWeights.init(c.seed, c), c, first, device="cpu", hooks=FailAtThree())
    assert training_config(args).resume_from == tmp_path / "run"    # the restart finds the step-2 checkpoint
    assert main(argv) == 0
    rows = [json.loads(l) for l in (tmp_path / "run" / "metrics.jsonl").read_text().splitlines() if json.loads(l)["kind"] == "train"]
    assert [p.name for p in checkpoint_steps(tmp_path / "run")][-1] == "step_00000004" and rows[-1]["step"] == 4


def test_a_kernel_failure_stops_the_run_before_it_is_logged_or_checkpointed(tmp_path, monkeypatch):
    """Kernels report a failed wait or an overflowing buffer through a status word; the loop reads it before every log line and
    checkpoint. Here the read is faked: from the fourth check on it reports a peer timeout. The run must stop there, and neither
    the log nor the checkpoint directory may contain the step whose results are suspect."""
    import lyra_b200.training.train as T
    from lyra_b200.ops.native import NativeError

    checks = []

    def fake_status(device):
        checks.append(device)
        if len(checks) >= 4:
            raise NativeError("device 0: kernel reported 'timeout waiting for a peer flag'")

    monkeypatch.setattr(T, "check_device_status", fake_status)
    c = small_config()
    tcfg = replace(_tcfg(tmp_path), steps=8, log_every=1, checkpoint_every=2, eval_every=None, eval_data_path=None, numerics_every=None)
    with pytest.raises(NativeError, match="peer flag"):
        train(ModelWeights.init(0, c), c, tcfg, device="cpu")
    # checks: log step 1, log step 2, save step 2, log step 3 (raises)
    rows = [json.loads(l)["step"] for l in (tmp_path / "run" / "metrics.jsonl").read_text().splitlines() if json.loads(l)["kind"] == "train"]
    assert rows == [1, 2]
    assert [p.name for p in checkpoint_steps(tmp_path / "run")] == ["step_00000002"]


def test_gs_locations_are_mirrored_through_the_sync_tool(tmp_path, monkeypatch):
    """``gs://`` run directories: staged locally, pulled once when first named, pushed after a save. The sync tool is replaced by
    a script that copies between a fake bucket directory and the staging directory."""
    import stat
    import sys

    from lyra_b200.nn import checkpoints as C

    bucket = tmp_path / "bucket"
    (bucket / "runs" / "a" / "step_00000002").mkdir(parents=True)
    (bucket / "runs" / "a" / "step_00000002" / "_CHECKPOINT_METADATA").write_text("{}")
    tool = tmp_path / "fake_rsync.py"
    tool.write_text(
        "import shutil, sys\n"
        f"root = {str(bucket)!r}\n"
        "conv = lambda p: root + '/' + p.removeprefix('gs://fake/') if p.startswith('gs://fake/') else p\n"
        "src, dst = conv(sys.argv[-2]), conv(sys.argv[-1])\n"
        "import os\n"
        "if os.path.isdir(src): shutil.copytree(src, dst, dirs_exist_ok=True)\n")
    tool.chmod(tool.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("LYRA_GS_SYNC", f"{sys.executable} {tool}")
    monkeypatch.setenv("LYRA_GS_CACHE", str(tmp_path / "cache"))
    monkeypatch.setattr(C, "_REMOTES", {})
    local = C.checkpoint_path("gs://fake/runs/a")
    assert local == (tmp_path / "cache" / "fake" / "runs" / "a").resolve()
    assert [p.name for p in C.checkpoint_steps(local)] == ["step_00000002"]          # pulled from the bucket
    (local / "step_00000004").mkdir()
    (local / "step_00000004" / "_CHECKPOINT_METADATA").write_text("{}")
    assert C.sync_remote(local / "step_00000004") is True
    assert (bucket / "runs" / "a" / "step_00000004" / "_CHECKPOINT_METADATA").is_file()   # pushed back
    assert C.sync_remote(tmp_path / "elsewhere") is False
    assert C.checkpoint_path("~/x") == C.checkpoint_path(str(C.Path.home() / "x"))


def test_a_single_step_run_uses_the_peak_learning_rates():
    from dataclasses import replace as _replace

    from lyra_b200.training.presets import TRAINING_PRESETS

    tcfg = _replace(TRAINING_PRESETS["train-dev"], steps=1)
    adam_lr, muon_lr, scale = wsd_lr(0, tcfg)
    assert abs(float(scale) - 1.0) < 1e-6
    assert abs(float(adam_lr) - tcfg.adam_max_lr) < 1e-9 and abs(float(muon_lr) - tcfg.muon_max_lr) < 1e-9


def test_validation_replays_the_same_batches_and_the_last_one_follows_the_final_checkpoint(tmp_path, monkeypatch):
    """Evaluation runs before the first step, on its cadence and after the last step's checkpoint; every evaluation reads the
    same leading batches of the evaluation file, in file order, whatever the (shuffled) training loader does."""
    from lyra_b200.training import train as train_module

    c = small_config(seq_len=8, n_layers=1, mlp_map=("dense",), vocab_size=64, padded_vocab_size=64)
    T, n_eval = c.seq_len, 3
    held_out = ((np.arange(6 * T + 1) * 7 + 3) % c.vocab_size).astype(np.int32)      # a recognisable pattern, no two windows alike
    np.save(tmp_path / "held_out.npy", held_out)
    tcfg = TrainingConfig(steps=5, batch_size=1, accumulation_steps=1, data_path=token_file(tmp_path / "tok.npy", n=40 * T, vocab=c.vocab_size),
                          data_loader=DataLoaderConfig(worker_count=0, shuffle=True), eval_data_path=tmp_path / "held_out.npy", eval_every=3,
                          eval_batches=n_eval, checkpoint_every=1000, checkpoint_path=tmp_path / "out")
    last_checkpoint = tcfg.checkpoint_path / f"step_{tcfg.steps:08d}"
    windows_per_eval, checkpoint_seen = [], []
    original = train_module.run_validation

    def spy(stepper, batches, **kw):
        checkpoint_seen.append(last_checkpoint.is_dir())
        taken = []

        def recording():
            for x, y in batches:
                taken.append((np.array(x).reshape(-1), np.array(y).reshape(-1)))
                yield x, y

        result = original(stepper, recording(), **kw)
        windows_per_eval.append(taken)
        return result

    monkeypatch.setattr(train_module, "run_validation", spy)
    monkeypatch.setattr(train_module, "plot_run", lambda run_dir: None)
    train_module.train(ModelWeights.init(0, c), c, tcfg)

    logged = [json.loads(line) for line in (tcfg.checkpoint_path / "metrics.jsonl").read_text().splitlines()]
    assert [row["step"] for row in logged if row["kind"] == "eval"] == [0, 3, 5]
    assert checkpoint_seen == [False, False, True]          # only the last evaluation comes after the final checkpoint
    expected = [(held_out[i * T:(i + 1) * T], held_out[i * T + 1:(i + 1) * T + 1]) for i in range(n_eval)]
    for taken in windows_per_eval:
        assert len(taken) == n_eval
        for (x, y), (want_x, want_y) in zip(taken, expected):
            assert np.array_equal(x, want_x) and np.array_equal(y, want_y)
