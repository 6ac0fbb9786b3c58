"""Training state and its checkpoints: the six checkpointables of the reference
(``params, muon_moment, adam_mu, adam_nu, adam_count, loader``; lyra/training/state.py:48-113)."""

from __future__ import annotations

import shutil
from dataclasses import dataclass, replace
from pathlib import Path

import torch

from lyra_b200.config import ModelConfig
from lyra_b200.model import ModelWeights
from lyra_b200.nn.checkpoints import checkpoint_steps, load_checkpointables, resolve_checkpoint, save_checkpointables
from lyra_b200.nn.params import tree_dict
from lyra_b200.training.optimizer import ADAM_TAGS, MUON_TAGS, OptimizerState


@dataclass
class TrainState:
    params: ModelWeights
    optimizer: OptimizerState


@dataclass(frozen=True)
class RestoredTrainState:
    state: TrainState
    step: int
    path: Path
    loader_state: bytes


def init_train_state(params: ModelWeights, mcfg: ModelConfig, tcfg) -> TrainState:
    return TrainState(params, OptimizerState.init(params, ModelWeights.spec(mcfg), tcfg))


def train_state_checkpointables(state: TrainState, loader_state: bytes) -> dict:
    opt = state.optimizer
    return {
        "params": state.params,
        "muon_moment": opt.muon_moment,
        "adam_mu": opt.adam_mu,
        "adam_nu": opt.adam_nu,
        "adam_count": opt.adam_count,
        "loader": {"state": loader_state.decode()},
    }


def save_checkpoint(directory: Path, step: int, state: TrainState, loader_state: bytes, run_config: dict, *, keep: int, rt=None) -> Path:
    """Saves ``step_<step>`` and deletes all but the ``keep`` most recent finished checkpoints."""
    path = Path(directory) / f"step_{step:08d}"
    primary = rt is None or rt.rank == 0
    if primary and path.exists():  # a partial save from an interrupted run
        shutil.rmtree(path)
    if primary:
        print(f"\n[checkpoint] Saving {path}")
    save_checkpointables(path, train_state_checkpointables(state, loader_state), custom_metadata={"run_config": run_config}, rt=rt)
    if primary:
        for old in checkpoint_steps(Path(directory))[:-keep]:
            shutil.rmtree(old)
    return path


def load_train_state(source, mcfg: ModelConfig, tcfg, *, device="cpu", rt=None) -> RestoredTrainState:
    path = resolve_checkpoint(source)
    spec = ModelWeights.spec(mcfg)
    leaves = tree_dict(spec)
    muon = {p: replace(s, dtype=tcfg.muon_moment_dtype) for p, s in leaves.items() if s.tag in MUON_TAGS}
    mu = {p: replace(s, dtype=tcfg.adam_mu_dtype) for p, s in leaves.items() if s.tag in ADAM_TAGS}
    nu = {p: replace(s, dtype=tcfg.adam_nu_dtype) for p, s in leaves.items() if s.tag in ADAM_TAGS}
    loaded = load_checkpointables(
        path,
        {"params": spec, "muon_moment": muon, "adam_mu": mu, "adam_nu": nu,
         "adam_count": torch.zeros((), dtype=torch.int32), "loader": None},
        device=device, rt=rt,
    )
    optimizer = OptimizerState(muon_moment=loaded["muon_moment"], adam_mu=loaded["adam_mu"], adam_nu=loaded["adam_nu"],
                               adam_count=loaded["adam_count"])
    return RestoredTrainState(
        state=TrainState(loaded["params"], optimizer),
        step=int(path.name.removeprefix("step_")),
        path=path,
        loader_state=loaded["loader"]["state"].encode(),
    )
