"""What the three entry points share: where the package lives, which device a process uses, and how the processes of a
``torch.distributed.run`` launch join into a tensor-parallel group."""

from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def default_weights(variant: str) -> str:
    """Where the training presets save a variant's checkpoints and serving / evaluation look for them."""
    return str(ROOT / "chkpt" / variant)


@dataclass
class Placement:
    """Device and process-group facts of this process."""

    device: str
    on_gpu: bool
    world: int
    rank: int
    runtime: Any = None                     # TensorParallel when the launch has several processes

    @property
    def primary(self) -> bool:
        return self.rank == 0

    def say(self, *args, **kwargs) -> None:
        """``print`` on the first rank only."""
        if self.primary:
            print(*args, **kwargs)

    @property
    def shard_fn(self) -> Callable | None:
        return self.runtime.shard_info if self.runtime is not None else None


def place(choice: str) -> Placement:
    """``choice``: the ``--device`` flag (auto / cpu / gpu). One process per GPU; LOCAL_RANK picks the GPU."""
    import torch

    on_gpu = choice == "gpu" or (choice == "auto" and torch.cuda.is_available())
    world, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    if on_gpu:
        torch.cuda.set_device(local)
    return Placement(device=f"cuda:{local}" if on_gpu else "cpu", on_gpu=on_gpu, world=world, rank=int(os.environ.get("RANK", "0")))


def join_tensor_parallel(where: Placement, config) -> Placement:
    """Several processes: the model is split over them (heads and hidden units), every rank sees the same inputs."""
    if where.world > 1:
        import torch.distributed as dist

        from lyra_b200.parallel.tp import TensorParallel

        dist.init_process_group("nccl" if where.on_gpu else "gloo")
        where.rank = dist.get_rank()
        where.runtime = TensorParallel(config, where.rank, where.world)
    return where
