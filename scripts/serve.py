"""Interactive chat with a checkpoint: this framework's own checkpoints or GPT-OSS ``original/`` checkpoints (Harmony format).

Flags follow the reference's ``scripts/serve.py``. Under ``python -m torch.distributed.run --nproc-per-node N --master-addr
127.0.0.1 scripts/serve.py ...`` the model is split tensor-parallel over the N processes (a model that does not fit one GPU):
the first process owns the terminal, the others receive each prompt from it and take part in every model call."""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Literal

import tyro

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")   # load kernels with the library, not at first launch (multi-rank waits)

try:
    from scripts._launch import default_weights, join_tensor_parallel, place
except ImportError:                        # run as a file: scripts/ itself is the import root
    from _launch import default_weights, join_tensor_parallel, place


@dataclass(frozen=True)
class Args:
    variant: str = "lyra-small"
    """Which model variant the checkpoint belongs to."""
    weights: str | None = None
    """Checkpoint (or run) directory; chkpt/<variant> when omitted."""
    format: Literal["orbax", "gpt-oss"] = "orbax"
    """orbax: a checkpoint written by scripts/train.py; gpt-oss: an original/ GPT-OSS checkpoint (Harmony chat format)."""
    device: Literal["auto", "cpu", "gpu"] = "auto"
    """auto takes a GPU when there is one."""
    max_new_tokens: int = 256
    """Upper bound of the tokens generated for one reply."""
    max_cache_length: int | None = None
    """KV-cache length (conversation so far plus the reply); the model's context length when omitted."""
    temperature: float | None = None
    """Sampling temperature; the variant's own setting when omitted."""
    top_k: int | None = None
    """Sample among the k most likely tokens; the variant's own setting when omitted."""
    fp8: bool = False
    """Keep expert / MLP weights and the KV cache as block-scaled e4m3."""


def main(argv: list[str] | None = None) -> int:
    args = tyro.cli(Args, args=argv)
    from lyra_b200.generate import InferenceConfig, apply_inference_overrides, load_model, serve_model
    from lyra_b200.gpt_oss import load_gpt_oss_model
    from lyra_b200.variants import model_variant

    settings = InferenceConfig(weights=args.weights or default_weights(args.variant), max_new_tokens=args.max_new_tokens,
                               max_cache_length=args.max_cache_length, temperature=args.temperature, top_k=args.top_k, fp8=args.fp8)
    config = apply_inference_overrides(model_variant(args.variant), settings)
    where = join_tensor_parallel(place(args.device), config)
    terminal = {}
    if where.runtime is not None:
        from lyra_b200.parallel.tp import shared_terminal

        terminal = shared_terminal(where.runtime)          # prompts typed on the first rank reach all of them
    chat_format = args.format == "gpt-oss"
    if chat_format:
        model = load_gpt_oss_model(settings.weights, config, device=where.device, shard_fn=where.shard_fn)
    else:
        model = load_model(config, settings, device=where.device, rt=where.runtime)
    serve_model(model, config, settings, harmony=chat_format, device=where.device, rt=where.runtime, **terminal)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
