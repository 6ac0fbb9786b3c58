"""Parameter runtime: specs, tags, tree utilities, initialisation, shard geometry.

Parameters live in nested dataclasses whose leaf paths (``layers/3/mlp/mlp_up``, ``tok/emb``) equal
the reference's (lyra/nn/checkpoints.py:40-41), so checkpoints describe the same tree. A leaf is an
``ArraySpec`` before initialisation and a ``torch.Tensor`` (this rank's shard) after.
"""

from __future__ import annotations

import dataclasses
import hashlib
import math
from dataclasses import dataclass
from enum import Enum, auto
from typing import Any, Callable, Iterator

import torch

from lyra_b200.nn.quant import QArray


class Tag(Enum):
    """Optimizer routing (lyra/nn/params.py:21-26): MATRIX -> Muon, everything else -> Adam."""

    DEFAULT = auto()
    SCALAR = auto()
    BIAS = auto()
    MATRIX = auto()
    EMBEDDING = auto()


@dataclass(frozen=True)
class ArraySpec:
    shape: tuple[int, ...]
    dtype: torch.dtype
    kind: str  # name of the sharding rule, see SHARD_DIMS
    init: str  # initialiser name, see _INITIALIZERS
    tag: Tag = Tag.DEFAULT
    init_scale: float = 1.0


# (fsdp dim, model(TP) dim, expert dim) per parameter kind - the reference's rule table
# (lyra/nn/params.py:226-249) with None = replicated on that axis.
SHARD_DIMS: dict[str, tuple[int | None, int | None, int | None]] = {
    "emb": (0, None, None),
    "unemb": (0, None, None),
    "norm_scale": (None, None, None),
    "attn_q": (0, 1, None),
    "attn_kv": (0, 1, None),
    "attn_qkv_bias": (None, 0, None),
    "attn_sink": (None, 0, None),
    "attn_out": (1, 0, None),
    "attn_out_bias": (None, None, None),
    "router": (0, None, None),
    "router_bias": (None, None, None),
    "moe_mlp_up": (1, 3, 0),
    "moe_mlp_down": (2, 1, 0),
    "moe_mlp_up_bias": (None, 2, 0),
    "moe_mlp_down_bias": (None, None, 0),
    "dense_mlp_up": (0, 2, None),
    "dense_mlp_down": (1, 0, None),
    "dense_mlp_up_bias": (None, 2, None),
    "dense_mlp_down_bias": (None, None, None),
}


# --------------------------------------------------------------------------- tree utilities
def is_spec(x: object) -> bool:
    return isinstance(x, ArraySpec)


def _is_leaf(x: object) -> bool:
    return isinstance(x, (torch.Tensor, ArraySpec, QArray)) or not (
        dataclasses.is_dataclass(x) or isinstance(x, (list, tuple, dict))
    )


def tree_items(tree: Any, prefix: str = "") -> Iterator[tuple[str, Any]]:
    """Yields ``(path, leaf)`` for every non-None leaf, in field order."""
    if tree is None:
        return
    if _is_leaf(tree):
        yield prefix, tree
        return
    if dataclasses.is_dataclass(tree):
        children = ((f.name, getattr(tree, f.name)) for f in dataclasses.fields(tree))
    elif isinstance(tree, dict):
        children = tree.items()
    else:
        children = ((str(i), v) for i, v in enumerate(tree))
    for name, child in children:
        yield from tree_items(child, f"{prefix}/{name}" if prefix else str(name))


def tree_map(fn: Callable[..., Any], tree: Any, *rest: Any) -> Any:
    """Structure-preserving map over leaves; ``None`` fields stay ``None`` (absent optional parameters)."""
    if tree is None:
        return None
    if _is_leaf(tree):
        return fn(tree, *rest)
    if dataclasses.is_dataclass(tree):
        return type(tree)(**{
            f.name: tree_map(fn, getattr(tree, f.name), *(getattr(r, f.name) for r in rest)) for f in dataclasses.fields(tree)
        })
    if isinstance(tree, dict):
        return {k: tree_map(fn, v, *(r[k] for r in rest)) for k, v in tree.items()}
    return type(tree)(tree_map(fn, v, *(r[i] for r in rest)) for i, v in enumerate(tree))


def tree_leaves(tree: Any) -> list[Any]:
    return [leaf for _, leaf in tree_items(tree)]


def tree_dict(tree: Any) -> dict[str, Any]:
    return dict(tree_items(tree))


# --------------------------------------------------------------------------- initialisers
_TRUNC_STD = 0.87962566103423978  # std of a unit normal truncated to [-2, 2]


def _fans(shape: tuple[int, ...], in_axis: int = -2, out_axis: int = -1) -> tuple[float, float]:
    if len(shape) < 2:
        return float(shape[0]) if shape else 1.0, float(shape[0]) if shape else 1.0
    receptive = math.prod(shape) / (shape[in_axis] * shape[out_axis])
    return shape[in_axis] * receptive, shape[out_axis] * receptive


def _trunc_normal(shape, std: float, gen: torch.Generator, device) -> torch.Tensor:
    t = torch.empty(shape, dtype=torch.float32, device=device)
    s = std / _TRUNC_STD
    torch.nn.init.trunc_normal_(t, mean=0.0, std=s, a=-2.0 * s, b=2.0 * s, generator=gen)
    return t


def _init_lecun(shape, scale, gen, device):
    fan_in, _ = _fans(shape)
    return _trunc_normal(shape, math.sqrt(scale / fan_in), gen, device)


def _init_emb(shape, scale, gen, device):  # variance 1 / n_embd for both emb and unemb
    return _trunc_normal(shape, math.sqrt(scale / shape[1]), gen, device)


_INITIALIZERS: dict[str, Callable] = {
    "lecun_normal": _init_lecun,
    "fan_in_trunc": _init_lecun,
    "emb": _init_emb,
    "zeros": lambda shape, scale, gen, device: torch.zeros(shape, dtype=torch.float32, device=device),
    "ones": lambda shape, scale, gen, device: torch.ones(shape, dtype=torch.float32, device=device),
}


def _leaf_seed(seed: int, path: str, sub: int = 0) -> int:
    h = hashlib.blake2b(f"{seed}:{path}:{sub}".encode(), digest_size=8).digest()
    return int.from_bytes(h, "little") & 0x7FFFFFFFFFFFFFFF


@dataclass(frozen=True)
class ShardInfo:
    """Which slice of the global array a rank holds: ``{dim: (index, parts)}``."""

    slices: tuple[tuple[int, int, int], ...] = ()  # (dim, index, parts)
    absent: bool = False  # this rank holds no part of the leaf (it is owned elsewhere); a 0-element placeholder stands in

    def local_shape(self, shape: tuple[int, ...]) -> tuple[int, ...]:
        out = list(shape)
        for dim, _, parts in self.slices:
            assert out[dim] % parts == 0, (shape, dim, parts)
            out[dim] //= parts
        return tuple(out)

    def narrow(self, t: torch.Tensor) -> torch.Tensor:
        for dim, index, parts in self.slices:
            n = t.shape[dim] // parts
            t = t.narrow(dim, index * n, n)
        return t


def init_leaf(spec: ArraySpec, seed: int, path: str, device, shard: ShardInfo | None = None) -> torch.Tensor:
    """Initialises one leaf. Every leaf draws from its own generator keyed by ``(seed, path)`` so adding
    or removing a parameter (e.g. the output gate) never changes any other parameter's initial value
    (the invariant of lyra/model.py:713-721). Stacked expert weights draw one stream per expert
    (``stacked_init``, lyra/model.py:145-151), which lets an expert-parallel rank initialise only its experts."""
    fn = _INITIALIZERS[spec.init]
    shard = shard or ShardInfo()
    if shard.absent:
        return torch.empty(0, dtype=spec.dtype, device=device)
    stacked = spec.kind.startswith("moe_mlp") and spec.init not in ("zeros", "ones")
    if stacked:
        expert_slices = [s for s in shard.slices if s[0] == 0]
        rest = ShardInfo(tuple(s for s in shard.slices if s[0] != 0))
        n_exp = spec.shape[0]
        lo, hi = 0, n_exp
        if expert_slices:
            _, index, parts = expert_slices[0]
            lo, hi = index * (n_exp // parts), (index + 1) * (n_exp // parts)
        outs = []
        for e in range(lo, hi):
            gen = torch.Generator(device=device).manual_seed(_leaf_seed(seed, path, e + 1))
            full = fn(spec.shape[1:], spec.init_scale, gen, device)
            # dims of `rest` refer to the stacked array; shift by one for the per-expert array
            for dim, index, parts in rest.slices:
                n = full.shape[dim - 1] // parts
                full = full.narrow(dim - 1, index * n, n)
            outs.append(full.to(spec.dtype))
        return torch.stack(outs, dim=0).contiguous()
    gen = torch.Generator(device=device).manual_seed(_leaf_seed(seed, path))
    full = fn(spec.shape, spec.init_scale, gen, device)
    return shard.narrow(full).to(spec.dtype).contiguous()


def init_weights(spec_tree: Any, seed: int, device="cpu", shard_fn: Callable[[str, ArraySpec], ShardInfo] | None = None) -> Any:
    return _map_with_path(lambda path, leaf: init_leaf(leaf, seed, path, device, shard_fn(path, leaf) if shard_fn else None), spec_tree)


def _map_with_path(fn: Callable[[str, Any], Any], tree: Any, prefix: str = "") -> Any:
    if tree is None:
        return None
    if _is_leaf(tree):
        return fn(prefix, tree)
    join = lambda name: f"{prefix}/{name}" if prefix else str(name)
    if dataclasses.is_dataclass(tree):
        return type(tree)(**{f.name: _map_with_path(fn, getattr(tree, f.name), join(f.name)) for f in dataclasses.fields(tree)})
    if isinstance(tree, dict):
        return {k: _map_with_path(fn, v, join(k)) for k, v in tree.items()}
    return type(tree)(_map_with_path(fn, v, join(i)) for i, v in enumerate(tree))


map_with_path = _map_with_path


def param_count(spec_tree: Any) -> int:
    return sum(math.prod(leaf.shape) for leaf in tree_leaves(spec_tree))
