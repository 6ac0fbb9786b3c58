"""Checkpoint directories in the Orbax-v1 "checkpointables" layout, written without Orbax.

    <run>/step_00000020/
        _CHECKPOINT_METADATA                 JSON; ``custom_metadata.run_config`` carries the run configuration
        params/  muon_moment/  adam_mu/  adam_nu/  adam_count/      one pytree checkpointable each
            _METADATA                        JSON tree description (leaf path -> shape, dtype, chunk grid)
            <leaf.path.with.dots>/zarr.json  zarr-v3 array metadata
            <leaf.path.with.dots>/c/i/j      raw little-endian chunks, one per shard of the array
        loader/metadata                      JSON ``{"state": "<loader state>"}``

This mirrors what the reference relies on (lyra/training/state.py:48-67, lyra/nn/checkpoints.py:12-52):
only directories that contain ``_CHECKPOINT_METADATA`` and are not temp-named count as checkpoints, arrays are
stored as *global* arrays (every rank writes only the chunks it owns, and a restore may use a different world
size), and leaf paths are the ``/``-joined field names of the parameter tree. A checkpoint is written into
``<name>.orbax-checkpoint-tmp-<n>`` and renamed when complete, so an interrupted save never looks finished.
Chunk files are read and written by the native I/O pool (``csrc/io/chunk_io.cpp``) when it is built.
"""

from __future__ import annotations

import ctypes
import itertools
import json
import math
import os
import shutil
import time
from pathlib import Path
from typing import Any

import numpy as np
import torch

from lyra_b200.nn.params import ArraySpec, ShardInfo, map_with_path, tree_dict

TMP_MARK = ".orbax-checkpoint-tmp-"
METADATA_FILE = "_CHECKPOINT_METADATA"

_ZARR_DTYPES = {
    torch.float32: "float32", torch.bfloat16: "bfloat16", torch.float16: "float16", torch.int32: "int32",
    torch.int64: "int64", torch.uint8: "uint8", torch.float8_e4m3fn: "float8_e4m3fn", torch.float8_e5m2: "float8_e5m2",
    torch.int8: "int8", torch.float64: "float64",
}
_TORCH_DTYPES = {v: k for k, v in _ZARR_DTYPES.items()}


# --------------------------------------------------------------------------- paths
_REMOTES: dict[Path, str] = {}          # local staging directory -> the gs:// location it mirrors


def _sync_command() -> list[str]:
    """The external tool that mirrors a directory to / from object storage: ``LYRA_GS_SYNC`` or ``gsutil -m rsync -r``."""
    return os.environ.get("LYRA_GS_SYNC", "gsutil -m rsync -r").split()


def checkpoint_path(source) -> Path:
    """Local absolute path of a checkpoint or run directory. A ``gs://bucket/dir`` location (the reference accepts those through
    etils, lyra/nn/checkpoints.py:12-14) is mirrored: it maps to a staging directory under ``LYRA_GS_CACHE`` (default
    ``~/.cache/lyra_b200/gs``), filled from the bucket the first time it is named in this process (so a resume finds its
    checkpoints), and pushed back by ``sync_remote`` after every checkpoint and at the end of a run - the run itself reads and
    writes local files only, as the reference does for its logs."""
    text = str(source)
    if not text.startswith("gs://"):
        return Path(os.path.abspath(os.path.expanduser(text)))
    cache = Path(os.path.expanduser(os.environ.get("LYRA_GS_CACHE", "~/.cache/lyra_b200/gs")))
    local = (cache / text.removeprefix("gs://").strip("/")).resolve()
    if local not in _REMOTES:
        import subprocess

        local.mkdir(parents=True, exist_ok=True)
        _REMOTES[local] = text.rstrip("/")
        done = subprocess.run([*_sync_command(), _REMOTES[local], str(local)], capture_output=True, text=True)
        if done.returncode != 0 and any(local.iterdir()):
            raise OSError(f"could not mirror {text} into {local}: {done.stderr.strip()[-300:]}")
    return local


def sync_remote(path) -> bool:
    """Pushes ``path``'s mirrored root (if it lies in one) back to its ``gs://`` location. Returns whether anything was mirrored."""
    import subprocess

    path = Path(path).resolve()
    for local, remote in _REMOTES.items():
        if path == local or local in path.parents:
            done = subprocess.run([*_sync_command(), str(local), remote], capture_output=True, text=True)
            if done.returncode != 0:
                raise OSError(f"could not push {local} to {remote}: {done.stderr.strip()[-300:]}")
            return True
    return False


def is_checkpoint(path: Path) -> bool:
    return (path / METADATA_FILE).is_file() and TMP_MARK not in path.name


def checkpoint_steps(directory: Path) -> list[Path]:
    if not directory.is_dir():
        return []
    steps = [p for p in directory.glob("step_*") if is_checkpoint(p)]
    return sorted(steps, key=lambda p: int(p.name.removeprefix("step_")))


def resolve_checkpoint(source) -> Path:
    """A checkpoint directory itself, or the latest finished ``step_*`` of a run directory."""
    path = checkpoint_path(source)
    if is_checkpoint(path):
        return path
    steps = checkpoint_steps(path)
    if not steps:
        raise FileNotFoundError(f"No completed checkpoint in {path}")
    return steps[-1]


def checkpoint_run_config(path: Path) -> dict:
    return json.loads((path / METADATA_FILE).read_text())["custom_metadata"]["run_config"]


# --------------------------------------------------------------------------- raw chunk I/O
def _bytes_view(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous().cpu().reshape(-1)
    return t.view(torch.uint8).numpy().reshape(-1) if t.numel() else np.zeros(0, np.uint8)


def _io_lib():
    try:
        from lyra_b200.ops import native

        return native.io()
    except Exception:
        return None


def write_files(items: list[tuple[Path, np.ndarray]]) -> None:
    """Writes byte buffers to files, in parallel through the native pool when available."""
    for path, _ in items:
        path.parent.mkdir(parents=True, exist_ok=True)
    lib = _io_lib()
    if lib is None or not items:
        for path, buf in items:
            with open(path, "wb") as f:
                f.write(buf.tobytes())
        return
    n = len(items)
    paths = (ctypes.c_char_p * n)(*[str(p).encode() for p, _ in items])
    ptrs = (ctypes.c_void_p * n)(*[b.ctypes.data if b.size else 0 for _, b in items])
    sizes = (ctypes.c_longlong * n)(*[b.size for _, b in items])
    lib.lyra_io_write_files.restype = ctypes.c_int
    rc = lib.lyra_io_write_files(n, paths, ptrs, sizes, 8)
    if rc != 0:
        raise OSError(f"native chunk write failed for {items[rc - 1][0] if rc > 0 else 'unknown'}")


def read_files(items: list[tuple[Path, np.ndarray]]) -> None:
    lib = _io_lib()
    if lib is None or not items:
        for path, buf in items:
            data = np.fromfile(path, dtype=np.uint8)
            if data.size != buf.size:
                raise OSError(f"{path}: expected {buf.size} bytes, found {data.size}")
            buf[:] = data
        return
    n = len(items)
    paths = (ctypes.c_char_p * n)(*[str(p).encode() for p, _ in items])
    ptrs = (ctypes.c_void_p * n)(*[b.ctypes.data if b.size else 0 for _, b in items])
    sizes = (ctypes.c_longlong * n)(*[b.size for _, b in items])
    lib.lyra_io_read_files.restype = ctypes.c_int
    rc = lib.lyra_io_read_files(n, paths, ptrs, sizes, 8)
    if rc != 0:
        raise OSError(f"native chunk read failed for {items[rc - 1][0] if rc > 0 else 'unknown'}")


# --------------------------------------------------------------------------- array (zarr v3, one chunk per shard)
def _leaf_dir(path: str) -> str:
    return path.replace("/", ".") if path else "value"


def _chunk_grid(shape: tuple[int, ...], shard: ShardInfo) -> tuple[tuple[int, ...], tuple[int, ...]]:
    parts = [1] * len(shape)
    index = [0] * len(shape)
    for dim, idx, n in shard.slices:
        parts[dim] *= n
        index[dim] = idx
    return tuple(parts), tuple(index)


def _zarr_json(shape, chunk_shape, dtype: torch.dtype) -> dict:
    return {
        "zarr_format": 3, "node_type": "array", "shape": list(shape), "data_type": _ZARR_DTYPES[dtype],
        "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": [max(int(c), 1) for c in chunk_shape]}},
        "chunk_key_encoding": {"name": "default", "configuration": {"separator": "/"}},
        "fill_value": 0, "codecs": [{"name": "bytes", "configuration": {"endian": "little"}}], "attributes": {},
    }


def _chunk_file(base: Path, index: tuple[int, ...]) -> Path:
    return base / "c" / Path(*map(str, index)) if index else base / "c"


def save_tree(root: Path, tree: Any, *, shard_of=None, writes_leaf=None, is_primary: bool = True, all_leaves=None) -> None:
    """Writes one pytree checkpointable. ``shard_of(path, tensor) -> (global_shape, ShardInfo)`` describes how the
    local tensor sits in the global array; ``writes_leaf(path)`` says whether this rank writes its chunk (one writer
    per distinct shard). The primary rank also writes the tree and array metadata."""
    leaves = tree_dict(tree)
    files: list[tuple[Path, np.ndarray]] = []
    meta: dict[str, dict] = {}
    if all_leaves and is_primary:  # leaves owned by other ranks: the primary writes their array metadata
        for path, (gshape, dtype, parts) in all_leaves.items():
            if path in leaves and leaves[path].numel() > 0:
                continue
            base = root / _leaf_dir(path)
            base.mkdir(parents=True, exist_ok=True)
            chunk_shape = tuple(s // p for s, p in zip(gshape, parts))
            (base / "zarr.json").write_text(json.dumps(_zarr_json(gshape, chunk_shape, dtype)))
            meta[path] = {"shape": list(gshape), "dtype": _ZARR_DTYPES[dtype], "chunks": list(parts)}
    for path, t in leaves.items():
        if not isinstance(t, torch.Tensor):
            t = torch.as_tensor(t)
        if all_leaves and t.numel() == 0 and path in all_leaves and math.prod(all_leaves[path][0]) > 0:
            continue  # placeholder of a leaf owned elsewhere
        gshape, shard = shard_of(path, t) if shard_of else (tuple(t.shape), ShardInfo())
        parts, index = _chunk_grid(gshape, shard)
        chunk_shape = tuple(s // p for s, p in zip(gshape, parts))
        base = root / _leaf_dir(path)
        if is_primary:
            base.mkdir(parents=True, exist_ok=True)
            (base / "zarr.json").write_text(json.dumps(_zarr_json(gshape, chunk_shape, t.dtype)))
            meta[path] = {"shape": list(gshape), "dtype": _ZARR_DTYPES[t.dtype], "chunks": list(parts)}
        if writes_leaf is None or writes_leaf(path):
            files.append((_chunk_file(base, index), _bytes_view(t)))
    write_files(files)
    if is_primary:
        (root / "_METADATA").write_text(json.dumps({"tree_metadata": meta, "use_zarr3": True, "store_array_data_equal_to_fill_value": True}))


def tree_metadata(root: Path) -> dict[str, dict]:
    return json.loads((root / "_METADATA").read_text())["tree_metadata"]


def load_leaf(root: Path, path: str, shard: ShardInfo, dtype: torch.dtype | None = None, device="cpu") -> torch.Tensor:
    """Reads the region of a saved global array that ``shard`` selects, from whatever chunking it was saved with."""
    base = root / _leaf_dir(path)
    z = json.loads((base / "zarr.json").read_text())
    gshape = tuple(z["shape"])
    sdtype = _TORCH_DTYPES[z["data_type"]]
    cshape = tuple(z["chunk_grid"]["configuration"]["chunk_shape"]) if gshape else ()
    lo = [0] * len(gshape)
    hi = list(gshape)
    for dim, idx, n in shard.slices:
        size = (hi[dim] - lo[dim]) // n
        lo[dim], hi[dim] = lo[dim] + idx * size, lo[dim] + (idx + 1) * size
    out = torch.empty([h - l for l, h in zip(lo, hi)], dtype=sdtype)
    ranges = [range(l // c, (h - 1) // c + 1) if h > l else range(0) for l, h, c in zip(lo, hi, cshape)]
    reads, placements = [], []
    for cidx in itertools.product(*ranges):
        buf = torch.empty(cshape, dtype=sdtype)
        reads.append((_chunk_file(base, cidx), buf.reshape(-1).view(torch.uint8).numpy() if buf.numel() else np.zeros(0, np.uint8)))
        placements.append((cidx, buf))
    if not gshape:
        buf = torch.empty((), dtype=sdtype)
        reads.append((_chunk_file(base, ()), buf.reshape(1).view(torch.uint8).numpy()))
        read_files(reads)
        out = buf.clone()
    else:
        read_files(reads)
        for cidx, buf in placements:
            src, dst = [], []
            for d, ci in enumerate(cidx):
                c0 = ci * cshape[d]
                a, b = max(lo[d], c0), min(hi[d], c0 + cshape[d])
                src.append(slice(a - c0, b - c0))
                dst.append(slice(a - lo[d], b - lo[d]))
            out[tuple(dst)] = buf[tuple(src)]
    if dtype is not None and dtype != sdtype:
        out = out.to(dtype)
    return out.to(device)


# --------------------------------------------------------------------------- checkpointables
def _barrier(rt) -> None:
    if rt is not None:
        rt.barrier()


def save_checkpointables(path: Path, checkpointables: dict[str, Any], *, custom_metadata: dict | None = None, rt=None) -> None:
    """Atomic multi-rank save of named checkpointables (pytrees of tensors, or JSON-able dicts)."""
    primary = rt is None or rt.rank == 0
    tmp = path.with_name(path.name + TMP_MARK + "0")
    if primary:
        if tmp.exists():
            shutil.rmtree(tmp)
        tmp.mkdir(parents=True)
    _barrier(rt)
    start_ns = time.time_ns()
    handlers = {}
    for name, value in checkpointables.items():
        root = tmp / name
        if isinstance(value, dict) and all(isinstance(v, (str, int, float, bool, type(None))) for v in value.values()):
            handlers[name] = "json"
            if primary:
                root.mkdir(parents=True, exist_ok=True)
                (root / "metadata").write_text(json.dumps(value))
            continue
        handlers[name] = "pytree"
        save_tree(root, value, shard_of=(rt.shard_of if rt is not None else None),
                  writes_leaf=(rt.writes_leaf if rt is not None else None), is_primary=primary,
                  all_leaves=(rt.checkpoint_leaves(name, value) if rt is not None else None))
    _barrier(rt)
    if primary:
        (tmp / METADATA_FILE).write_text(json.dumps({
            "item_handlers": handlers, "init_timestamp_nsecs": start_ns, "commit_timestamp_nsecs": time.time_ns(),
            "custom_metadata": custom_metadata or {},
        }))
        if path.exists():
            shutil.rmtree(path)
        os.rename(tmp, path)
    _barrier(rt)


def load_checkpointables(path: Path, abstract: dict[str, Any], *, device="cpu", rt=None) -> dict[str, Any]:
    """Restores named checkpointables. Each entry of ``abstract`` is a tree of ``ArraySpec`` (or tensors giving
    shape/dtype), ``None`` for a JSON checkpointable. The saved parameter tree must have exactly the requested
    leaf paths."""
    mismatch = f"Checkpoint {path} does not match the model config; load it with the variant it was trained with."
    out: dict[str, Any] = {}
    for name, tree in abstract.items():
        root = path / name
        if tree is None:
            out[name] = json.loads((root / "metadata").read_text())
            continue
        saved = tree_metadata(root)
        want = tree_dict(tree)
        if name == "params" and set(saved) != set(want):
            raise ValueError(mismatch)

        def load(p, leaf, root=root, saved=saved):
            if p not in saved:
                raise ValueError(mismatch)
            gshape = tuple(leaf.shape)
            if tuple(saved[p]["shape"]) != gshape and not isinstance(leaf, torch.Tensor):
                raise ValueError(mismatch)
            shard = rt.shard_info(p, leaf) if (rt is not None and isinstance(leaf, ArraySpec)) else ShardInfo()
            if shard.absent:
                return torch.empty(0, dtype=getattr(leaf, "dtype", torch.float32), device=device)
            return load_leaf(root, p, shard, getattr(leaf, "dtype", None), device)

        out[name] = map_with_path(load, tree)
    return out
