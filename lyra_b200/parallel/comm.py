"""Buffers and data movement behind ``Runtime``: the bf16 weight slab, the gradient slab and the small-leaf
staging area, each allocated once in peer-mapped (symmetric) memory on the ``b200`` path, and the operations on
them - weight gather from the owners, gradient pull-reduce to the owners, small-leaf all-reduce, stream-ordered
cross-rank barriers built from epoch flags. On the ``nccl`` path the same operations are torch.distributed calls."""

from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

BF16 = torch.bfloat16
NVLS = os.environ.get("LYRA_NVLS", "0") == "1"   # replicated-leaf gradients: in-switch all-reduce (multimem) where the allocation has a multicast address
ALIGN = 256  # bytes; every sub-buffer starts on this boundary so 16-byte vector accesses and TMA bases stay aligned


def _ptr_array(ptrs: list[int]):
    return (ctypes.c_longlong * len(ptrs))(*ptrs)


class SymmetricSlab:
    """One peer-mapped allocation of ``nbytes`` on every rank plus everyone's base pointers."""

    def __init__(self, nbytes: int, device, group_name: str):
        import torch.distributed._symmetric_memory as symm_mem

        nbytes = max((nbytes + ALIGN - 1) // ALIGN * ALIGN, ALIGN)
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        # Cleared and finished BEFORE the handle exchange: a peer can store into this buffer as soon as it holds the address,
        # and the exchange cannot complete on any rank before every rank has entered it. (Clearing afterwards let a fast peer's
        # first rows land before a slower owner's queued memset ran, which then wiped them.)
        self.buffer.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm_mem.rendezvous(self.buffer, group_name)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        # address through which NVSwitch reduces / broadcasts over every rank's copy (0 where multicast is not available)
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)

    def view(self, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        return self.buffer[offset:offset + nbytes].view(dtype)

    def peers_at(self, offset: int) -> list[int]:
        return [p + offset for p in self.peer_ptrs]


class Comm:
    def __init__(self, rt, entries: list[tuple[str, tuple[int, ...], int]], grad_dtype: torch.dtype):
        self.rt = rt
        self.world, self.rank, self.device = rt.world, rt.rank, rt.device
        self.p2p = rt.implementation == "b200"
        self.entries = entries
        self.entries_by_name = {name: (shape, owner) for name, shape, owner in entries}
        self.grad_dtype = grad_dtype
        gsize = torch.empty((), dtype=grad_dtype).element_size()
        self.w_dtype = BF16 if rt.mcfg.compute_dtype == BF16 or self.p2p else rt.mcfg.compute_dtype
        self.w_size = torch.empty((), dtype=self.w_dtype).element_size()
        self.w_off, self.g_off, self.numel, self.owner = {}, {}, {}, {}
        w_total = g_total = 0
        for name, shape, owner in entries:
            n = math.prod(shape)
            self.numel[name], self.owner[name] = n, owner
            self.w_off[name], self.g_off[name] = w_total, g_total
            w_total += (n * self.w_size + ALIGN - 1) // ALIGN * ALIGN
            g_total += (n * gsize + ALIGN - 1) // ALIGN * ALIGN
        self.small_cap = 16 << 20  # bytes of replicated-leaf gradients (fp32)
        if self.p2p:
            from lyra_b200.ops import native

            self.native = native
            self.lib = native.kernels()
            name = dist.group.WORLD.group_name
            self.w_slab = SymmetricSlab(w_total, self.device, name)
            self.g_slab = SymmetricSlab(g_total, self.device, name)
            self.small_slab = SymmetricSlab(self.small_cap, self.device, name)
            self.flag_slab = SymmetricSlab(4096, self.device, name)   # [0:64) barrier flags, [64:128) EP count flags, [128:192) EP data flags
            self.epoch = 0
            self.w_buf, self.g_buf = self.w_slab.buffer, self.g_slab.buffer
        else:
            self.w_buf = torch.zeros(max(w_total, ALIGN), dtype=torch.uint8, device=self.device)
            self.g_buf = torch.zeros(max(g_total, ALIGN), dtype=torch.uint8, device=self.device)
        # "fused": eligible weights are not pulled eagerly; the first forward GEMM that uses one pulls it inside the kernel
        self.fused_gather = self.p2p and os.environ.get("LYRA_GATHER", "fused") == "fused"
        self.pending: dict[str, bool] = {}
        self.ag_flags: dict[str, torch.Tensor] = {}
        self.ag_calls: dict[str, int] = {}
        self._grad_views: dict[int, torch.Tensor] = {}
        self._reduced: dict[str, torch.Tensor] = {}
        self._sq_partial: torch.Tensor | None = None
        self.grad_sumsq: dict[str, torch.Tensor] = {}            # owned leaf -> sum of squares of its reduced gradient, per matrix
        for name, shape, owner in entries:
            if owner == self.rank:
                self._reduced[name] = torch.empty((self.numel[name] + 7) // 8 * 8, dtype=torch.float32 if grad_dtype == torch.float32 else BF16, device=self.device)

    # ------------------------------------------------------------------ views
    def weight_view(self, name: str) -> torch.Tensor:
        off, n = self.w_off[name], self.numel[name]
        return self.w_buf[off:off + self.w_size * n].view(self.w_dtype)

    def grad_view(self, name: str) -> torch.Tensor:
        off, n = self.g_off[name], self.numel[name]
        size = torch.empty((), dtype=self.grad_dtype).element_size()
        return self.g_buf[off:off + size * n].view(self.grad_dtype)

    def grad_view_of(self, w: torch.Tensor) -> torch.Tensor:
        key = id(w)
        if key not in self._grad_views:
            name = next(n for n, v in self.rt._views.items() if v is w)
            self._grad_views[key] = self.grad_view(name).view(w.shape)
        return self._grad_views[key]

    def zero_grads(self) -> None:
        self.g_buf.zero_()

    # ------------------------------------------------------------------ barriers
    def barrier(self) -> None:
        """Stream-ordered barrier: every rank raises its flag on all peers, then waits for all flags of this epoch."""
        if not self.p2p:
            dist.barrier()
            return
        self.epoch += 1
        nat = self.native
        stream = nat.stream_ptr()
        nat.check(self.lib.lyra_signal(_ptr_array(self.flag_slab.peers_at(0)), self.world, self.rank, self.epoch, stream), "signal")
        nat.check(self.lib.lyra_wait(ctypes.c_void_p(self.flag_slab.buffer.data_ptr()), self.world, self.epoch,
                                     nat.ptr(nat.status_word()), stream), "wait")
        nat.count_launch(2)

    # ------------------------------------------------------------------ weights: owner -> everyone
    @torch.no_grad()
    def gather_weights(self) -> None:
        if not self.p2p:
            for name, shape, owner in self.entries:
                dist.broadcast(self.weight_view(name), src=owner)
            return
        nat = self.native
        self.barrier()                                           # owners have written their bf16 copies
        stream = nat.stream_ptr()
        order = sorted(range(len(self.entries)), key=lambda i: ((self.entries[i][2] - self.rank - 1) % self.world, i))
        for i in order:                                          # start with the next rank's leaves: spreads the load over owners
            name, shape, owner = self.entries[i]
            if owner == self.rank:
                continue
            if self.fused_gather and self._fusable(name, shape):
                self.pending[name] = True
                continue
            off, n = self.w_off[name], self.numel[name]
            nbytes = (n * 2 + 15) // 16 * 16
            nat.check(self.lib.lyra_p2p_copy(ctypes.c_void_p(self.w_buf.data_ptr() + off), ctypes.c_void_p(self.w_slab.peer_ptrs[owner] + off),
                                             ctypes.c_longlong(nbytes), stream), "p2p_copy")
            nat.count_launch()
        self.barrier()                                           # nobody overwrites a copy that is still being pulled

    def _fusable(self, name: str, shape: tuple[int, ...]) -> bool:
        """Weights consumed as the ``[K, N]`` operand of a forward linear: K rows of N contiguous columns, K % 64 == 0."""
        leaf = name.split("#")[0].split("/")[-1]
        if leaf in ("emb", "unemb"):
            return False
        return len(shape) in (2, 3) and shape[0] % 64 == 0 and math.prod(shape[1:]) % 8 == 0

    def ag_info(self, name: str):
        """Description of the pending fused pull of ``name`` for ``ops.gemm.gemm_allgather``, or None."""
        if not self.pending.get(name):
            return None
        if name not in self.ag_flags:
            n_cols = self.numel[name] // self.entries_by_name[name][0][0]
            self.ag_flags[name] = torch.zeros((n_cols + 255) // 256, dtype=torch.int32, device=self.device)
            self.ag_calls[name] = 0
        owner = self.owner[name]

        def done():
            self.pending[name] = False
            self.ag_calls[name] += 1

        # the kernel's slab counters grow by one per piece and call, so the epoch is this leaf's own call number
        return {"src": [self.w_slab.peer_ptrs[owner] + self.w_off[name]], "my_rank": 1, "flags": self.ag_flags[name],
                "epoch": self.ag_calls[name] + 1, "done": done}

    def finish_pending(self) -> None:
        """Pulls whatever was not touched by a forward pass (e.g. before a checkpoint of compute copies or an eval of part of the model)."""
        nat = self.native
        for name, todo in list(self.pending.items()):
            if todo:
                off, n, owner = self.w_off[name], self.numel[name], self.owner[name]
                nat.check(self.lib.lyra_p2p_copy(ctypes.c_void_p(self.w_buf.data_ptr() + off), ctypes.c_void_p(self.w_slab.peer_ptrs[owner] + off),
                                                 ctypes.c_longlong((n * 2 + 15) // 16 * 16), nat.stream_ptr()), "p2p_copy")
                self.pending[name] = False

    # ------------------------------------------------------------------ gradients: everyone -> owner
    @torch.no_grad()
    def reduce_grads(self) -> dict[str, torch.Tensor]:
        out = {}
        if not self.p2p:
            for name, shape, owner in self.entries:
                g = self.grad_view(name)
                dist.reduce(g, dst=owner)
                if owner == self.rank:
                    out[name] = g
            return out
        nat = self.native
        if self.fused_gather:
            self.finish_pending()                                # a leaf no forward touched is pulled before its owner may rewrite it
        self.barrier()                                           # every rank finished accumulating
        stream = nat.stream_ptr()
        in_bf16 = int(self.grad_dtype == BF16)
        owned = [(name, shape) for name, shape, owner in self.entries if owner == self.rank]
        if owned and self._sq_partial is None:
            # per-block sums of squares of every owned leaf's reduced gradient, written by the pull-reduce itself; a leaf's block
            # count never changes, so the unused tail of its row stays zero and one sum over the block axis finishes all leaves
            self.lib.lyra_reduce_pull_norm_blocks.restype = ctypes.c_int
            blocks = [int(self.lib.lyra_reduce_pull_norm_blocks(ctypes.c_longlong((self.numel[n] + 7) // 8 * 8))) for n, _ in owned]
            self._sq_partial = torch.zeros(len(owned), max(blocks), 2, dtype=torch.float32, device=self.device)
        for i, (name, shape) in enumerate(owned):
            n = self.numel[name]
            n8 = (n + 7) // 8 * 8                                # every leaf's region is 256-byte aligned and its padding stays zero
            dst = self._reduced[name]                            # (padded to n8 elements)
            # a [C, 2, H] up-projection interleaves two matrices (gate and linear halves) in runs of H elements
            halves = name.split("#")[0].endswith("mlp_up") and len(shape) == 3 and shape[1] == 2 and shape[2] % 8 == 0
            nat.check(self.lib.lyra_reduce_pull_norm(nat.ptr(dst), _ptr_array(self.g_slab.peers_at(self.g_off[name])), self.world,
                                                     ctypes.c_longlong(n8), in_bf16, in_bf16, ctypes.c_longlong(shape[2] if halves else 0),
                                                     2 if halves else 1, nat.ptr(self._sq_partial[i]), stream), "reduce_pull_norm")
            nat.count_launch()
            out[name] = dst[:n]
        self.grad_sumsq = {}
        if owned:
            sums = self._sq_partial.sum(1)                       # [leaves, 2], fixed summation order
            for i, (name, shape) in enumerate(owned):
                halves = name.split("#")[0].endswith("mlp_up") and len(shape) == 3 and shape[1] == 2 and shape[2] % 8 == 0
                self.grad_sumsq[name] = sums[i, : 2 if halves else 1]
        self.barrier()                                           # buffers may be zeroed for the next step after this
        return out

    @torch.no_grad()
    def all_reduce_small(self, grads: dict[str, torch.Tensor]) -> None:
        """Sums the gradients of replicated leaves over ranks, in place, identically on every rank."""
        if not grads:
            return
        names = sorted(grads)
        flat = torch.cat([grads[n].reshape(-1).float() for n in names])
        if not self.p2p or flat.numel() * 4 > self.small_cap:
            dist.all_reduce(flat)
        elif NVLS and self.small_slab.multicast_ptr:
            # in-switch reduction: one multimem.ld_reduce per element of this rank's slice instead of `world` peer loads per element
            nat = self.native
            n = flat.numel()
            pad = 4 * self.world
            npad = (n + pad - 1) // pad * pad
            stage = self.small_slab.view(0, npad, torch.float32)
            stage.zero_()
            stage[:n] = flat
            self.barrier()
            nat.check(self.lib.lyra_multimem_all_reduce(ctypes.c_void_p(self.small_slab.multicast_ptr), ctypes.c_longlong(npad), self.world, self.rank,
                                                        nat.stream_ptr()), "multimem_all_reduce")
            nat.count_launch()
            self.barrier()
            flat = stage[:n].clone()
        else:
            nat = self.native
            n = flat.numel()
            n8 = (n + 7) // 8 * 8
            stage = self.small_slab.view(0, n8, torch.float32)
            stage.zero_()
            stage[:n] = flat
            self.barrier()
            out = torch.empty(n8, dtype=torch.float32, device=self.device)
            nat.check(self.lib.lyra_reduce_pull(nat.ptr(out), _ptr_array(self.small_slab.peers_at(0)), self.world, ctypes.c_longlong(n8), 0, 0,
                                                nat.stream_ptr()), "reduce_pull small")
            nat.count_launch()
            self.barrier()
            flat = out[:n]
        off = 0
        for name in names:
            g = grads[name]
            g.copy_(flat[off:off + g.numel()].view(g.shape).to(g.dtype))
            off += g.numel()
