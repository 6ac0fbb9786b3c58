"""Expert-parallel mixture-of-experts layer: dropless token exchange + local grouped expert MLP + weighted combine
(the job of lyra/kernels/ep_moe.py in the reference, which off-TPU falls back to a dense [E, N, C] all-to-all).

Receive layout on the expert's rank: expert-major, then source-rank-major (lyra/kernels/ep_moe.py:9-37), every expert's
rows padded to a multiple of 128 so each GEMM tile belongs to one expert.

* ``b200`` path: counts are pushed into every peer's counts matrix, each rank derives the full layout on the device,
  token rows are stored straight into the owner's receive buffer over NVLink, epoch flags order the phases, and expert
  outputs are stored straight back into the source rank's combine buffer. No host synchronisation, no collective call.
* ``nccl`` path (baseline / CPU): the same exchange with ``all_to_all_single`` and host-side split sizes.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from lyra_b200.config import ModelConfig
from lyra_b200.ops import api as ops
from lyra_b200.ops import reference as ref

from lyra_b200.nn.quant import QArray, dequantize
from lyra_b200.utils.phases import span

BF16 = torch.bfloat16
EP_DECODE_MAX_ROWS = 512   # assignments per rank up to which an inference exchange uses the weight-streaming small-M products
FUSED_RETURN = os.environ.get("LYRA_EP_FUSED_RETURN", "1") != "0"   # expert outputs leave through the GEMM epilogue (peer stores), no return kernel
CAPACITY = float(os.environ.get("LYRA_EP_CAPACITY", "4.0"))  # receive-buffer rows as a multiple of the balanced load (never above the world size)


def ep_moe_forward(rt, xn, scores, indices, w, c: ModelConfig):
    Kr = c.n_active_routed_experts
    r_scores, r_idx = scores[:, :Kr].contiguous(), indices[:, :Kr].contiguous()
    quantised = isinstance(w.mlp_up, QArray) or isinstance(w.mlp_down, QArray)
    shared_done = 0
    if rt.implementation == "b200" and xn.is_cuda and quantised:   # bf16 experts: the tile GEMM path below is the faster one (measured, EP2)
        out = _ep_moe_decode(rt, xn.contiguous(), r_scores.float(), r_idx, w, c)
    elif rt.implementation == "b200" and xn.is_cuda:
        # the first shared expert (score 1 by construction, lyra/model.py:474) runs inside the exchange, where it fills the wait for
        # the routed rows to come back
        sh_up = sh_down = None
        if c.n_shared_experts and ops.use_kernels(xn, c.implementation):
            sh_up, sh_down = rt.shared_expert_weights(w.mlp_up, w.mlp_down, 0)
            shared_done = 1
        out = _EPMoEKernel.apply(xn.contiguous(), r_scores.float(), r_idx, w.mlp_up, w.mlp_down, w.mlp_up_bias, w.mlp_down_bias, sh_up, sh_down, rt, c)
    else:
        out = _ep_moe_collectives(rt, xn, r_scores, r_idx, w, c)
    for j in range(shared_done, c.n_shared_experts):
        up, down = rt.shared_expert_weights(w.mlp_up, w.mlp_down, j)
        impl = c.implementation
        h = ops.linear_swiglu(xn, up, None, c.swiglu_beta, c.swiglu_limit, impl)
        o = ops.linear(h, down, None, impl)
        out = out + o * scores[:, Kr + j, None].to(o.dtype)
    return out


@torch.no_grad()
def _ep_moe_decode(rt, xn, scores, indices, w, c: ModelConfig):
    """Inference-only exchange for a handful of rows per expert: dispatch into the owners' receive buffers, the two expert
    products with the small-M weight-streaming kernel (bf16 or block-scaled e4m3 weights, empty experts skipped), return,
    weighted combine. Large row counts with quantised weights dequantise the local experts and use the tile GEMM."""
    from lyra_b200.nn.quant import dequantize
    from lyra_b200.ops import cuda_ops, decode as dec, elementwise as ew, gemm as G

    F_, K = indices.shape
    C = xn.shape[1]
    up, down = w.mlp_up, w.mlp_down
    El = (up.qval if isinstance(up, QArray) else up).shape[0]
    wu = up if isinstance(up, QArray) else cuda_ops.bf16_weight(up).view(El, C, -1)
    wd = down if isinstance(down, QArray) else cuda_ops.bf16_weight(down)
    n_up = (wu.qval if isinstance(wu, QArray) else wu).shape[-1]
    H = n_up // 2
    ub = cuda_ops.fp32_param(w.mlp_up_bias).reshape(El, n_up) if w.mlp_up_bias is not None else None
    db = cuda_ops.fp32_param(w.mlp_down_bias).reshape(El, C) if w.mlp_down_bias is not None else None
    ex = _Exchange(rt, indices, C)
    bufs = ex.buf.for_layer(-1)
    small = F_ * K <= EP_DECODE_MAX_ROWS and dec.decode_gemm_supported(C, n_up, wu) and dec.decode_gemm_supported(H, C, wd)
    x_recv = ex.dispatch(xn.to(BF16), K, bufs["recv"], bufs["meta"], pad=not small)   # the small-M products read real rows only
    if small:
        valid = ex.valid                                         # real rows per local expert, from the layout kernel
        most = ex.W * F_ * K                                     # an expert can receive at most every assignment of every rank
        usual = -(-2 * most // ex.E)                             # twice the balanced load
        act = dec.decode_gemm(x_recv, wu, offsets=ex.offsets, counts=valid, bias=ub, swiglu=True, swiglu_beta=c.swiglu_beta,
                              swiglu_limit=c.swiglu_limit, active_groups=El, max_group_rows=most, typical_group_rows=usual)
        rows = dec.decode_gemm(act, wd, offsets=ex.offsets, counts=valid, bias=db, active_groups=El, max_group_rows=most, typical_group_rows=usual)
    else:
        wu_t = dequantize(wu, BF16) if isinstance(wu, QArray) else wu
        wd_t = dequantize(wd, BF16) if isinstance(wd, QArray) else wd
        cap = ex.buf.cap
        act = G.grouped_gemm(x_recv, wu_t, ex.tile_group, bias=ub, swiglu=True, swiglu_beta=c.swiglu_beta, swiglu_limit=c.swiglu_limit,
                             out=torch.empty(cap, H, dtype=BF16, device=xn.device))
        rows = G.grouped_gemm(act, wd_t, ex.tile_group, bias=db, out=torch.empty(cap, C, dtype=BF16, device=xn.device))
    ret = ex.collect(rows, bufs["meta"], bufs["ret"])
    ident = rt._ep_state.setdefault("ident", {})
    if F_ * K not in ident:
        ident[F_ * K] = torch.arange(F_ * K, device=xn.device)
    return ew.combine_rows(ret, ident[F_ * K], scores, F_, K)


# ============================================================================================ baseline: collectives
class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send_splits, recv_splits, group):
        ctx.splits, ctx.group = (send_splits, recv_splits), group
        out = x.new_empty(sum(recv_splits), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), recv_splits, send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        send_splits, recv_splits = ctx.splits
        out = g.new_empty(sum(send_splits), *g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), send_splits, recv_splits, group=ctx.group)
        return out, None, None, None


def _ep_moe_collectives(rt, xn, scores, indices, w, c: ModelConfig):
    F_, K = indices.shape
    E, El, W = c.n_experts, rt.e_local, rt.world
    flat = indices.reshape(-1)
    order = torch.argsort(flat, stable=True)                       # assignments sorted by expert (= by destination rank)
    counts = torch.bincount(flat, minlength=E)
    all_counts = [torch.zeros_like(counts) for _ in range(W)]
    dist.all_gather(all_counts, counts, group=rt.group)
    all_counts = torch.stack(all_counts)                           # [source, expert]
    send_splits = counts.view(W, El).sum(1).tolist()
    recv_counts = all_counts[:, rt.rank * El:(rt.rank + 1) * El]   # [source, local expert]
    recv_splits = recv_counts.sum(1).tolist()
    rows = xn[order // K]
    recv = _AllToAll.apply(rows, send_splits, recv_splits, rt.group)   # source-major, expert-sorted within a source
    # reorder to expert-major
    src_id = torch.repeat_interleave(torch.arange(W, device=xn.device), torch.tensor(recv_splits, device=xn.device))
    exp_id = torch.cat([torch.repeat_interleave(torch.arange(El, device=xn.device), recv_counts[s]) for s in range(W)]) if recv.shape[0] else src_id
    up, down = w.mlp_up, w.mlp_down
    if (ops.use_kernels(xn, c.implementation) and recv.shape[0] > 0 and not isinstance(up, QArray) and not isinstance(down, QArray)):
        # collectives for the exchange, this repository's kernels for the local expert MLP (each received row is a "token" with one
        # expert and score 1): the comparison point for the peer-memory exchange with everything else equal
        t = ops.moe_experts(recv.contiguous(), recv.new_ones(recv.shape[0], 1, dtype=torch.float32), exp_id[:, None].contiguous(), up, w.mlp_up_bias,
                            down, w.mlp_down_bias, c.swiglu_beta, c.swiglu_limit, c.implementation)
        back = _AllToAll.apply(t, recv_splits, send_splits, rt.group)          # rows in `order` order
        unsort = torch.empty_like(order)
        unsort[order] = torch.arange(order.numel(), device=order.device)
        ret = back[unsort].view(F_, K, xn.shape[-1])
        return torch.einsum("fkc,fk->fc", ret.float(), scores.float()).to(xn.dtype)
    perm = torch.argsort(exp_id * W + src_id, stable=True)
    grouped = recv[perm]
    groups = recv_counts.sum(0)
    if isinstance(up, QArray):                                   # block-scaled e4m3 experts (inference): this mode dequantises them
        up = dequantize(up, xn.dtype).reshape(El, xn.shape[-1], 2, -1)
    if isinstance(down, QArray):
        down = dequantize(down, xn.dtype)
    C, H = up.shape[1], up.shape[3]
    t = ref.grouped_gemm_autograd(grouped, up.reshape(El, C, 2 * H), groups, None if w.mlp_up_bias is None else w.mlp_up_bias.reshape(El, 2 * H))
    t = ref.swiglu(t.reshape(-1, 2, H), c.swiglu_beta, c.swiglu_limit).to(xn.dtype)
    t = ref.grouped_gemm_autograd(t, down, groups, w.mlp_down_bias)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), device=perm.device)
    back = _AllToAll.apply(t[inv], recv_splits, send_splits, rt.group)      # rows in `order` order
    unsort = torch.empty_like(order)
    unsort[order] = torch.arange(order.numel(), device=order.device)
    ret = back[unsort].view(F_, K, C)
    return torch.einsum("fkc,fk->fc", ret.float(), scores.float()).to(xn.dtype)


# ============================================================================================ product: peer-memory kernels
# Flag slots of the runtime's flag slab (bytes): [64:128) counts exchange, [128:192) dispatch phase and [192:256) return phase of
# the barrier-ordered exchange, [256:320) "backward receive scratch is free again" of the tile-granular exchange.
FLAG_COUNTS, FLAG_DISPATCH, FLAG_RETURN, FLAG_SCRATCH_FREE = 64, 128, 192, 256
_CTR_OF_FLAG = {FLAG_COUNTS: 0, FLAG_DISPATCH: 1, FLAG_RETURN: 2, FLAG_SCRATCH_FREE: 3}
FWD, BWD = 0, 1


class EPBuffers:
    """Peer-mapped buffers of the exchange, created on first use (the same order on every rank)."""

    def __init__(self, rt, F_: int, K: int, C: int, layers: list[int] | None = None):
        from lyra_b200.parallel.comm import SymmetricSlab

        self.rt = rt
        name = dist.group.WORLD.group_name
        E, W = rt.mcfg.n_experts, rt.world
        self.cap = ((int(min(CAPACITY, float(W)) * F_ * K) + 127) // 128 + rt.e_local) * 128
        self.A = F_ * K
        dev = rt.device
        self.counts = [SymmetricSlab(W * E * 4, dev, name) for _ in range(2)]
        self._scratch: dict[str, list] = {}                      # backward-pass buffers, created by the first backward
        self.layer: dict[int, dict] = {}
        self.calls = 0
        self.C, self.name = C, name
        # tile-granular exchange: arrival counters that peers bump (per 128-row tile and direction, then one per direction for
        # returned rows), and this rank's running totals of what it expects. Counters only grow; nothing is ever reset.
        self.n_tiles = self.cap // 128
        self._sync = SymmetricSlab((2 * self.n_tiles + 64) * 4, dev, name)
        self.expect = torch.zeros(2 * self.n_tiles, dtype=torch.int32, device=dev)
        self.ret_expect = torch.zeros(2, dtype=torch.int32, device=dev)
        if layers is not None:
            # Everything a step will need, now, in one place: creating a peer-mapped buffer stalls the host (handle exchange), and a
            # rank stalled in the middle of a step keeps its peers' GPUs spinning in their bounded waits. After this, steps allocate
            # no peer-mapped memory.
            for idx in layers:
                self.for_layer(idx)
            if any(i >= 0 for i in layers):                      # training: the backward pass's scratch as well
                self.scratch_recv, self.scratch_ret
            torch.cuda.synchronize(dev)
            dist.barrier()

    def arrive_view(self, direction: int) -> torch.Tensor:
        return self._sync.view(direction * self.n_tiles * 4, self.n_tiles, torch.int32)

    def arrive_peers(self, direction: int) -> list[int]:
        return self._sync.peers_at(direction * self.n_tiles * 4)

    def expect_view(self, direction: int) -> torch.Tensor:
        return self.expect[direction * self.n_tiles:(direction + 1) * self.n_tiles]

    def returned_view(self, direction: int) -> torch.Tensor:
        return self._sync.view((2 * self.n_tiles + direction) * 4, 1, torch.int32)

    def returned_peers(self, direction: int) -> list[int]:
        return self._sync.peers_at((2 * self.n_tiles + direction) * 4)

    def _lazy(self, kind: str, nbytes: int) -> list:
        from lyra_b200.parallel.comm import SymmetricSlab

        if kind not in self._scratch:                            # same call order on every rank (symmetric allocation is collective)
            self._scratch[kind] = [SymmetricSlab(nbytes, self.rt.device, self.name) for _ in range(2)]
        return self._scratch[kind]

    @property
    def scratch_recv(self) -> list:
        """Backward receive buffers (two, by call parity); inference never allocates them."""
        return self._lazy("recv", self.cap * self.C * 2)

    @property
    def scratch_ret(self) -> list:
        return self._lazy("ret", self.A * self.C * 2)

    def for_layer(self, idx: int) -> dict:
        from lyra_b200.parallel.comm import SymmetricSlab

        if idx not in self.layer:
            dev = self.rt.device
            self.layer[idx] = {
                "recv": SymmetricSlab(self.cap * self.C * 2, dev, self.name),
                "meta": SymmetricSlab(self.cap * 4, dev, self.name),
                "score": SymmetricSlab(self.cap * 4, dev, self.name),
                "ret": SymmetricSlab(self.A * self.C * 2, dev, self.name),
            }
        return self.layer[idx]


def _arr(ptrs):
    return (ctypes.c_longlong * len(ptrs))(*ptrs)


class _Exchange:
    """One routing decision: layout + the dispatch / return primitives for both directions.

    Two protocols share the layout. The barrier-ordered one (``tiles=False``; decode, and the comparison path) separates
    dispatch, expert products and return with all-rank flag phases. The tile-granular one (``tiles=True``) has no phase
    barrier: senders bump one arrival counter per 128-row tile of the receiver's buffer and the receiver's first grouped GEMM
    waits per tile inside its TMA producer (``dispatch_tiles`` + ``gemm_waits``); the down-projection's epilogue counts the
    rows it stores on each source rank, which waits for exactly its own rows (``wait_returned``)."""

    def __init__(self, rt, indices: torch.Tensor, C: int, tiles: bool = False):
        from lyra_b200.ops import native

        self.rt, self.nat, self.lib = rt, native, native.kernels()
        F_, K = indices.shape
        key = (F_, K, C)
        sets = rt._ep_state.setdefault("sets", {})               # one buffer set per problem size (prefill and decode alternate)
        if key not in sets:
            moe_layers = [i for i, kind in enumerate(rt.mcfg.mlp_map) if kind == "moe"]
            sets[key] = EPBuffers(rt, F_, K, C, layers=(moe_layers + [-1]) if torch.is_grad_enabled() else [-1])
        rt._ep_state["key"], rt._ep_state["buf"] = key, sets[key]
        self.buf: EPBuffers = sets[key]
        self.F, self.K, self.C = F_, K, C
        self.W, self.E, self.El, self.rank = rt.world, rt.mcfg.n_experts, rt.e_local, rt.rank
        self.tiles = tiles
        comm = rt._comm
        self.flags = comm.flag_slab
        dev = indices.device
        flat = indices.reshape(-1)
        self.expert_of = flat.to(torch.int32).contiguous()
        plan = getattr(rt, "routing_plan", None)                 # counts and permutation already made by the routing kernels of this layer call
        rt.routing_plan = None
        if plan is not None and plan.order.numel() == flat.numel() and plan.counts.numel() <= self.E:
            if plan.counts.numel() == self.E:                    # no shared experts behind the routed ones: the plan's counts as they are
                counts = plan.counts
            else:
                counts = torch.zeros(self.E, dtype=torch.int32, device=dev)
                counts[: plan.counts.numel()] = plan.counts
            self.order, self.rank_in_expert = plan.order, plan.rank_in_expert
        else:
            counts = ref.count_ids(flat, self.E).to(torch.int32)
            order = torch.argsort(flat, stable=True)
            if tiles:
                self.order = order.to(torch.int32)
            else:
                starts = torch.cumsum(counts, 0) - counts
                rie = torch.empty_like(order)
                rie[order] = torch.arange(flat.numel(), device=dev) - starts[flat[order]].long()
                self.rank_in_expert = rie.to(torch.int32).contiguous()
        # counts exchange
        self.buf.calls += 1
        par = self.buf.calls & 1
        self.counts_slab = self.buf.counts[par]
        stream = native.stream_ptr()
        # epochs live in device counters (one per flag slot), so the launch sequence is the same every time and can be
        # replayed from a CUDA graph
        if getattr(rt, "_ep_ctr", None) is None:
            rt._ep_ctr = torch.zeros(4, dtype=torch.int32, device=dev)
        self.ctr = rt._ep_ctr
        native.check(self.lib.lyra_ep_counts_push_ctr(native.ptr(counts), _arr(self.counts_slab.peer_ptrs), _arr(self.flags.peers_at(FLAG_COUNTS)), self.W,
                                                      self.rank, self.E, ctypes.c_void_p(self.ctr.data_ptr()), stream), "ep_counts_push")
        with span("ep_wait"):
            native.check(self.lib.lyra_wait_ctr(ctypes.c_void_p(self.flags.buffer.data_ptr() + FLAG_COUNTS), self.W, ctypes.c_void_p(self.ctr.data_ptr()),
                                                native.ptr(native.status_word()), stream), "wait")
        # A training exchange keeps a private copy for its backward pass (the slab is rewritten by the call after next). An
        # inference call is over before that: a peer's push of the call after next follows this rank's push of the next call,
        # which this rank's stream runs after everything of this call.
        self.counts_mat = self.counts_slab.view(0, self.W * self.E, torch.int32)
        if torch.is_grad_enabled():
            self.counts_mat = self.counts_mat.clone()
        nt = self.buf.n_tiles
        ints = torch.empty(self.E + (self.El + 1) + nt + 1 + self.El + (2 * (self.E + 1) + 2 * nt if tiles else 0), dtype=torch.int32, device=dev)
        parts = [self.E, self.El + 1, nt, 1, self.El] + ([self.E + 1, self.E + 1, nt, nt] if tiles else [])
        views = torch.split(ints, parts)
        self.send_base, self.offsets, self.tile_group, self.total, self.valid = views[:5]
        if tiles:
            self.starts, self.send_starts, self.tile_valid, self.tile_perm = views[5:]
            native.check(self.lib.lyra_ep_layout_tiles(native.ptr(self.counts_mat), self.W, self.rank, self.E, self.El, self.buf.cap,
                                                       native.ptr(self.send_base), native.ptr(self.offsets), native.ptr(self.tile_group),
                                                       native.ptr(self.total), native.ptr(self.starts), native.ptr(self.send_starts),
                                                       native.ptr(self.tile_valid), native.ptr(self.tile_perm), native.ptr(native.status_word()),
                                                       stream), "ep_layout_tiles")
        else:
            native.check(self.lib.lyra_ep_layout(native.ptr(self.counts_mat), self.W, self.rank, self.E, self.El, self.buf.cap, native.ptr(self.send_base),
                                                 native.ptr(self.offsets), native.ptr(self.tile_group), native.ptr(self.total), native.ptr(self.valid),
                                                 native.ptr(native.status_word()), stream), "ep_layout")
        native.count_launch(3)

    # ---------------------------------------------------------------------------------- flags
    def signal(self, flag_offset: int) -> None:
        """Raises this rank's flag of the slot on every peer (epoch = the slot's device counter + 1)."""
        ctr = ctypes.c_void_p(self.ctr.data_ptr() + 4 * _CTR_OF_FLAG[flag_offset])
        self.nat.check(self.lib.lyra_signal_ctr(_arr(self.flags.peers_at(flag_offset)), self.W, self.rank, ctr, self.nat.stream_ptr()), "signal")
        self.nat.count_launch()

    def wait(self, flag_offset: int) -> None:
        """Waits until every rank's flag of the slot has reached this rank's device counter of the slot."""
        nat = self.nat
        ctr = ctypes.c_void_p(self.ctr.data_ptr() + 4 * _CTR_OF_FLAG[flag_offset])
        with span("ep_wait"):
            nat.check(self.lib.lyra_wait_ctr(ctypes.c_void_p(self.flags.buffer.data_ptr() + flag_offset), self.W, ctr, nat.ptr(nat.status_word()),
                                             nat.stream_ptr()), "wait")
        nat.count_launch()

    def _phase(self, flag_offset: int) -> None:
        """Raises this rank's flag on all peers and waits for everyone's: all stores of the phase have landed."""
        self.signal(flag_offset)
        self.wait(flag_offset)

    # ---------------------------------------------------------------------------------- barrier-ordered protocol
    def dispatch(self, src: torch.Tensor, src_div: int, recv_slab, meta_slab, pad: bool = True) -> torch.Tensor:
        """``pad=False``: the padding rows of the groups keep whatever they held (for consumers that read real rows only)."""
        nat = self.nat
        nat.check(self.lib.lyra_ep_dispatch(nat.ptr(src), nat.ptr(self.expert_of), nat.ptr(self.rank_in_expert), nat.ptr(self.send_base),
                                            _arr(recv_slab.peer_ptrs), _arr(meta_slab.peer_ptrs) if meta_slab is not None else None, self.W, self.rank,
                                            self.El, self.buf.cap, self.F * self.K, src_div, self.C, nat.stream_ptr()), "ep_dispatch")
        self._phase(FLAG_DISPATCH)
        nat.count_launch()
        if not pad:
            return recv_slab.view(0, self.buf.cap * self.C, BF16).view(self.buf.cap, self.C)
        return self._zero_pad(recv_slab)

    def _zero_pad(self, recv_slab) -> torch.Tensor:
        nat = self.nat
        recv = recv_slab.view(0, self.buf.cap * self.C, BF16).view(self.buf.cap, self.C)
        nat.check(self.lib.lyra_ep_zero_pad(nat.ptr(recv), nat.ptr(self.offsets), nat.ptr(self.counts_mat), self.W, self.rank, self.E, self.El,
                                            self.buf.cap, self.C, nat.stream_ptr()), "ep_zero_pad")
        nat.count_launch()
        return recv

    def build_row_dest(self, meta_slab) -> torch.Tensor:
        """Scatter map of this exchange's receive buffer: ``rank << 24 | slot`` of the assignment each real row came from, -1
        for padding (valid once the dispatch has landed; the return leg of forward and backward both use it)."""
        nat = self.nat
        self.row_dest = torch.empty(self.buf.cap, dtype=torch.int32, device=self.offsets.device)
        meta = meta_slab.view(0, self.buf.cap, torch.int32)
        nat.check(self.lib.lyra_ep_row_dest(nat.ptr(meta), nat.ptr(self.offsets), nat.ptr(self.counts_mat), self.W, self.rank, self.E, self.El,
                                            self.buf.cap, nat.ptr(self.row_dest), nat.stream_ptr()), "ep_row_dest")
        nat.count_launch()
        return self.row_dest

    def returned(self, ret_slab) -> torch.Tensor:
        """After a product whose epilogue stored its rows into the source ranks' return buffers: wait until every rank's
        stores have landed, then view this rank's buffer ``[F*K, C]``."""
        self._phase(FLAG_RETURN)
        return ret_slab.view(0, self.F * self.K * self.C, BF16).view(self.F * self.K, self.C)

    def collect(self, rows: torch.Tensor, meta_slab, ret_slab) -> torch.Tensor:
        nat = self.nat
        meta = meta_slab.view(0, self.buf.cap, torch.int32)
        nat.check(self.lib.lyra_ep_return(nat.ptr(rows), nat.ptr(meta), nat.ptr(self.offsets), nat.ptr(self.counts_mat), self.W, self.rank, self.E,
                                          self.El, _arr(ret_slab.peer_ptrs), self.buf.cap, self.C, nat.stream_ptr()), "ep_return")
        self._phase(FLAG_RETURN)
        nat.count_launch()
        return ret_slab.view(0, self.F * self.K * self.C, BF16).view(self.F * self.K, self.C)

    # ---------------------------------------------------------------------------------- tile-granular protocol
    def dispatch_tiles(self, src: torch.Tensor, src_div: int, recv_slab, meta_slab, direction: int, score_slab=None, scores=None) -> torch.Tensor:
        """Starts the rows on their way and returns the receive buffer at once. Its first reader must be a grouped GEMM given
        ``gemm_waits(direction)``; when that GEMM has finished, every row has landed and later kernels may read the buffer freely."""
        nat, buf = self.nat, self.buf
        stream = nat.stream_ptr()
        nat.check(self.lib.lyra_ep_expect_bump(nat.ptr(buf.expect_view(direction)), nat.ptr(self.tile_valid), buf.n_tiles, stream), "ep_expect_bump")
        recv = self._zero_pad(recv_slab)     # padding rows are never written by a sender, so this may run beside the incoming stores
        nat.check(self.lib.lyra_ep_dispatch_sorted(nat.ptr(src), nat.ptr(self.order), nat.ptr(self.starts), nat.ptr(self.send_base),
                                                   nat.ptr(self.send_starts), nat.ptr(scores) if scores is not None else None, _arr(recv_slab.peer_ptrs),
                                                   _arr(meta_slab.peer_ptrs) if meta_slab is not None else None,
                                                   _arr(score_slab.peer_ptrs) if score_slab is not None else None, _arr(buf.arrive_peers(direction)),
                                                   self.W, self.rank, self.E, self.El, buf.cap, self.F * self.K, src_div, self.C, stream), "ep_dispatch_sorted")
        nat.count_launch(2)
        return recv

    def gemm_waits(self, direction: int) -> dict:
        return {"tile_perm": self.tile_perm, "arrive": self.buf.arrive_view(direction), "expect": self.buf.expect_view(direction)}

    def wait_returned(self, ret_slab, direction: int, n_cols: int) -> torch.Tensor:
        """Waits until the rows this rank dispatched have all come back (every 256-column tile of each), then views them."""
        nat, buf = self.nat, self.buf
        add = self.F * self.K * ((n_cols + 255) // 256)
        with span("ep_wait"):
            nat.check(self.lib.lyra_wait_arrivals(nat.ptr(buf.returned_view(direction)), ctypes.c_void_p(buf.ret_expect.data_ptr() + 4 * direction), add,
                                                  nat.ptr(nat.status_word()), 0, nat.stream_ptr()), "wait_arrivals")
        nat.count_launch()
        return ret_slab.view(0, self.F * self.K * self.C, BF16).view(self.F * self.K, self.C)


TILE_DISPATCH = os.environ.get("LYRA_EP_TILE_DISPATCH", "1") != "0"   # tile-granular exchange (no phase barriers) for the training path
SCORE_IN_EPILOGUE = os.environ.get("LYRA_EP_SCORE_EPILOGUE", "1") != "0"   # the down-projection's epilogue multiplies by the routing score


def _shared_forward(xn, sh_up, sh_down, beta, limit, keep_pre: bool):
    """The shared expert on this rank's own tokens: plain dense products from the replicated bf16 copies (a pending pull of a
    copy from its owner rides inside the first product that uses it)."""
    from lyra_b200.ops import cuda_ops, elementwise as ew, gemm as G

    C, _, H = sh_up.shape
    wu, wd = cuda_ops.bf16_weight(sh_up).view(C, 2 * H), cuda_ops.bf16_weight(sh_down)
    pre = None
    if keep_pre:
        pre = cuda_ops._forward_gemm(xn, sh_up, wu)
        act = ew.swiglu_fwd(pre, beta, limit)
    else:
        if cuda_ops.AG_HOOK is not None and cuda_ops.AG_HOOK(sh_up) is not None:   # land the weight first; the SwiGLU-epilogue GEMM has no fused pull
            cuda_ops._forward_gemm(xn[:128], sh_up, wu)
        act = G.gemm_swiglu(xn, wu, swiglu_beta=beta, swiglu_limit=limit)
    return cuda_ops._forward_gemm(act, sh_down, wd), pre


def _shared_backward(xn, dout, sh_up, sh_down, pre, beta, limit):
    from lyra_b200.ops import cuda_ops, elementwise as ew, gemm as G

    C, _, H = sh_up.shape
    wu, wd = cuda_ops.bf16_weight(sh_up).view(C, 2 * H), cuda_ops.bf16_weight(sh_down)
    if pre is None:
        pre = G.gemm(xn, wu, b_mn=True)
    act = ew.swiglu_fwd(pre, beta, limit)
    if sh_down.requires_grad:
        cuda_ops._accumulate_wgrad(sh_down, act, dout)
    d_act = G.gemm(dout, wd)
    del act
    d_pre = ew.swiglu_bwd(pre, d_act, beta, limit)
    del pre, d_act
    if sh_up.requires_grad:
        cuda_ops._accumulate_wgrad(sh_up, xn, d_pre)
    return G.gemm(d_pre, wu)


class _EPMoEKernel(torch.autograd.Function):
    """Routed experts over the exchange plus, when given, the shared expert on the local tokens. The shared expert is part of
    this function so that its products can be launched where this rank would otherwise idle: after its last obligation to
    the other ranks (the return leg) has been issued and before it waits for its own rows to come back."""

    @staticmethod
    def forward(ctx, xn, scores, indices, w_up, w_down, up_bias, down_bias, sh_up, sh_down, rt, c):
        from lyra_b200.ops import cuda_ops, elementwise as ew, gemm as G

        F_, K = indices.shape
        El, C, _, H = w_up.shape
        training = any(ctx.needs_input_grad)
        ub = up_bias.detach().float().reshape(El, 2 * H) if up_bias is not None else None      # local experts' biases (GPT-OSS)
        db = down_bias.detach().float().reshape(El, C) if down_bias is not None else None
        tiles = TILE_DISPATCH
        scaled = tiles and SCORE_IN_EPILOGUE
        ex = _Exchange(rt, indices, C, tiles=tiles)
        # training keeps every layer's receive buffer for its backward pass; without gradients one set serves all layers
        # (a layer's exchange completes, on every rank, before the next layer's dispatch can be signalled)
        bufs = ex.buf.for_layer(rt._layer if training else -1)
        waits = {}
        if tiles:
            x_recv = ex.dispatch_tiles(xn, K, bufs["recv"], bufs["meta"], FWD, bufs["score"] if scaled else None, scores if scaled else None)
            waits = ex.gemm_waits(FWD)
        else:
            x_recv = ex.dispatch(xn, K, bufs["recv"], bufs["meta"])
        wu, wd = cuda_ops.bf16_weight(w_up).view(El, C, 2 * H), cuda_ops.bf16_weight(w_down)
        cap = ex.buf.cap
        # The receive buffer is sized for the worst case; only the 128-row tiles that belong to an expert are computed,
        # and only those rows are read afterwards, so the outputs need no zero fill.
        pre = None
        if cuda_ops.SAVE_PREACT and training:
            # memory to spare (several ranks): keep the pre-activations so that backward skips the up-projection recompute,
            # the largest GEMM of the layer on the rank with the most rows
            pre = G.grouped_gemm(x_recv, wu, ex.tile_group, bias=ub, out=torch.empty(cap, 2 * H, dtype=BF16, device=xn.device), **waits)
            act = ew.swiglu_fwd(pre, c.swiglu_beta, c.swiglu_limit, rows_dev=ex.total)
        else:
            act = G.grouped_gemm(x_recv, wu, ex.tile_group, bias=ub, swiglu=True, swiglu_beta=c.swiglu_beta, swiglu_limit=c.swiglu_limit,
                                 out=torch.empty(cap, H, dtype=BF16, device=xn.device), **waits)
        sh_out = sh_pre = None
        if tiles:
            # down-projection: the epilogue scales each row by its routing score, stores it into its source rank's return buffer and
            # counts it there; then the shared expert fills the time until this rank's own rows are back
            ex.build_row_dest(bufs["meta"])
            row_scale = bufs["score"].view(0, cap, torch.float32) if scaled else None
            G.grouped_gemm(act, wd, ex.tile_group, bias=db, row_dest=ex.row_dest, peer_out=bufs["ret"].peer_ptrs, row_scale=row_scale,
                           peer_count=ex.buf.returned_peers(FWD))
            if sh_up is not None:
                sh_out, sh_pre = _shared_forward(xn, sh_up, sh_down, c.swiglu_beta, c.swiglu_limit, cuda_ops.SAVE_PREACT and training)
            ret = ex.wait_returned(bufs["ret"], FWD, C)
        elif FUSED_RETURN:   # down-projection whose epilogue stores each row straight into its source rank's return buffer
            ex.build_row_dest(bufs["meta"])
            G.grouped_gemm(act, wd, ex.tile_group, bias=db, row_dest=ex.row_dest, peer_out=bufs["ret"].peer_ptrs)
            ret = ex.returned(bufs["ret"])
        else:
            down = G.grouped_gemm(act, wd, ex.tile_group, bias=db, out=torch.empty(cap, C, dtype=BF16, device=xn.device))
            ret = ex.collect(down, bufs["meta"], bufs["ret"])
        if sh_up is not None and sh_out is None:
            sh_out, sh_pre = _shared_forward(xn, sh_up, sh_down, c.swiglu_beta, c.swiglu_limit, cuda_ops.SAVE_PREACT and training)
        ident = torch.arange(F_ * K, device=xn.device)
        out = ew.gather_sum_rows(ret, ident, F_, K) if scaled else ew.combine_rows(ret, ident, scores, F_, K)
        if sh_out is not None:
            out = out + sh_out
        ctx.save_for_backward(xn, scores, w_up, w_down, ident)
        ctx.ex, ctx.bufs, ctx.cfg, ctx.rt = ex, bufs, (c.swiglu_beta, c.swiglu_limit), rt
        ctx.biases = (up_bias, down_bias)
        ctx.shared = (sh_up, sh_down, sh_pre)
        ctx.pre, ctx.scaled = pre, scaled
        return out

    @staticmethod
    def backward(ctx, dout):
        from lyra_b200.ops import cuda_ops, elementwise as ew, gemm as G

        xn, scores, w_up, w_down, ident = ctx.saved_tensors
        ex, bufs, (beta, limit) = ctx.ex, ctx.bufs, ctx.cfg
        sh_up, sh_down, sh_pre = ctx.shared
        ctx.shared = None
        F_, K = scores.shape
        El, C, _, H = w_up.shape
        cap, dev = ex.buf.cap, dout.device
        tiles = ex.tiles
        dout = dout.contiguous()
        ret = bufs["ret"].view(0, F_ * K * C, BF16).view(F_ * K, C)
        d_ret, dscores = ew.combine_rows_bwd(ret, dout, ident, scores, F_ * K, dense=True)
        if ctx.scaled:
            # the buffer holds score x row, so <row, dout> = <score x row, dout> / score. A score that underflowed to zero in the
            # softmax (logit gap beyond ~100) has lost its row; its gradient is then taken as zero.
            dscores = torch.where(scores > 1e-30, dscores / scores.clamp_min(1e-30), torch.zeros_like(dscores))
        x_recv = bufs["recv"].view(0, cap * C, BF16).view(cap, C)
        wu, wd = cuda_ops.bf16_weight(w_up).view(El, C, 2 * H), cuda_ops.bf16_weight(w_down)
        up_bias, down_bias = ctx.biases
        ub = up_bias.detach().float().reshape(El, 2 * H) if up_bias is not None else None
        waits = {}
        if tiles:
            # One receive scratch serves every layer's backward. Its previous reader on any rank was that rank's previous backward
            # exchange, which raised the "free" flag behind its last read; by now (an attention backward later) the flags are
            # normally all up, so this wait costs nothing.
            par = 0
            ex.wait(FLAG_SCRATCH_FREE)
            d_down = ex.dispatch_tiles(d_ret, 1, ex.buf.scratch_recv[par], None, BWD)
            waits = ex.gemm_waits(BWD)
        else:
            par = ex.buf.calls & 1
            d_down = ex.dispatch(d_ret, 1, ex.buf.scratch_recv[par], None)
        # the recompute of the pre-activations reads only the forward's rows: it runs while the gradient rows are still arriving
        pre = ctx.pre if ctx.pre is not None else G.grouped_gemm(x_recv, wu, ex.tile_group, bias=ub, out=torch.empty(cap, 2 * H, dtype=BF16, device=dev))
        ctx.pre = None
        # first reader of the incoming rows: the product that waits per tile
        d_act = G.grouped_gemm(d_down, wd, ex.tile_group, w_kmajor=True, out=torch.empty(cap, H, dtype=BF16, device=dev), **waits)
        act = ew.swiglu_fwd(pre, beta, limit, rows_dev=ex.total)
        gd = cuda_ops.GRAD_DTYPE
        if w_down.requires_grad:
            if w_down.grad is None:
                w_down.grad = G.grouped_wgrad(act, d_down, ex.offsets, El).to(gd)
            else:
                G.grouped_wgrad(act, d_down, ex.offsets, El, out=w_down.grad, accumulate=True)
        del act
        d_pre = ew.swiglu_bwd(pre, d_act, beta, limit, rows_dev=ex.total)
        del pre, d_act
        if w_up.requires_grad:
            if w_up.grad is None:
                w_up.grad = G.grouped_wgrad(x_recv, d_pre, ex.offsets, El).view(w_up.shape).to(gd)
            else:
                G.grouped_wgrad(x_recv, d_pre, ex.offsets, El, out=w_up.grad.view(El, C, 2 * H), accumulate=True)
        if up_bias is not None or down_bias is not None:   # per-expert column sums over the rows of each local expert (no host sync);
            # they read the receive scratch, so they come before anything that tells the other ranks it is free
            gid = ex.tile_group.long().repeat_interleave(128)
            dead = (gid < 0)[:, None]                       # rows of unused tiles hold uninitialised memory: mask, do not multiply
            gid = gid.clamp(min=0)
            if up_bias is not None and up_bias.requires_grad:
                cuda_ops._add_grad(up_bias, torch.zeros(El, 2 * H, dtype=torch.float32, device=dev).index_add_(0, gid, d_pre.float().masked_fill(dead, 0.0)))
            if down_bias is not None and down_bias.requires_grad:
                cuda_ops._add_grad(down_bias, torch.zeros(El, C, dtype=torch.float32, device=dev).index_add_(0, gid, d_down.float().masked_fill(dead, 0.0)))
        dx_sh = None
        if tiles:
            G.grouped_gemm(d_pre, wu, ex.tile_group, w_kmajor=True, row_dest=ex.row_dest, peer_out=ex.buf.scratch_ret[par].peer_ptrs,
                           peer_count=ex.buf.returned_peers(BWD))
            ex.signal(FLAG_SCRATCH_FREE)                    # this rank has read the last of its receive scratch
            if sh_up is not None:
                dx_sh = _shared_backward(xn, dout, sh_up, sh_down, sh_pre, beta, limit)
            dx_a = ex.wait_returned(ex.buf.scratch_ret[par], BWD, C)
        elif FUSED_RETURN:
            G.grouped_gemm(d_pre, wu, ex.tile_group, w_kmajor=True, row_dest=ex.row_dest, peer_out=ex.buf.scratch_ret[par].peer_ptrs)
            dx_a = ex.returned(ex.buf.scratch_ret[par])
        else:
            dx_recv = G.grouped_gemm(d_pre, wu, ex.tile_group, w_kmajor=True, out=torch.empty(cap, C, dtype=BF16, device=dev))
            dx_a = ex.collect(dx_recv, bufs["meta"], ex.buf.scratch_ret[par])
        if sh_up is not None and dx_sh is None:
            dx_sh = _shared_backward(xn, dout, sh_up, sh_down, sh_pre, beta, limit)
        dxn = ew.gather_sum_rows(dx_a, ident, F_, K)
        if dx_sh is not None:
            dxn = dxn + dx_sh
        return dxn, dscores, None, None, None, None, None, None, None, None, None
