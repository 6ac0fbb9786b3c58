"""Host-side caches of the inference path: fp32 copies of parameters stored in another dtype, and the fused q | k | v matrix.
Both must follow in-place updates of the parameters and must not survive the parameter they were made from."""

import gc

import torch


def test_fp32_param_is_cached_until_the_parameter_changes():
    from lyra_b200.ops import cuda_ops

    p = torch.nn.Parameter(torch.randn(6).bfloat16())
    full = torch.nn.Parameter(torch.randn(6))
    with torch.no_grad():
        assert cuda_ops.fp32_param(full) is full and cuda_ops.fp32_param(None) is None
        a = cuda_ops.fp32_param(p)
        assert a.dtype == torch.float32 and cuda_ops.fp32_param(p) is a
        p.mul_(2.0)
        b = cuda_ops.fp32_param(p)
        assert b is not a and torch.equal(b, p.float())
    # inside a gradient computation the conversion stays in the graph
    out = cuda_ops.fp32_param(p)
    assert out.requires_grad and out is not b


def test_fp32_param_does_not_serve_a_recycled_object():
    from lyra_b200.ops import cuda_ops

    with torch.no_grad():
        for seed in range(8):                      # freed tensors give their ids to later ones
            p = torch.full((4,), float(seed)).bfloat16()
            assert torch.equal(cuda_ops.fp32_param(p), p.float())
            del p
            gc.collect()


def test_fused_columns_follow_their_parts():
    from lyra_b200.ops import cuda_ops

    q, k, v = (torch.randn(8, n).bfloat16() for n in (16, 8, 8))
    bq, bv = torch.randn(16), torch.randn(8).bfloat16()
    with torch.no_grad():
        w, b = cuda_ops.fused_columns((q, k, v), (bq, None, bv))
        assert w.shape == (8, 32) and torch.equal(w, torch.cat([q, k, v], 1))
        assert torch.equal(b, torch.cat([bq, torch.zeros(8), bv.float()]))
        assert cuda_ops.fused_columns((q, k, v), (bq, None, bv))[0] is w           # cached
        k.add_(1.0)
        w2, _ = cuda_ops.fused_columns((q, k, v), (bq, None, bv))
        assert w2 is not w and torch.equal(w2, torch.cat([q, k, v], 1))
        w3, b3 = cuda_ops.fused_columns((q, k, v), (None, None, None))
        assert b3 is None and torch.equal(w3, w2)


def test_heartbeat_done_lets_slower_ranks_finish(tmp_path):
    """A rank that ran all its steps announces "done": the others' remaining checks pass instead of reporting a lost peer."""
    import torch.distributed as dist

    from lyra_b200.parallel.health import Heartbeat, PeerLost

    store = dist.FileStore(str(tmp_path / "store"), 2)
    fast, slow = Heartbeat(store, 0, 2), Heartbeat(store, 1, 2)
    fast.beat(0)
    slow.beat(0)
    fast.check(0, timeout=1.0)
    fast.done()
    for step in range(1, 4):                       # the slower rank still has steps to go
        slow.beat(step)
        slow.check(step, timeout=1.0)
    fast.leave()                                   # leaving early is still reported
    slow.beat(4)
    try:
        slow.check(4, timeout=1.0)
        raise AssertionError("a rank that left must be reported")
    except PeerLost as e:
        assert e.rank == 0


def test_caches_notice_updates_made_behind_the_version_counters():
    """The optimizer kernels rewrite parameters through raw pointers (no version bump): ``weights_changed`` retires what was
    derived from the old values."""
    from lyra_b200.ops import cuda_ops

    q, k, v = (torch.randn(4, n).bfloat16() for n in (8, 4, 4))
    b = torch.randn(8).bfloat16()
    with torch.no_grad():
        w0, _ = cuda_ops.fused_columns((q, k, v), (None, None, None))
        f0 = cuda_ops.fp32_param(b)
        q.data.view(torch.int16).add_(1)          # a write that PyTorch does not see as one, like a kernel's
        b.data.view(torch.int16).add_(1)
        cuda_ops.weights_changed()
        w1, _ = cuda_ops.fused_columns((q, k, v), (None, None, None))
        f1 = cuda_ops.fp32_param(b)
    assert w1 is not w0 and torch.equal(w1, torch.cat([q, k, v], 1))
    assert f1 is not f0 and torch.equal(f1, b.float())


def test_pending_pulls_keep_derived_copies_from_being_made(monkeypatch):
    from lyra_b200.ops import cuda_ops

    a, b = torch.ones(2), torch.ones(3)
    assert not cuda_ops.pull_pending(a, b, None)                       # no sharding runtime: nothing is ever pending
    monkeypatch.setattr(cuda_ops, "AG_HOOK", lambda w: {"src": 0} if w is b else None)
    assert not cuda_ops.pull_pending(a) and cuda_ops.pull_pending(a, b)
