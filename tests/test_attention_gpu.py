"""tcgen05 flash attention against the fp32 PyTorch reference."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, Nq, Nkv, T, S, D, seed=0):
    torch.manual_seed(seed)
    q = torch.randn(B, T, Nq, D, device="cuda").bfloat16().transpose(1, 2)
    k = torch.randn(B, S, Nkv, D, device="cuda").bfloat16().transpose(1, 2)
    v = torch.randn(B, S, Nkv, D, device="cuda").bfloat16().transpose(1, 2)
    sinks = torch.randn(Nq, device="cuda")
    return q, k, v, sinks


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("window", [0, 128])
@pytest.mark.parametrize("T", [256, 1000])
def test_flash_fwd(D, window, T):
    from lyra_b200.ops import attention as A, native
    from lyra_b200.ops import reference as ref

    q, k, v, sinks = _inputs(2, 4, 2, T, T, D)
    scale = D ** -0.5
    out, lse = A.flash_fwd(q, k, v, sinks, scale, window)
    native.check_status()
    ro, rl = ref.attention(q.float(), k.float(), v.float(), sinks, scale, window)
    assert (out.float() - ro).abs().max().item() < 3e-2
    assert (lse - rl).abs().max().item() < 2e-2
    out2, _ = A.flash_fwd(q, k, v, sinks, scale, window)
    assert torch.equal(out, out2)


def test_flash_fwd_rescales_and_merges_the_two_key_streams():
    """Large score ranges over many key tiles: the running maxima of the even and the odd key tiles drift apart by far more
    than the lazy-rescale threshold, so both the accumulator rescale and the final merge of the two streams are exercised."""
    from lyra_b200.ops import attention as A, native
    from lyra_b200.ops import reference as ref

    q, k, v, sinks = _inputs(1, 4, 2, 1664, 1664, 128, seed=5)
    q = (q.float() * 6.0).bfloat16()
    k = k.clone()
    k[:, :, 1200:1210] *= 3.0                    # a late burst of strong keys, in an odd and an even tile
    out, lse = A.flash_fwd(q, k, v, sinks, 128 ** -0.5, 0)
    native.check_status()
    ro, rl = ref.attention(q.float(), k.float(), v.float(), sinks, 128 ** -0.5, 0)
    assert (out.float() - ro).abs().max().item() < 4e-2
    assert (lse - rl).abs().max().item() < 3e-2


def test_flash_fwd_offset_queries():
    """T != S: queries start at position q_start of a longer key sequence (chunked prefill)."""
    from lyra_b200.ops import attention as A
    from lyra_b200.ops import reference as ref

    q, k, v, sinks = _inputs(1, 4, 1, 128, 512, 128, seed=1)
    for window in (0, 128):
        out, lse = A.flash_fwd(q, k, v, sinks, 128 ** -0.5, window, q_start=384)
        ro, rl = ref.attention(q.float(), k.float(), v.float(), sinks, 128 ** -0.5, window, 384)
        assert (out.float() - ro).abs().max().item() < 3e-2
        assert (lse - rl).abs().max().item() < 2e-2


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("window", [0, 128])
@pytest.mark.parametrize("T", [256, 712])
def test_flash_bwd(D, window, T):
    from lyra_b200.ops import attention as A, native
    from lyra_b200.ops import reference as ref

    q, k, v, sinks = _inputs(2, 4, 2, T, T, D, seed=3)
    scale = D ** -0.5
    d_out = (torch.randn(2, T, 4, D, device="cuda") * 0.1).bfloat16().transpose(1, 2)
    qf, kf, vf, sf = (t.float().detach().requires_grad_(True) for t in (q, k, v, sinks))
    ro, _ = ref.attention(qf, kf, vf, sf, scale, window)
    ro.backward(d_out.float())
    out, lse = A.flash_fwd(q, k, v, sinks, scale, window)
    dq, dk, dv, dsinks = A.flash_bwd(q, k, v, out, d_out, lse, sinks, scale, window)
    native.check_status()

    def rel(a, b):
        return ((a.float() - b).norm() / b.norm().clamp_min(1e-9)).item()

    assert rel(dq, qf.grad) < 2e-2
    assert rel(dk, kf.grad) < 2e-2
    assert rel(dv, vf.grad) < 2e-2
    assert rel(dsinks, sf.grad) < 2e-2
    again = A.flash_bwd(q, k, v, out, d_out, lse, sinks, scale, window)
    assert torch.equal(dk, again[1]) and torch.equal(dq, again[0])  # deterministic
