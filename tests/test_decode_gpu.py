"""Split-KV decode attention kernel against an fp32 PyTorch evaluation of the same softmax (bf16 and fp8 caches)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(q, k, v, sinks, scale, window, pos):
    """q [B, Nq, 1, D]; k, v [B, Nkv, S, D] fp32; softmax over visible keys plus one sink logit per head."""
    B, Nq, _, D = q.shape
    Nkv = k.shape[1]
    G = Nq // Nkv
    lo = max(0, pos - window + 1) if window else 0
    kk = k[:, :, lo:pos + 1].repeat_interleave(G, dim=1)
    vv = v[:, :, lo:pos + 1].repeat_interleave(G, dim=1)
    s = torch.einsum("bhtd,bhsd->bhts", q.float(), kk) * scale
    s = torch.cat([s, sinks.float().view(1, Nq, 1, 1).expand(B, Nq, 1, 1)], dim=-1)
    p = torch.softmax(s, dim=-1)[..., :-1]
    return torch.einsum("bhts,bhsd->bhtd", p, vv)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("window", [0, 128])
@pytest.mark.parametrize("pos", [0, 37, 700, 4095])
@pytest.mark.parametrize("shape", [(2, 8, 2), (3, 16, 2), (1, 4, 4)])
def test_decode_attention_bf16(D, window, pos, shape):
    from lyra_b200.ops import decode, native

    B, Nq, Nkv = shape
    S = 4096
    torch.manual_seed(pos + D)
    q = torch.randn(B, Nq, 1, D, device="cuda").bfloat16()
    k = torch.randn(B, Nkv, S, D, device="cuda").bfloat16()
    v = torch.randn(B, Nkv, S, D, device="cuda").bfloat16()
    k[:, :, pos + 1:] = float("nan")     # positions after `pos` must never be read into the result
    v[:, :, pos + 1:] = float("nan")
    sinks = torch.randn(Nq, device="cuda")
    out = decode.decode_attention(q, k, v, sinks, D ** -0.5, window, pos)
    native.check_status()
    ref = _reference(q, k.float().nan_to_num(0.0), v.float().nan_to_num(0.0), sinks, D ** -0.5, window, pos)
    assert out.shape == (B, Nq, 1, D)
    assert torch.isfinite(out.float()).all()
    assert (out.float() - ref).abs().max().item() < 2e-2
    assert torch.equal(out, decode.decode_attention(q, k, v, sinks, D ** -0.5, window, pos))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("window", [0, 128])
def test_decode_attention_fp8_cache(D, window):
    from lyra_b200.nn.quant import dequantize, quantize
    from lyra_b200.ops import decode, native

    B, Nq, Nkv, S, pos = 2, 16, 2, 2048, 1500
    torch.manual_seed(3)
    q = torch.randn(B, Nq, 1, D, device="cuda").bfloat16()
    k = quantize(torch.randn(B, Nkv, S, D, device="cuda") * 3, torch.float8_e4m3fn, block=(1, D))
    v = quantize(torch.randn(B, Nkv, S, D, device="cuda") * 0.5, torch.float8_e4m3fn, block=(1, D))
    sinks = torch.randn(Nq, device="cuda")
    out = decode.decode_attention(q, k, v, sinks, D ** -0.5, window, pos)
    native.check_status()
    ref = _reference(q, dequantize(k, torch.bfloat16).float(), dequantize(v, torch.bfloat16).float(), sinks, D ** -0.5, window, pos)
    assert (out.float() - ref).abs().max().item() < 2e-2


def test_decode_attention_device_position():
    """The position may live on the device: the same launch arguments serve successive positions."""
    from lyra_b200.ops import decode, native

    B, Nq, Nkv, S, D = 2, 8, 2, 1024, 64
    torch.manual_seed(5)
    q = torch.randn(B, Nq, 1, D, device="cuda").bfloat16()
    k = torch.randn(B, Nkv, S, D, device="cuda").bfloat16()
    v = torch.randn(B, Nkv, S, D, device="cuda").bfloat16()
    sinks = torch.zeros(Nq, device="cuda")
    pos_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    for pos in (5, 300, 1023):
        pos_dev.fill_(pos)
        out = decode.decode_attention(q, k, v, sinks, D ** -0.5, 0, 0, pos_dev=pos_dev)
        native.check_status()
        ref = _reference(q, k.float(), v.float(), sinks, D ** -0.5, 0, pos)
        assert (out.float() - ref).abs().max().item() < 2e-2


def test_decode_matches_prefill_kernel():
    """One decode step equals the last row of the tcgen05 prefill kernel over the same keys."""
    from lyra_b200.ops import attention as A, decode

    B, Nq, Nkv, T, D = 2, 8, 2, 512, 128
    torch.manual_seed(7)
    q = torch.randn(B, T, Nq, D, device="cuda").bfloat16().transpose(1, 2)
    k = torch.randn(B, T, Nkv, D, device="cuda").bfloat16().transpose(1, 2)
    v = torch.randn(B, T, Nkv, D, device="cuda").bfloat16().transpose(1, 2)
    sinks = torch.randn(Nq, device="cuda")
    full, _ = A.flash_fwd(q, k, v, sinks, D ** -0.5, 0)
    one = decode.decode_attention(q[:, :, -1:].contiguous(), k.contiguous(), v.contiguous(), sinks, D ** -0.5, 0, T - 1)
    assert (one.float() - full[:, :, -1:].float()).abs().max().item() < 2e-2
