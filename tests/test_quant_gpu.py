"""CUDA quantisation kernels against the PyTorch formulas evaluated on the CPU."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,block", [((3, 256, 384), (128, 128)), ((512, 256), (64, 64)), ((2, 4, 64, 128), (1, 128)), ((2, 2880, 5760), (64, 64))])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fp8_quantize_dequantize_match_cpu(shape, block, dtype):
    from lyra_b200.nn.quant import dequantize, quantize

    torch.manual_seed(0)
    x = (torch.randn(shape) * 3).to(dtype)
    x.view(-1)[::97] = 0
    ref = quantize(x, torch.float8_e4m3fn, block)                   # CPU tensors take the PyTorch path
    got = quantize(x.cuda(), torch.float8_e4m3fn, block)
    assert got.scale.shape == ref.scale.shape
    assert torch.allclose(got.scale.cpu(), ref.scale, rtol=1e-6, atol=0)
    assert torch.equal(got.qval.cpu().view(torch.uint8), ref.qval.view(torch.uint8))
    back = dequantize(got, torch.bfloat16)
    assert torch.equal(back.cpu(), dequantize(ref, torch.bfloat16))


def test_mxfp4_decode_matches_cpu():
    from lyra_b200.gpt_oss import dequantize_mxfp4, quantize_mxfp4

    torch.manual_seed(1)
    x = torch.randn(4, 96, 256) * torch.logspace(-3, 3, 96)[None, :, None]
    blocks, scales = quantize_mxfp4(x)
    ref = dequantize_mxfp4(blocks, scales)
    got = dequantize_mxfp4(blocks.cuda(), scales.cuda())
    assert got.shape == ref.shape and got.dtype == torch.bfloat16
    assert torch.equal(got.cpu(), ref)
