"""GPT-OSS checkpoints: loader for the ``original/*.safetensors`` layout (lyra/gpt_oss.py:15-93) and a writer that
produces random-weight checkpoints in the same layout for benchmarks.

Layout facts: fused ``attn.qkv`` rows are split into q / k / v and transposed to ``[in, out]``; the vocabulary is padded
to ``padded_vocab_size`` rows; expert weights are MXFP4 (two e2m1 values per byte, low nibble first, one e8m0 scale per
32 values, ``value * 2**(scale - 127)``) stored ``[experts, out, in/32, 16]`` and decoded to bf16 ``[experts, in, out]``;
GLU columns are interleaved (gate, linear, gate, ...) and get de-interleaved into ``[..., 2, hidden]``.
"""

from __future__ import annotations

from dataclasses import replace
from pathlib import Path

import torch

from lyra_b200.config import ModelConfig

FP4_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def dequantize_mxfp4(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """``blocks [..., G, 16] uint8``, ``scales [..., G] uint8`` -> bf16 ``[..., G * 32]``."""
    blocks = blocks.to(torch.uint8)
    if blocks.is_cuda and blocks.shape[-1] == 16 and blocks.numel() > 0:
        from lyra_b200.ops import native

        if native.kernels_available():      # one pass on the GPU: 17 bytes in, 64 bytes out per block
            import ctypes

            blocks, scales = blocks.contiguous(), scales.to(torch.uint8).contiguous()
            out = torch.empty(*blocks.shape[:-2], blocks.shape[-2] * 32, dtype=torch.bfloat16, device=blocks.device)
            native.check(native.kernels().lyra_mxfp4_decode(native.ptr(blocks), native.ptr(scales), native.ptr(out),
                                                            ctypes.c_longlong(blocks.numel() // 16), native.stream_ptr()), "mxfp4_decode")
            native.count_launch()
            return out
    lut = torch.tensor(FP4_VALUES, dtype=torch.bfloat16, device=blocks.device)
    lo, hi = lut[(blocks & 0x0F).long()], lut[(blocks >> 4).long()]
    unpacked = torch.stack((lo, hi), dim=-1)  # [..., G, 16, 2]
    exp = (scales.to(torch.int32) - 127)[..., None, None]
    scaled = torch.ldexp(unpacked.float(), exp).to(torch.bfloat16)
    return scaled.reshape(*blocks.shape[:-2], -1)


def quantize_mxfp4(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`dequantize_mxfp4` (round to nearest e2m1 under a power-of-two block scale); ``x [..., K]``, K % 32 == 0."""
    xb = x.float().reshape(*x.shape[:-1], -1, 32)
    amax = xb.abs().amax(-1, keepdim=True).clamp_min(2.0 ** -126)
    exp = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    scaled = xb / torch.exp2(exp)
    lut = torch.tensor(FP4_VALUES[:8], dtype=torch.float32, device=x.device)
    mag = (scaled.abs()[..., None] - lut).abs().argmin(-1)
    code = (mag + 8 * (scaled < 0)).to(torch.uint8)
    packed = code[..., 0::2] | (code[..., 1::2] << 4)
    return packed.contiguous(), (exp.squeeze(-1) + 127).to(torch.uint8)


def _deinterleave_glu(x: torch.Tensor) -> torch.Tensor:
    return torch.cat([x[..., 0::2], x[..., 1::2]], dim=-1).reshape(*x.shape[:-1], 2, -1)


def _interleave_glu(x: torch.Tensor) -> torch.Tensor:
    """``[..., 2, H] -> [..., 2H]`` with gate / linear columns alternating."""
    return torch.stack((x[..., 0, :], x[..., 1, :]), dim=-1).reshape(*x.shape[:-2], -1)


def load_gpt_oss_model(source, config: ModelConfig, device="cpu", expert_slice: tuple[int, int] | None = None, shard_fn=None):
    """Reads a GPT-OSS checkpoint into a ``ModelWeights`` tree (then applies ``ModelWeights.quantize``).
    ``expert_slice = (lo, hi)`` keeps only experts ``lo:hi`` (an expert-parallel rank's share); ``shard_fn(path, spec)``
    (a runtime's ``shard_info``) keeps this rank's slice of every leaf (a tensor-parallel rank's heads and hidden units)."""
    from safetensors import safe_open

    from lyra_b200.model import ModelWeights

    path = Path(source).expanduser()
    if (path / "original").is_dir():
        path = path / "original"
    files: dict[str, Path] = {}
    for file in sorted(path.glob("*.safetensors")):
        with safe_open(file, framework="pt") as f:
            files |= dict.fromkeys(f.keys(), file)

    def get(name: str) -> torch.Tensor:
        with safe_open(files[name], framework="pt") as f:
            return f.get_tensor(name)

    def place(value, spec, dtype=None, path=None):
        assert tuple(value.shape) == tuple(spec.shape) or expert_slice is not None, (value.shape, spec.shape)
        if shard_fn is not None:
            value = shard_fn(path, spec).narrow(value)
        return value.to(dtype or spec.dtype).to(device).contiguous()

    def padded_vocab(name: str):
        value = get(name)
        return torch.nn.functional.pad(value, (0, 0, 0, config.padded_vocab_size - value.shape[0]))

    ex = (lambda t: t[expert_slice[0]:expert_slice[1]]) if expert_slice else (lambda t: t)
    spec = ModelWeights.spec(config)
    q_dim, kv_dim = config.n_attn_heads * config.head_dim, config.n_kv_heads * config.head_dim
    tok = replace(spec.tok, emb=place(padded_vocab("embedding.weight"), spec.tok.emb, path="tok/emb"),
                  unemb=place(padded_vocab("unembedding.weight"), spec.tok.unemb, path="tok/unemb"),
                  norm_scale=place(get("norm.scale"), spec.tok.norm_scale, path="tok/norm_scale"))
    layers = []
    for index, layer in enumerate(spec.layers):
        block, attn, mlp = f"block.{index}", layer.attn, layer.mlp  # GPT-OSS is MoE in every layer
        at, ml = f"layers/{index}/attn/", f"layers/{index}/mlp/"
        q, k, v = torch.split(get(f"{block}.attn.qkv.weight"), [q_dim, kv_dim, kv_dim])
        qb, kb, vb = torch.split(get(f"{block}.attn.qkv.bias"), [q_dim, kv_dim, kv_dim])
        attn = replace(
            attn, q=place(q.T, attn.q, path=at + "q"), k=place(k.T, attn.k, path=at + "k"), v=place(v.T, attn.v, path=at + "v"),
            q_bias=place(qb, attn.q_bias, path=at + "q_bias"), k_bias=place(kb, attn.k_bias, path=at + "k_bias"),
            v_bias=place(vb, attn.v_bias, path=at + "v_bias"), sinks=place(get(f"{block}.attn.sinks"), attn.sinks, path=at + "sinks"),
            out=place(get(f"{block}.attn.out.weight").T, attn.out, path=at + "out"),
            out_bias=place(get(f"{block}.attn.out.bias"), attn.out_bias, path=at + "out_bias"),
            norm_scale=place(get(f"{block}.attn.norm.scale"), attn.norm_scale, path=at + "norm_scale"),
        )
        up = dequantize_mxfp4(ex(get(f"{block}.mlp.mlp1_weight.blocks")).to(device), ex(get(f"{block}.mlp.mlp1_weight.scales")).to(device)).transpose(1, 2)
        down = dequantize_mxfp4(ex(get(f"{block}.mlp.mlp2_weight.blocks")).to(device), ex(get(f"{block}.mlp.mlp2_weight.scales")).to(device)).transpose(1, 2)
        mlp = replace(
            mlp, router=place(get(f"{block}.mlp.gate.weight").T, mlp.router, path=ml + "router"),
            router_bias=place(get(f"{block}.mlp.gate.bias"), mlp.router_bias, path=ml + "router_bias"),
            mlp_up=place(_deinterleave_glu(up), mlp.mlp_up, torch.bfloat16, path=ml + "mlp_up"),
            mlp_up_bias=place(_deinterleave_glu(ex(get(f"{block}.mlp.mlp1_bias"))), mlp.mlp_up_bias, path=ml + "mlp_up_bias"),
            mlp_down=place(down, mlp.mlp_down, torch.bfloat16, path=ml + "mlp_down"),
            mlp_down_bias=place(ex(get(f"{block}.mlp.mlp2_bias")), mlp.mlp_down_bias, path=ml + "mlp_down_bias"),
            norm_scale=place(get(f"{block}.mlp.norm.scale"), mlp.norm_scale, path=ml + "norm_scale"),
        )
        layers.append(replace(layer, attn=attn, mlp=mlp))
    return ModelWeights.quantize(ModelWeights(tok=tok, layers=layers), config)


def write_random_gpt_oss_checkpoint(path, config: ModelConfig, seed: int = 0, device="cpu", layers_per_file: int = 4) -> Path:
    """Writes random weights of ``config``'s architecture in the GPT-OSS ``original/`` layout (bf16 tensors, MXFP4 experts)."""
    from safetensors.torch import save_file

    out = Path(path).expanduser() / "original"
    out.mkdir(parents=True, exist_ok=True)
    c = config
    g = torch.Generator(device=device).manual_seed(seed)
    rnd = lambda *shape, std=0.02: (torch.randn(*shape, generator=g, device=device) * std).to(torch.bfloat16)
    q_dim, kv_dim = c.n_attn_heads * c.head_dim, c.n_kv_heads * c.head_dim
    H = c.expert_hidden
    tensors = {"embedding.weight": rnd(c.vocab_size, c.n_embd), "unembedding.weight": rnd(c.vocab_size, c.n_embd),
               "norm.scale": torch.ones(c.n_embd, dtype=torch.bfloat16)}
    file_index = 0

    def flush():
        nonlocal tensors, file_index
        if tensors:
            save_file({k: v.cpu().contiguous() for k, v in tensors.items()}, str(out / f"model-{file_index:05d}.safetensors"))
            tensors, file_index = {}, file_index + 1

    for i in range(c.n_layers):
        b = f"block.{i}"
        up_blocks, up_scales = quantize_mxfp4(rnd(c.n_experts, 2 * H, c.n_embd, std=c.n_embd ** -0.5).float())
        down_blocks, down_scales = quantize_mxfp4(rnd(c.n_experts, c.n_embd, H, std=H ** -0.5).float())
        tensors |= {
            f"{b}.attn.norm.scale": torch.ones(c.n_embd, dtype=torch.bfloat16),
            f"{b}.attn.qkv.weight": rnd(q_dim + 2 * kv_dim, c.n_embd, std=c.n_embd ** -0.5),
            f"{b}.attn.qkv.bias": rnd(q_dim + 2 * kv_dim),
            f"{b}.attn.sinks": rnd(c.n_attn_heads, std=1.0),
            f"{b}.attn.out.weight": rnd(c.n_embd, q_dim, std=q_dim ** -0.5),
            f"{b}.attn.out.bias": rnd(c.n_embd),
            f"{b}.mlp.norm.scale": torch.ones(c.n_embd, dtype=torch.bfloat16),
            f"{b}.mlp.gate.weight": rnd(c.n_experts, c.n_embd, std=c.n_embd ** -0.5),
            f"{b}.mlp.gate.bias": rnd(c.n_experts),
            f"{b}.mlp.mlp1_weight.blocks": up_blocks, f"{b}.mlp.mlp1_weight.scales": up_scales,
            f"{b}.mlp.mlp1_bias": rnd(c.n_experts, 2 * H),
            f"{b}.mlp.mlp2_weight.blocks": down_blocks, f"{b}.mlp.mlp2_weight.scales": down_scales,
            f"{b}.mlp.mlp2_bias": rnd(c.n_experts, c.n_embd),
        }
        if (i + 1) % layers_per_file == 0:
            flush()
    flush()
    return out
