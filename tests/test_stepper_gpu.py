"""``Stepper.train_step`` on one GPU: microbatches staged from pinned host memory on the copy stream must give exactly the
update that device-resident inputs give. With four or more microbatches the staged token blocks of an early microbatch are
released on the host while its backward kernels (embedding gradient, cross-entropy backward) are still queued; the blocks
must not be recycled for a later microbatch's copy before those kernels have run."""

from dataclasses import replace

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_staged_inputs_give_the_same_update_as_resident_inputs():
    from lyra_b200.config import ModelConfig
    from lyra_b200.model import ModelWeights
    from lyra_b200.nn.params import tree_dict
    from lyra_b200.ops import native
    from lyra_b200.training.state import init_train_state
    from lyra_b200.training.steps import Stepper
    from lyra_b200.training.train import TrainingConfig

    c = ModelConfig(name="stage-test", seq_len=1024, n_embd=512, n_layers=6, head_dim=128, n_attn_heads=4, n_kv_heads=2,
                    use_sdpa_output_gate=True, n_routed_experts=7, n_shared_experts=1, n_active_experts=3,
                    mlp_map=("dense", "moe") * 3, vocab_size=4000, padded_vocab_size=4096, tie_embeddings=False)
    A, B = 6, 4
    tcfg = TrainingConfig(steps=4, batch_size=B, accumulation_steps=A)
    rng = np.random.default_rng(0)
    xs = rng.integers(0, c.vocab_size, size=(A, B, c.seq_len)).astype(np.int32)     # every microbatch has its own tokens
    ys = np.roll(xs, -1, axis=-1)
    host = (torch.from_numpy(xs).pin_memory(), torch.from_numpy(ys).pin_memory())
    resident = (torch.from_numpy(xs).cuda(), torch.from_numpy(ys).cuda())
    after = {}
    for name, (x, y) in {"resident": resident, "staged": host}.items():
        w = ModelWeights.init(3, c, device="cuda")
        st = Stepper(init_train_state(w, c, tcfg), c, tcfg, device="cuda")
        for step in range(2):
            out = st.train_step(x, y, step)
        torch.cuda.synchronize()
        native.check_status()
        after[name] = (float(out["loss"]), {p: t.detach().clone() for p, t in tree_dict(w).items() if t.numel()})
    assert after["staged"][0] == after["resident"][0]
    for p, t in after["resident"][1].items():
        assert torch.equal(t, after["staged"][1][p]), p
