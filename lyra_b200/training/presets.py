"""Training presets (lyra/training/presets.py:6-34): schedule = 16/7630 warm-up, 50 % stable, cosine to 0."""

from __future__ import annotations

from lyra_b200.training.train import CHECKPOINT_DIR, DATA_DIR, TrainingConfig


def _pretraining(variant: str, *, steps: int, accumulation_steps: int, batch_size: int = 4) -> TrainingConfig:
    return TrainingConfig(
        steps=steps, batch_size=batch_size, accumulation_steps=accumulation_steps, decay_type="cosine",
        warmup_fraction=16 / 7630, stable_fraction=0.5, eval_data_path=DATA_DIR / "val", eval_every=steps // 100,
        eval_batches=16, sample_every=steps // 100, numerics_every=32, checkpoint_keep=3,
        checkpoint_path=CHECKPOINT_DIR / variant,
    )


TRAINING_PRESETS = {
    "train-dev": TrainingConfig(steps=100, batch_size=2, accumulation_steps=1, numerics_every=10, checkpoint_path=CHECKPOINT_DIR / "dev"),
    "train-tiny": TrainingConfig(steps=20, batch_size=2, accumulation_steps=1, eval_every=None, checkpoint_every=20,
                                 checkpoint_path=CHECKPOINT_DIR / "tiny"),
    "train-small": _pretraining("lyra-small", steps=308000, accumulation_steps=4),
    "train-medium": _pretraining("lyra-medium", steps=490000, accumulation_steps=8, batch_size=8),
    "train-large": _pretraining("lyra-large", steps=353000, accumulation_steps=8, batch_size=16),
    "train-max": _pretraining("lyra-max", steps=353000, accumulation_steps=4, batch_size=32),
}
