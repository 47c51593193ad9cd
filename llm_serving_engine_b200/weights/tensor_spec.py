"""What a part expects of the checkpoint: a tensor's shape and its kind."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class TensorSpec:
    """``kind`` decides how the tensor is held and how random weights draw it:
    ``matrix`` (held in the compute dtype; N(0, 0.02)), ``bias`` (float32 vector;
    N(0, 0.02)), ``norm`` (float32 vector; 1 + U(-0.1, 0.1)), ``mixing`` (a small
    float32 square matrix; identity + U(-0.1, 0.1)), ``positive`` (a float32
    vector of positive numbers; U(0.1, 1)), ``filter`` (a small float32 table of
    convolution weights, [channels, taps]; N(0, 0.3)), ``table`` (integers, held as int32)."""

    shape: tuple[int, ...]
    kind: str = "matrix"

    def __post_init__(self) -> None:
        if self.kind not in ("matrix", "bias", "norm", "mixing", "positive", "filter", "table"):
            raise ValueError(f"unknown tensor kind {self.kind!r}")
