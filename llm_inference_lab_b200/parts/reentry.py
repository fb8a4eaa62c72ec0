"""Re-entries: what happens to the residual stream between two layer calls."""
from __future__ import annotations

from ..kernels import ops
from .base import StreamReentry, register_part
from .spec import PartSpec, TensorSpec


class ConcatProjection(StreamReentry):
    """x <- W [x ; x0]: the stream and the embedding output side by side through one matrix
    [hidden, 2 hidden] (the stream's columns first).  Opens a pass over looped layers.  Both inputs are
    32-bit streams; they are rounded to the storage type for the product, which leaves in 32-bit."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        return [TensorSpec(spec["name"], (spec["hidden"], 2 * spec["hidden"]))]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        w = weights[spec["name"]]
        self.weight = (w if w.dtype == dtype else w.to(dtype)).contiguous()

    def forward(self, x, x0):
        both = ops.stream_concat(x, x0, self.dtype)
        return ops.linear(both, self.weight, None, out_f32=True)


register_part("reentry", "concat_projection", ConcatProjection)
