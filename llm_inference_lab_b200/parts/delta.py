"""Recurrent mixer: the generalized delta rule."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import CacheView, Mixer, StepContext, register_part
from .spec import FixedState, PartSpec, TensorSpec


class GeneralDelta(Mixer):
    """Per head a state matrix S [key channel, value channel] in 32-bit, carried token by token:

        S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T,      o_t = S_t^T r_t

    r, k, v = W_r h, W_k h, W_v h (heads x dim each); decay w = exp(-rate * sigmoid(W_w2 tanh(W_w1 h) + w0))
    per head and key channel through a low-rank pair; removal rate a = sigmoid(W_a h + b_a); u the key
    divided by sqrt(sum k^2 + 1e-6).  Each head's o is divided by its root mean square, the heads side by
    side are multiplied by a plain weight and by sigmoid(W_g h), and W_o closes.  `decay_rate` is a
    parameter (exp(-1/2) where a design fixes it so).

    The six matrices that read h are concatenated at load time: one product.  Everything that enters the
    recurrence besides the products themselves is formed in 32-bit inside the recurrence kernel
    (`csrc/kernels/delta_rule.cu`), which serves prompts' portions and single decoded tokens alike."""
    decode_graph_safe = True


    NAMES = ("r", "k", "v", "g", "a")

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, hd, p = spec["hidden"], spec["heads"] * spec["dim"], spec.prefix
        rank = int(spec.get("decay_rank") or -1)      # -1: the checkpoint's tensors say
        out = [TensorSpec(p + n, (hd, h)) for n in cls.NAMES]
        out += [TensorSpec(p + "a.b", (hd,), init="bias"), TensorSpec(p + "w1", (rank, h)),
                TensorSpec(p + "w2", (hd, rank)), TensorSpec(p + "w0", (hd,), init="bias"),
                TensorSpec(p + "norm", (hd,), init="norm"), TensorSpec(p + "o", (h, hd))]
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return FixedState((spec["heads"], spec["dim"], spec["dim"]))

    @classmethod
    def libraries(cls, spec, dtype):
        return [("delta_rule", {"LAB_HEAD_DIM": int(spec["dim"])})]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.heads, self.dim = int(spec["heads"]), int(spec["dim"])
        if not ops.delta_rule_supported(self.dim):
            raise ValueError(f"general_delta: head size {self.dim} is outside what the recurrence kernel takes")
        self.hd = self.heads * self.dim
        w = lambda n: self._weight(weights, n)  # noqa: E731
        self.w_in = torch.cat([w(n) for n in self.NAMES] + [w("w1")], dim=0).contiguous()
        self.w_up = w("w2").contiguous()
        self.decay_bias, self.rate_bias, self.norm_weight = w("w0"), w("a.b"), w("norm")
        self.w_o = w("o").contiguous()
        self.eps = float(spec["eps"])
        self.decay_rate = float(spec.get("decay_rate", math.exp(-0.5)))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        proj = ops.linear(x, self.w_in, None, out_f32=True)
        middle = ops.tanh_cast(proj[:, 5 * self.hd:], self.dtype, self.dim)
        decay_pre = ops.linear(middle, self.w_up, None, out_f32=True)
        o = ops.delta_rule(proj, decay_pre, self.decay_bias, self.rate_bias, self.norm_weight, cache.state, ctx,
                           self.heads, self.dim, self.eps, self.decay_rate, write=cache.write)
        return ops.linear(o, self.w_o, None, out_f32=True, allow_partial=True)


register_part("mixer", "general_delta", GeneralDelta)
