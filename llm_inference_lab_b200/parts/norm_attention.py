"""Grouped-query attention with norms over the whole q and k projections and a gate on the heads' outputs."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import CacheView, Mixer, StepContext, register_part
from .spec import PagedKV, PartSpec, TensorSpec


class GatedNormAttention(Mixer):
    """q = W_q h, k = W_k h, v = W_v h (`bias`: each with a bias), `heads` query heads of `dim` entries,
    `kv_heads` key/value heads (query head h reads key/value head h // (heads / kv_heads)), values of `vdim`
    entries.  q and k are RMS-normed over their whole projections, all heads at once, with plain weights; no
    rotation.  score = q . k * `scale`; a query at position i sees the keys j <= i, with `chunk` > 0 only
    those of its own chunk (i // chunk == j // chunk, chunks counted from position 0 of the sequence);
    softmax; the heads' outputs are multiplied by sigmoid(W_g h), one number per head (`gate` "head") or per
    entry ("element"); W_o closes.  `own_kv` False: the layer has no key and value tensors and reads the cache
    another layer call fills (its cache is the other call's, not written here).

    The matrices that read h are concatenated at load time: one product, taken in 32-bit (the norms and the
    gate are 32-bit), from which one kernel norms q and k, rounds, and stores k and v in their page slots.
    Heads are cached `ops.padded_head(dim, vdim)` wide with zeros beyond their own size, so that any pair of
    sizes runs on the attention kernels; the gate kernel packs the `vdim` real entries of every head for W_o.
    `forward_inner` leaves the gated heads (times a constant) in a buffer of the caller, for mixers that share
    one output projection with others."""
    decode_graph_safe = True

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, H, G, D, V, p = spec["hidden"], spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"], spec.prefix
        gate = H if spec["gate"] == "head" else H * V
        out = [TensorSpec(p + "q", (H * D, h)), TensorSpec(p + "q.norm", (H * D,), init="norm"),
               TensorSpec(p + "g", (gate, h)), TensorSpec(p + "o", (h, H * V))]
        if spec.get("own_kv", True):
            out += [TensorSpec(p + "k", (G * D, h)), TensorSpec(p + "v", (G * V, h)),
                    TensorSpec(p + "k.norm", (G * D,), init="norm")]
        if spec.get("bias"):
            out.append(TensorSpec(p + "q.b", (H * D,), init="bias"))
            if spec.get("own_kv", True):
                out += [TensorSpec(p + "k.b", (G * D,), init="bias"), TensorSpec(p + "v.b", (G * V,), init="bias")]
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec):
        # a chunk's keys stay in their pages as all keys do: pages are given back when the request ends
        return PagedKV(spec["kv_heads"], ops.padded_head(spec["dim"], spec["vdim"]), 0)

    @classmethod
    def libraries(cls, spec, dtype):
        out = [("norm_attention", {})]
        head = ops.padded_head(spec["dim"], spec["vdim"])
        if dtype == torch.bfloat16 and ops.attention_tc_supported(head):
            out.append(("attention_tc", {"LAB_HEAD_DIM": head}))
            if head in (64, 128):
                out.append(("attention_tc05", {"LAB_HEAD_DIM": head}))
        else:
            out.append(("attention_plain", {}))
        return out

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.n_q, self.n_kv, self.dim, self.vdim = (int(spec[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
        if self.n_q % self.n_kv:
            raise ValueError("gated_norm_attention: heads must be a multiple of kv_heads")
        if spec["gate"] not in ("head", "element"):
            raise ValueError(f"gated_norm_attention: gate {spec['gate']!r} is not one of 'head', 'element'")
        self.per_head = spec["gate"] == "head"
        self.head = ops.padded_head(self.dim, self.vdim)
        if self.head > 256:
            raise ValueError(f"gated_norm_attention: heads of {max(self.dim, self.vdim)} entries exceed the kernels' 256")
        self.scale, self.eps, self.chunk = float(spec["scale"]), float(spec["eps"]), int(spec.get("chunk") or 0)
        self.own_kv = bool(spec.get("own_kv", True))
        w = lambda n: self._weight(weights, n)  # noqa: E731
        names = ("q", "k", "v") if self.own_kv else ("q",)
        self.w_in = torch.cat([w(n) for n in names] + [w("g")], dim=0).contiguous()
        self.bias = torch.cat([w(n + ".b") for n in names], dim=0).contiguous() if spec.get("bias") else None
        self.gate_at = sum(w(n).shape[0] for n in names)
        self.norm_q = w("q.norm")
        self.norm_k = w("k.norm") if self.own_kv else None
        self.w_o = w("o").contiguous()
        self.out_width = self.n_q * self.vdim

    def forward_inner(self, x: torch.Tensor, ctx: StepContext, cache: CacheView, out=None, mult: float = 1.0, proj=None):
        """The gated heads side by side [tokens, heads * vdim], times `mult`, in the storage type.  `proj`: the
        32-bit product of x with `w_in`, where the caller has formed it already (as columns of a wider one)."""
        group = ctx.groups[cache.group]
        if proj is None:
            proj = ops.linear(x, self.w_in, None, out_f32=True, allow_partial=True)
        write = cache.write and self.own_kv
        q = ops.qk_norm_store(proj, self.bias, self.norm_q, self.norm_k, group.row_slot if write else None,
                              cache.k if write else None, cache.v if write else None, self.n_q, self.n_kv, self.dim,
                              self.vdim, self.head, self.eps, has_kv=self.own_kv)
        attn = ops.attention(q, cache.k, cache.v, ctx, group, self.n_q, self.n_kv, self.head, 0, self.scale,
                             chunk=self.chunk)
        return ops.head_gate(attn, proj, self.gate_at, self.per_head, self.n_q, self.vdim, self.head, mult, out=out)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        return ops.linear(self.forward_inner(x, ctx, cache), self.w_o, None, out_f32=True, allow_partial=True)


register_part("mixer", "gated_norm_attention", GatedNormAttention)
