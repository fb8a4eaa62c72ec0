"""Sogulix: a decoder whose layers mix two kinds of token mixers on a 32-bit residual stream.

config.json keys: ``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``logit_softcap``, ``loop``
(``start``, ``stop``, ``times``: layers start..stop-1 run `times` times in a row with the same weights and
a cache of their own in every pass; each pass opens with a projection of the stream beside the embedding
output), and ``layers``, a list whose entries give ``type`` (the mixer: ``general_delta`` or
``latent_attention``), ``mixer`` (its sizes and constants) and ``mlp`` (``kind`` ``dense`` with ``ff``, or
null).  Every layer is a parallel block: two norms of the same input (weights stored around zero), a
token shift before the mixer, per-channel scales on both results.  Tensor names: ``embed``,
``embed.norm``, ``loop.in``, ``l<i>.norm1|norm2|ls1|ls2|shift``, ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``,
``final.norm``, ``head``.  The rank of the decay's low-rank pair is the shape of ``l<i>.mix.w1``
(``mixer.decay_rank`` names it where there is no checkpoint yet: random-weights mode).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Optional

from .base import ConfigError, ModelConfig, finite_positive, optional, positive, required
from ..parts.spec import LayerCall, LayerSpec, ModelBlueprint, PartSpec, Reentry

MIXER_TYPES = ("general_delta", "latent_attention")
# The decay of the delta rule is exp(-DECAY_RATE * sigmoid(.)): fixed by the design.
DECAY_RATE = math.exp(-0.5)


def _need(obj: Any, key: str, where: str, kind=(int, float)):
    if not isinstance(obj, dict) or key not in obj:
        raise ConfigError(f"config.json of Sogulix lacks {where}.{key}")
    value = obj[key]
    if isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config key {where}.{key} has the wrong type: {value!r}")
    return value


def _positive_int(obj, key, where) -> int:
    value = _need(obj, key, where, (int,))
    if value <= 0:
        raise ConfigError(f"config key {where}.{key} must be positive, got {value!r}")
    return int(value)


@dataclasses.dataclass
class SogulixConfig(ModelConfig):
    architecture = "Sogulix"

    vocab: int = required(int, positive)
    width: int = required(int, positive)
    layers: Any = required("any")
    norm: Any = required("any")
    residual_mult: float = optional(float, 1.0)
    logit_softcap: Optional[float] = optional(float, None)
    loop: Any = optional("any", None)
    max_positions: int = optional(int, 1 << 17, positive, doc="longest sequence the engine plans for")

    def validate(self) -> None:
        finite_positive("norm.eps", _need(self.norm, "eps", "norm"))
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("'logit_softcap' must be positive or absent")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("'layers' must be a non-empty list")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"{where}.type must be one of {MIXER_TYPES}, got "
                                  f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            for key in ("dim", "heads"):
                _positive_int(m, key, where + ".mixer")
            if layer["type"] == "latent_attention":
                for key in ("kv_rank", "q_rank", "rot_dim", "vdim"):
                    _positive_int(m, key, where + ".mixer")
                finite_positive(where + ".mixer.scale", _need(m, "scale", where + ".mixer"))
                rot = m.get("rot")
                finite_positive(where + ".mixer.rot.base", _need(rot, "base", where + ".mixer.rot"))
                dims = _positive_int(rot, "dims", where + ".mixer.rot")
                if dims % 2 or dims > m["rot_dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims must be even and at most rot_dim")
                if m.get("mask") is not None:
                    _positive_int(m["mask"], "size", where + ".mixer.mask")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp.kind must be 'dense' (or mlp null)")
                _positive_int(mlp, "ff", where + ".mlp")
        if self.loop is not None:
            n = len(self.layers)
            start, stop = _need(self.loop, "start", "loop", (int,)), _need(self.loop, "stop", "loop", (int,))
            times = _positive_int(self.loop, "times", "loop")
            if not 0 <= start < stop <= n:
                raise ConfigError(f"'loop' must satisfy 0 <= start < stop <= {n}, got {start}, {stop}")
            del times

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture}
        out.update({k: v for k, v in dataclasses.asdict(self).items() if v is not None})
        return out

    def run_order(self) -> tuple[list[int], list[int]]:
        """Layer indices in the order they run, and the runs that open a pass of the loop."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n)), []
        start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order, opens = list(range(start)), []
        for _ in range(times):
            opens.append(len(order))
            order += list(range(start, stop))
        order += list(range(stop, n))
        return order, opens


def sogulix_blueprint(cfg: SogulixConfig) -> ModelBlueprint:
    """The design's layers as data: every size and constant comes from `cfg`."""
    eps, width = float(cfg.norm["eps"]), cfg.width
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "general_delta":
            mixer = PartSpec("general_delta", {
                "hidden": width, "heads": m["heads"], "dim": m["dim"], "eps": eps, "decay_rate": DECAY_RATE,
                "decay_rank": m.get("decay_rank")}, prefix=p + "mix.")
        else:
            mask = m.get("mask")
            mixer = PartSpec("latent_attention", {
                "hidden": width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps,
                "window": int(mask["size"]) if mask else 0, "sink": True,
                "rot_base": m["rot"]["base"], "rot_dims": m["rot"]["dims"]}, prefix=p + "mix.")
        mlp = layer.get("mlp")
        ffn = None
        if mlp is not None:
            ffn = PartSpec("gated_mlp", {"hidden": width, "intermediate": mlp["ff"], "act": "silu", "out_f32": True,
                                         "names": {"gate": "gate", "up": "up", "down": "down"}}, prefix=p + "mlp.")
        norms = tuple(PartSpec("rmsnorm_stream", {"hidden": width, "eps": eps, "offset": 1.0, "name": name}, prefix=p)
                      for name in (("norm1", "norm2") if mlp is not None else ("norm1",)))
        block = PartSpec("parallel_stream", {
            "hidden": width, "mult": cfg.residual_mult, "shift_name": "shift",
            "scale_names": ("ls1", "ls2") if mlp is not None else ("ls1",)}, prefix=p)
        layers.append(LayerSpec("parallel_stream", mixer, ffn, norms, hidden=width, block_spec=block))
    order, opens = cfg.run_order()
    calls = tuple(LayerCall(layer=i, cache=run) for run, i in enumerate(order))     # every run its own cache
    reentry = PartSpec("concat_projection", {"hidden": width, "name": "loop.in"})
    return ModelBlueprint(
        hidden=width, vocab=cfg.vocab,
        embedding=PartSpec("normed_token_embedding", {"vocab": cfg.vocab, "hidden": width, "eps": eps, "offset": 1.0,
                                                      "table": "embed", "norm": "embed.norm"}),
        layers=tuple(layers), order=calls,
        final_norm=PartSpec("rmsnorm_stream", {"hidden": width, "eps": eps, "offset": 1.0, "name": "norm"},
                            prefix="final."),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": width, "tied_to": None, "name": "head",
                                      "softcap": cfg.logit_softcap}),
        max_positions=cfg.max_positions, eos_token_ids=(),
        reentries=tuple(Reentry(before=run, part=reentry) for run in opens), stream_f32=True)
