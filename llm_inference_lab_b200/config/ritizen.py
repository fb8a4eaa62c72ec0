"""Ritizen: a decoder that adds the normed output of every sublayer to a 32-bit residual stream and
mixes three kinds of token mixers, layer by layer.

config.json keys: ``vocab``, ``width``, ``max_positions`` (rows of the learned position table), ``norm.eps``
and ``layers``, a list whose entries give ``type`` (the mixer), ``mixer`` (its sizes and constants) and
``mlp`` (``kind`` ``dense`` with ``ff``, or null for a layer without a feed-forward):

``attention``
    grouped-query softmax attention (``heads``, ``kv_heads``, ``dim`` per query/key head, ``vdim`` per value
    head, ``scale``), causal, without rotation, no biases, RMS norm of the whole q and of the whole k
    projection, one sigmoid gate per head on the heads' outputs.  ``kv_from``: j makes the layer read the
    keys and values that layer j caches instead of projecting its own.
``parallel``
    two mixers that read the same input, summed with ``left_scale`` and ``right_scale``: ``left`` a softmax
    attention as above but with biases on q, k, v, an element-wise sigmoid gate and a mask of chunks of
    ``mask.size`` positions; ``right`` a linear attention with one fixed ``decay`` per head (``heads``,
    ``dim``, ``vdim``).
``mamba2``
    a state-space mixer with a scalar decay per head and token (``heads``, ``vdim``, ``state``, ``groups``,
    ``conv`` taps, ``norm_groups``).

Each layer is x <- x + norm1(mixer(x)), then x <- x + norm2(ff(x)); the feed-forward is
W_down gelu_tanh(W_up h) with biases.  The embedding adds a learned position vector; the head is the
embedding table.  Tensor names: ``embed``, ``pos``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``,
``l<i>.mlp.up|down`` (+ ``.b``), ``final.norm``.
"""
from __future__ import annotations

import dataclasses
from typing import Any

from .base import ConfigError, ModelConfig, finite_positive, positive, required
from ..parts.spec import LayerCall, LayerSpec, ModelBlueprint, PartSpec

MIXER_TYPES = ("attention", "parallel", "mamba2")


def _need(obj: Any, key: str, where: str, kind=(int, float)):
    if not isinstance(obj, dict) or key not in obj:
        raise ConfigError(f"config.json of Ritizen lacks {where}.{key}")
    value = obj[key]
    if isinstance(value, bool) or not isinstance(value, kind):
        raise ConfigError(f"config key {where}.{key} has the wrong type: {value!r}")
    return value


def _positive_int(obj, key, where) -> int:
    value = _need(obj, key, where, (int,))
    if value <= 0:
        raise ConfigError(f"config key {where}.{key} must be positive, got {value!r}")
    return int(value)


def _check_attention(m, where, chunked: bool) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _positive_int(m, key, where)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}.heads must be a multiple of {where}.kv_heads")
    finite_positive(where + ".scale", _need(m, "scale", where))
    if chunked:
        _positive_int(_need(m, "mask", where, (dict,)), "size", where + ".mask")


@dataclasses.dataclass
class RitizenConfig(ModelConfig):
    architecture = "Ritizen"

    vocab: int = required(int, positive)
    width: int = required(int, positive)
    max_positions: int = required(int, positive, doc="rows of the learned position table")
    layers: Any = required("any")
    norm: Any = required("any")

    def validate(self) -> None:
        finite_positive("norm.eps", _need(self.norm, "eps", "norm"))
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("'layers' must be a non-empty list")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"{where}.type must be one of {MIXER_TYPES}, got "
                                  f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            m, kind = layer.get("mixer"), layer["type"]
            where += ".mixer"
            if not isinstance(m, dict):
                raise ConfigError(f"config.json of Ritizen lacks {where}")
            if kind == "attention":
                _check_attention(m, where, chunked=False)
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                        raise ConfigError(f"{where}.kv_from must name an earlier layer, got {src!r}")
                    other = self.layers[src]
                    if other["type"] != "attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}.kv_from must name an attention layer with keys and values of its own")
                    for key in ("kv_heads", "dim", "vdim"):
                        if other["mixer"][key] != m[key]:
                            raise ConfigError(f"{where}.{key} differs from layer {src}'s, whose keys and values it reads")
            elif kind == "parallel":
                _check_attention(_need(m, "left", where, (dict,)), where + ".left", chunked=True)
                right = _need(m, "right", where, (dict,))
                for key in ("heads", "dim", "vdim"):
                    _positive_int(right, key, where + ".right")
                decay = _need(right, "decay", where + ".right", (list,))
                if len(decay) != right["heads"] or not all(
                        isinstance(d, (int, float)) and not isinstance(d, bool) and 0 <= d <= 1 for d in decay):
                    raise ConfigError(f"{where}.right.decay must hold one number in [0, 1] per head")
                for key in ("left_scale", "right_scale"):
                    _need(m, key, where)
            else:
                for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                    _positive_int(m, key, where)
                if m["heads"] % m["groups"]:
                    raise ConfigError(f"{where}.heads must be a multiple of {where}.groups")
                if (m["heads"] * m["vdim"]) % m["norm_groups"]:
                    raise ConfigError(f"{where}.norm_groups must divide heads * vdim")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"layers[{i}].mlp.kind must be 'dense' (or mlp null)")
                _positive_int(mlp, "ff", f"layers[{i}].mlp")

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": self.architecture}
        out.update(dataclasses.asdict(self))
        return out


def _attention_spec(m, width, eps, prefix, *, bias: bool, gate: str, chunk: int = 0, own_kv: bool = True) -> PartSpec:
    return PartSpec("gated_norm_attention", {
        "hidden": width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
        "scale": float(m["scale"]), "eps": eps, "bias": bias, "gate": gate, "chunk": int(chunk), "own_kv": own_kv},
        prefix=prefix)


def ritizen_blueprint(cfg: RitizenConfig) -> ModelBlueprint:
    """The design's layers as data: every size and constant comes from `cfg`."""
    eps, width = float(cfg.norm["eps"]), cfg.width
    layers, calls, cache_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        cache, write = i, True
        if kind == "attention":
            src = m.get("kv_from")
            mixer = _attention_spec(m, width, eps, p + "mix.", bias=False, gate="head", own_kv=src is None)
            if src is not None:
                cache, write = cache_of[src], False
        elif kind == "parallel":
            left, right = m["left"], m["right"]
            mixer = PartSpec("side_by_side", {"hidden": width, "parts": (
                (_attention_spec(left, width, eps, p + "mix.left.", bias=True, gate="element",
                                 chunk=left["mask"]["size"]), float(m["left_scale"])),
                (PartSpec("decay_linear_attention", {
                    "hidden": width, "heads": right["heads"], "dim": right["dim"], "vdim": right["vdim"],
                    "decay": tuple(float(d) for d in right["decay"]), "eps": eps}, prefix=p + "mix.right."),
                 float(m["right_scale"])))}, prefix=p + "mix.")
        else:
            mixer = PartSpec("state_space", {
                "hidden": width, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"], "groups": m["groups"],
                "taps": m["conv"], "norm_groups": m["norm_groups"], "eps": eps}, prefix=p + "mix.")
        cache_of[i] = cache
        mlp = layer.get("mlp")
        ffn = None
        if mlp is not None:
            ffn = PartSpec("dense_mlp", {"hidden": width, "intermediate": mlp["ff"], "act": "gelu_tanh", "bias": True,
                                         "out_f32": True, "names": {"up": "up", "down": "down", "bias": ".b"}},
                           prefix=p + "mlp.")
        norms = tuple(PartSpec("rmsnorm_stream", {"hidden": width, "eps": eps, "offset": 0.0, "name": name}, prefix=p)
                      for name in (("norm1", "norm2") if mlp is not None else ("norm1",)))
        layers.append(LayerSpec("normed_sublayers_stream", mixer, ffn, norms, hidden=width))
        calls.append(LayerCall(layer=i, cache=cache, write=write))
    # cache ids are dense: layers that borrow another layer's keys and values own none
    ids = {c: n for n, c in enumerate(sorted({c.cache for c in calls}))}
    calls = tuple(LayerCall(c.layer, ids[c.cache], c.write) for c in calls)
    return ModelBlueprint(
        hidden=width, vocab=cfg.vocab,
        embedding=PartSpec("token_position_embedding", {"vocab": cfg.vocab, "hidden": width, "table": "embed",
                                                        "positions": "pos", "max_positions": cfg.max_positions}),
        layers=tuple(layers), order=calls,
        final_norm=PartSpec("rmsnorm_stream", {"hidden": width, "eps": eps, "offset": 0.0, "name": "norm"},
                            prefix="final."),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "hidden": width, "tied_to": "embed"}),
        max_positions=cfg.max_positions, eos_token_ids=(), stream_f32=True)
