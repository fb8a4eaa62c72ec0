"""Ritizen on the CPU: configuration, blueprint, caches made of parts, random-weights mode, and properties of
the plain implementation's mechanisms."""
import copy

import numpy as np
import pytest

import plain_ritizen as pr
from ritizen_helpers import SMALL, attention, config, mamba2, parallel


def _cfg(raw):
    from llm_inference_lab_b200.registry import resolve
    arch = resolve(raw)
    return arch, arch.config_class.from_dict(raw)


def test_registry_resolves_and_round_trips():
    arch, cfg = _cfg(SMALL["A"][0])
    assert arch.name == "Ritizen" and cfg.width == 72 and cfg.max_positions == 192
    again = arch.config_class.from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict() and cfg.to_dict()["architecture"] == "Ritizen"


def test_blueprint_layers_caches_and_tensors():
    from llm_inference_lab_b200.config.ritizen import ritizen_blueprint
    from llm_inference_lab_b200.models.builder import cache_plan, expected_tensors
    from llm_inference_lab_b200.parts.spec import CacheParts, FixedState, PagedKV
    _, cfg = _cfg(SMALL["A"][0])
    bp = ritizen_blueprint(cfg)
    assert bp.stream_f32 and bp.head.get("tied_to") == "embed" and bp.max_positions == 192
    # the layer that borrows keys and values reads the first layer's cache and owns none
    assert [(c.layer, c.cache, c.write) for c in bp.order] == [(0, 0, True), (1, 0, False), (2, 1, True), (3, 2, True)]
    plan = cache_plan(bp)
    assert plan.needs[0] == PagedKV(3, 32, 0)       # heads of 16 keys and 24 values are stored 32 wide
    assert plan.needs[1] == CacheParts((FixedState((4, 12, 8)), FixedState((3, 4 * 8 + 2 * 12))))
    assert plan.needs[2] == CacheParts((PagedKV(1, 32, 0), FixedState((3, 20, 12))))
    assert plan.group_windows == (0,) and plan.group_for(plan.needs[2].parts[0]) == 0
    shapes = {t.name: t.shape for t in expected_tensors(bp)}
    assert shapes["pos"] == (192, 72) and shapes["embed"] == (101, 72) and "head" not in shapes
    assert shapes["l0.mix.g"] == (6, 72) and shapes["l0.mix.q.norm"] == (96,) and shapes["l0.mix.k.norm"] == (48,)
    assert shapes["l0.mix.v"] == (72, 72) and shapes["l0.mix.o"] == (72, 144) and "l0.mix.q.b" not in shapes
    assert not any(n.startswith(("l1.mix.k", "l1.mix.v")) for n in shapes) and shapes["l1.mix.q"] == (96, 72)
    assert shapes["l2.mix.in"] == (2 * 32 + 2 * 12 + 4, 72) and shapes["l2.mix.conv"] == (56, 4)
    assert shapes["l2.mix.norm"] == (32,) and "l2.norm2" not in shapes and "l2.mlp.up" not in shapes
    assert shapes["l3.mix.left.g"] == (64, 72) and shapes["l3.mix.left.k.b"] == (24,) and shapes["l3.mix.left.v.b"] == (16,)
    assert shapes["l3.mix.right.k"] == (60, 72) and shapes["l3.mix.right.g"] == (36, 72)
    assert shapes["l3.mlp.up.b"] == (64,) and shapes["l3.mlp.down.b"] == (72,) and shapes["final.norm"] == (72,)


@pytest.mark.parametrize("bad", [
    lambda c: c["layers"][0].update(type="other"),
    lambda c: c["layers"][0]["mixer"].pop("vdim"),
    lambda c: c["layers"][0]["mixer"].update(heads=5),                      # no multiple of kv_heads
    lambda c: c["layers"][1]["mixer"].update(kv_from=1),                    # must be an earlier layer
    lambda c: c["layers"][1]["mixer"].update(kv_from=2),
    lambda c: c["layers"][1]["mixer"].update(dim=8),                        # differs from the layer it reads
    lambda c: c["layers"][2]["mixer"].update(norm_groups=5),
    lambda c: c["layers"][2]["mixer"].update(groups=3),
    lambda c: c["layers"][3]["mixer"]["left"].pop("mask"),
    lambda c: c["layers"][3]["mixer"]["right"].update(decay=[0.5]),         # one per head
    lambda c: c["layers"][3]["mixer"].pop("left_scale"),
    lambda c: c["layers"][3].update(mlp={"kind": "moe", "ff": 8}),
    lambda c: c.pop("max_positions"),
    lambda c: c["norm"].pop("eps"),
])
def test_configurations_that_are_refused(bad):
    from llm_inference_lab_b200.config.base import ConfigError
    raw = copy.deepcopy(SMALL["A"][0])
    bad(raw)
    with pytest.raises(ConfigError):
        _cfg(raw)


def test_random_weights_mode_writes_what_the_plain_model_reads(tmp_path):
    from helpers import make_model_folder
    raw = config([mamba2(2, 8, 4, 1, 2, 2, ff=16), parallel(attention(2, 1, 8, 8), 3, 1, 4, 4, (0.5,))], vocab=23, width=16,
                 max_positions=32)
    folder = make_model_folder(str(tmp_path / "m"), raw, 3, "bfloat16", std=0.1, scales={})
    cfg, w = pr.read_folder(folder)
    assert cfg["layers"][1]["mixer"]["left"]["mask"]["size"] == 3
    logits, layers = pr.forward(cfg, w, [1, 5, 22, 0, 7], return_layers=True)
    assert logits.shape == (5, 23) and layers.shape == (2, 5, 16) and np.isfinite(logits).all()


def test_plain_mechanisms_have_the_properties_the_design_names():
    rng = np.random.default_rng(0)
    # chunks are counted from position 0: position 10 opens a chunk of 10 and sees itself alone
    m = pr.chunk_mask(25, 10)
    assert m[9, :10].all() and not m[10, :10].any() and m[10, 10] and m[24, 20:25].all() and not m[24, :20].any()
    assert not pr.causal_mask(5)[2, 3] and pr.causal_mask(5)[3, :4].all()
    # the convolution's last tap meets the current token, and nothing comes from before the start
    u = rng.standard_normal((6, 2))
    taps = np.array([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])
    out = pr.causal_conv(u, taps, np.zeros(2))
    assert np.allclose(out[:, 0], u[:, 0]) and np.allclose(out[2:, 1], u[:-2, 1]) and np.allclose(out[:2, 1], 0)
    # the whole-projection norm divides by one root mean square over all heads, so a head's own size shows
    q = np.concatenate([np.full(8, 3.0), np.full(8, 1.0)])
    assert np.allclose(pr.rms_norm(q, np.ones(16), 0.0), q / np.sqrt(5.0))
    # a prefix's outputs do not change when tokens follow (every mixer is causal)
    raw, _ = SMALL["B"]
    from llm_inference_lab_b200.registry import resolve
    from llm_inference_lab_b200.models.builder import expected_tensors
    from llm_inference_lab_b200.weights.random_init import random_tensor
    arch = resolve(raw)
    specs = expected_tensors(arch.blueprint(arch.config_class.from_dict(raw)))
    w = {s.name: random_tensor(s, 1, 0.1, 0.1, {}).double().numpy() for s in specs}
    ids = [int(t) for t in rng.integers(0, raw["vocab"], size=30)]
    full = pr.forward(raw, w, ids)
    assert np.abs(pr.forward(raw, w, ids[:17]) - full[:17]).max() < 1e-9


def test_bench_configurations_are_valid():
    import bench
    for shape in sorted(bench.RITIZEN_SHAPES):
        raw = bench.ritizen_config(shape, 4)
        arch, cfg = _cfg(raw)
        assert [layer["type"] for layer in raw["layers"]] == ["attention", "attention", "mamba2", "parallel"]
        assert cfg.width == bench.SHAPES[shape]["hidden_size"] and raw["layers"][1]["mixer"]["kv_from"] == 0
        from llm_inference_lab_b200.models.builder import expected_tensors
        assert len(expected_tensors(arch.blueprint(cfg))) > 40
