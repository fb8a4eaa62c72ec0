"""Sogulix on the CPU: configuration, run order, blueprint, random-weights mode and properties of the
plain implementation's mechanisms."""
import numpy as np
import pytest

import plain_sogulix as ps
from sogulix_helpers import SMALL, config, delta, latent


def _cfg(raw):
    from llm_inference_lab_b200.registry import resolve
    arch = resolve(raw)
    return arch, arch.config_class.from_dict(raw)


def test_registry_resolves_the_single_string_key():
    arch, cfg = _cfg(SMALL["A"][0])
    assert arch.name == "Sogulix" and cfg.width == 40 and cfg.to_dict()["architecture"] == "Sogulix"
    from llm_inference_lab_b200.config.base import ConfigError
    with pytest.raises(ConfigError):
        _cfg({"architecture": "NoSuchDesign"})


@pytest.mark.parametrize("loop,order,opens", [(None, [0, 1, 2], []), ((1, 3, 3), [0, 1, 2, 1, 2, 1, 2], [1, 3, 5]),
                                              ((0, 2, 2), [0, 1, 0, 1, 2], [0, 2]), ((0, 3, 1), [0, 1, 2], [0]),
                                              ((2, 3, 2), [0, 1, 2, 2], [2, 3])])
def test_run_order_and_caches(loop, order, opens):
    raw = config([delta(2, 16), latent(2, 8, 8, 8, 16, 16, window=5), delta(1, 8)], loop=loop)
    _, cfg = _cfg(raw)
    assert cfg.run_order() == (order, opens) == ps.run_order(raw)
    from llm_inference_lab_b200.config.sogulix import sogulix_blueprint
    from llm_inference_lab_b200.models.builder import cache_plan
    bp = sogulix_blueprint(cfg)
    assert [c.layer for c in bp.order] == order and [c.cache for c in bp.order] == list(range(len(order)))
    assert [r.before for r in bp.reentries] == opens
    plan = cache_plan(bp)
    kinds = [type(n).__name__ for n in plan.needs]
    assert kinds == ["FixedState" if i != 1 else "PagedLatent" for i in order]
    assert all(type(n).__name__ == "FixedState" and n.shape == (cfg.width,) for n in plan.block_needs)
    assert plan.group_windows == (5,)


def test_blueprint_names_every_tensor_and_reads_the_decay_rank_from_the_file():
    from llm_inference_lab_b200.config.sogulix import sogulix_blueprint
    from llm_inference_lab_b200.models.builder import expected_tensors
    raw = config([delta(2, 16, rank=None, ff=24), latent(3, 8, 4, 12, 20, 16, window=0, ff=None)], width=24, vocab=31)
    raw["layers"][0]["mixer"].pop("decay_rank")
    _, cfg = _cfg(raw)
    shapes = {t.name: t.shape for t in expected_tensors(sogulix_blueprint(cfg))}
    assert shapes["l0.mix.w1"] == (-1, 24) and shapes["l0.mix.w2"] == (32, -1)
    assert shapes["l1.mix.uq"] == (3 * 12, 16) and shapes["l1.mix.dkv"] == (24, 24) and shapes["l1.mix.sink"] == (3,)
    assert shapes["l1.mix.uk"] == (24, 20) and shapes["l1.mix.uv"] == (36, 20) and shapes["l1.mix.o"] == (24, 36)
    assert "l1.norm2" not in shapes and "l1.ls2" not in shapes and "l1.mlp.gate" not in shapes
    assert shapes["l0.mlp.down"] == (24, 24)
    assert {"embed", "embed.norm", "final.norm", "head", "l0.shift", "l0.ls1", "l0.ls2"} <= set(shapes)
    assert "loop.in" not in shapes      # no loop, no re-entry matrix


@pytest.mark.parametrize("bad", [
    lambda c: c["layers"][0].update(type="other"), lambda c: c["layers"][1]["mixer"].pop("kv_rank"),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), lambda c: c.update(loop={"start": 2, "stop": 1, "times": 1}),
    lambda c: c["norm"].pop("eps"), lambda c: c["layers"][0].update(mlp={"kind": "sparse", "ff": 8}),
    lambda c: c.pop("vocab")])
def test_config_errors_name_the_key(bad):
    import copy
    from llm_inference_lab_b200.config.base import ConfigError
    raw = copy.deepcopy(SMALL["A"][0])
    bad(raw)
    with pytest.raises(ConfigError):
        _cfg(raw)


def test_random_model_folder_round_trip(tmp_path):
    from helpers import make_model_folder
    raw, opt = SMALL["B"]
    folder = make_model_folder(str(tmp_path / "m"), raw, 3, "bfloat16", std=0.05, scales={})
    cfg, w = ps.read_folder(folder)
    assert cfg["architecture"] == "Sogulix" and w["l1.mix.w1"].shape == (16, 56)
    assert 0.0 <= w["l0.shift"].min() and w["l0.shift"].max() <= 1.0 and abs(w["l2.norm1"]).max() < 1.0
    logits = ps.forward(cfg, w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, raw["vocab"]) and np.isfinite(logits).all()
    # causal: a later token changes nothing before it
    again = ps.forward(cfg, w, [1, 2, 3, 9, 5])
    assert np.allclose(logits[:3], again[:3]) and not np.allclose(logits[3], again[3])


def test_plain_delta_rule_without_decay_and_removal_is_linear_attention():
    rng = np.random.default_rng(0)
    T, H, D, hid = 9, 2, 6, 10
    w = {"m." + n: rng.standard_normal((H * D, hid)) for n in ("r", "k", "v", "g")}
    w["m.a"] = np.zeros((H * D, hid))
    w["m.a.b"] = np.full(H * D, -80.0)         # removal rate 0
    w["m.w1"], w["m.w2"], w["m.w0"] = np.zeros((3, hid)), np.zeros((H * D, 3)), np.full(H * D, -80.0)   # decay 1
    w["m.norm"], w["m.o"] = np.ones(H * D), np.eye(H * D)
    h = rng.standard_normal((T, hid))
    got = ps.general_delta(h, w, "m.", {"heads": H, "dim": D}, 1e-9)
    r, k, v = ((h @ w["m." + n].T).reshape(T, H, D) for n in "rkv")
    o = np.zeros((T, H, D))
    for t in range(T):
        for n in range(H):
            o[t, n] = sum((k[s, n] @ r[t, n]) * v[s, n] for s in range(t + 1))
    want = ps.unit_rms(o, 1e-9).reshape(T, H * D) * ps.sigmoid(h @ w["m.g"].T)
    assert np.allclose(got, want, atol=1e-9)


def test_plain_latent_attention_window_and_sink():
    rng = np.random.default_rng(1)
    T, hid = 12, 8
    mixer = latent(2, 4, 4, 6, 5, 7, window=4)["mixer"]
    shapes = {"dq": (7, hid), "dq.norm": (7,), "uq": (16, 7), "dkv": (9, hid), "dkv.norm": (5,), "uk": (8, 5),
              "uv": (12, 5), "o": (hid, 12), "sink": (2,)}
    w = {"m." + n: rng.standard_normal(s) for n, s in shapes.items()}
    h = rng.standard_normal((T, hid))
    base = ps.latent_attention(h, w, "m.", mixer, 1e-6)
    moved = h.copy()
    moved[3] += 1.0                                  # token 3 is seen by rows 3..6 only
    out = ps.latent_attention(moved, w, "m.", mixer, 1e-6)
    changed = np.abs(out - base).max(axis=1) > 1e-12
    assert list(np.nonzero(changed)[0]) == [3, 4, 5, 6]
    w["m.sink"] = np.full(2, 60.0)                   # the sink takes all the weight: the output vanishes
    assert np.abs(ps.latent_attention(h, w, "m.", mixer, 1e-6)).max() < 1e-12 * np.abs(base).max() + 1e-15


def test_plain_token_shift_and_rotation():
    h = np.arange(12.0).reshape(4, 3)
    assert np.allclose(ps.token_shift(h, np.zeros(3)), h)
    assert np.allclose(ps.token_shift(h, np.ones(3))[1:], h[:-1]) and np.allclose(ps.token_shift(h, np.ones(3))[0], 0)
    v = np.random.default_rng(2).standard_normal((5, 2, 8))
    rot = ps.rotate_half_pairs(v, np.arange(5), 100.0, 4)
    assert np.allclose(rot[..., 4:], v[..., 4:]) and np.allclose(rot[0], v[0])          # the rest passes; angle 0
    assert np.allclose((rot[..., :4] ** 2).sum(-1), (v[..., :4] ** 2).sum(-1))         # a rotation
    # scores of rotated pairs depend on the distance only
    a, b = ps.rotate_half_pairs(v[:1].repeat(5, 0), np.arange(5), 100.0, 4), ps.rotate_half_pairs(
        v[1:2].repeat(5, 0), np.arange(5) + 3, 100.0, 4)
    dots = (a[:, 0, :4] * b[:, 0, :4]).sum(-1)
    assert np.allclose(dots, dots[0])
