"""Small Sogulix configurations for the tests: every size differs from one to the next, and none has
the sizes of a published model."""
from __future__ import annotations

import numpy as np


def delta(heads, dim, rank=8, ff=None):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, rot_dims=None, base=10000.0, ff=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "rot": {"base": base, "dims": rot_dims or rot_dim},
         "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, vocab=97, width=48, loop=None, mult=0.5, softcap=12.0, eps=1e-5):
    cfg = {"architecture": "Sogulix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
           "residual_mult": mult}
    if softcap:
        cfg["logit_softcap"] = softcap
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# A: both mixers, a loop over the last two layers run three times, windows that are no multiple of a page
SMALL_A = config([delta(2, 16, ff=40), latent(3, 16, 8, 24, 40, 32, window=21, ff=56), delta(3, 24, rank=4, ff=40)],
                 vocab=131, width=40, loop=(1, 3, 3), mult=0.4)
# B: the loop opens the model; a layer without a feed-forward; fewer rotated entries than the rotated part has;
# no window in one layer
SMALL_B = config([latent(2, 24, 16, 16, 24, 16, window=0, rot_dims=8, base=500.0), delta(1, 32, rank=16, ff=72),
                  latent(5, 8, 8, 8, 16, 24, window=37, ff=64)],
                 vocab=89, width=56, loop=(0, 2, 2), mult=1.0, softcap=None, eps=1e-6)
# C: no loop; one head, one layer of each kind
SMALL_C = config([latent(1, 32, 16, 32, 48, 40, window=64, ff=96), delta(4, 16, rank=8)], vocab=67, width=64, mult=0.7,
                 softcap=30.0)
SMALL = {"A": (SMALL_A, dict(seed=11, page_size=16)), "B": (SMALL_B, dict(seed=12, page_size=4)),
         "C": (SMALL_C, dict(seed=13, page_size=32))}

# Random N(0, std) weights give nearly uniform attention and a state that forgets nothing in particular:
# queries and keys are scaled up so that scores spread, sinks so that they matter.
SPREAD = {"mix.uq": 3.0, "mix.uk": 3.0, "mix.sink": 40.0, "mix.w0": 30.0, "mix.a.b": 30.0}


def sequences(rng, vocab, lengths):
    return {f"s{i}": [int(t) for t in rng.integers(0, vocab, size=n)] for i, n in enumerate(lengths)}


def plain_logits(folder, seqs):
    import plain_sogulix as ps
    cfg, w = ps.read_folder(folder)
    return {name: np.asarray(ps.forward(cfg, w, ids), dtype=np.float64) for name, ids in seqs.items()}
