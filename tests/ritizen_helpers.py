"""Small Ritizen configurations for the tests, and a step's context made by hand.  Every size differs from
one configuration to the next; none has the sizes of a published model."""
from __future__ import annotations

import numpy as np


def attention(heads, kv_heads, dim, vdim, scale=None, kv_from=None, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": float(scale if scale is not None else dim ** -0.5)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def parallel(left, chunk, right_heads, right_dim, right_vdim, decay, scales=(0.7, 1.3), ff=None):
    lm = dict(left["mixer"], mask={"size": chunk})
    return {"type": "parallel",
            "mixer": {"left": lm, "left_scale": scales[0], "right_scale": scales[1],
                      "right": {"heads": right_heads, "dim": right_dim, "vdim": right_vdim, "decay": list(decay)}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mamba2(heads, vdim, state, groups, conv, norm_groups, ff=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, vocab=97, width=48, max_positions=256, eps=1e-5):
    return {"architecture": "Ritizen", "vocab": vocab, "width": width, "max_positions": max_positions,
            "layers": layers, "norm": {"eps": eps}}


# A: every mixer; a layer that borrows keys and values; heads whose key and value sizes differ; a chunk that is no
# multiple of a page; a layer without a feed-forward
SMALL_A = config([attention(6, 3, 16, 24, ff=88), attention(6, 3, 16, 24, kv_from=0, scale=0.3),
                  mamba2(4, 8, 12, 1, 4, 1), parallel(attention(4, 1, 24, 16), 10, 3, 20, 12, (0.5, 0.9, 0.99), ff=64)],
                 vocab=101, width=72, max_positions=192)
# B: the side-by-side mixer opens the model; as many key/value heads as query heads; values wider than keys;
# two taps; groups of the state-space mixer and of its norm differ
SMALL_B = config([parallel(attention(2, 2, 32, 32, scale=0.2), 7, 1, 40, 24, (0.95,), scales=(1.0, 0.25)),
                  mamba2(4, 16, 8, 2, 2, 4, ff=40), attention(5, 5, 8, 40, ff=96)],
                 vocab=89, width=56, max_positions=200, eps=1e-6)
# C: a width that is no multiple of 8 (the products leave the tensor cores), one head everywhere, a convolution
# of one tap (no kept inputs), a chunk of one page
SMALL_C = config([mamba2(1, 20, 16, 1, 1, 1, ff=30), attention(1, 1, 48, 48), attention(1, 1, 48, 48, kv_from=1, ff=70),
                  parallel(attention(1, 1, 16, 16), 32, 1, 8, 8, (0.8,), ff=44)],
                 vocab=67, width=50, max_positions=160, eps=3e-6)
# D: heads of 64 and 128 entries (the sizes the tcgen05 attention is built for) with long portions
SMALL_D = config([attention(6, 3, 64, 64, ff=64), parallel(attention(2, 1, 128, 128), 96, 2, 32, 32, (0.9, 0.999))],
                 vocab=113, width=64, max_positions=464)
SMALL = {"A": (SMALL_A, dict(seed=11, page_size=16)), "B": (SMALL_B, dict(seed=12, page_size=4)),
         "C": (SMALL_C, dict(seed=13, page_size=32)), "D": (SMALL_D, dict(seed=14, page_size=16))}

# Random N(0, std) weights give nearly uniform attention: queries and keys are scaled up so that scores spread;
# the state-space mixer's step sizes and rates so that its state forgets at a visible pace.
SPREAD = {".q": 2.0, ".k": 2.0, "dt_bias": 20.0, "A_log": 20.0}


def sequences(rng, vocab, lengths):
    return {f"s{i}": [int(t) for t in rng.integers(0, vocab, size=n)] for i, n in enumerate(lengths)}


def plain_logits(folder, seqs):
    import plain_ritizen as pr
    cfg, w = pr.read_folder(folder)
    return {name: np.asarray(pr.forward(cfg, w, ids), dtype=np.float64) for name, ids in seqs.items()}


def make_ctx(q_lens, pos0, slots, page_size=4, num_pages=64, shuffle=None, dtype=None):
    """A step's context made by hand: request r brings q_lens[r] rows from position pos0[r]; its pages are
    taken from `shuffle` (a permutation of the pool), so that logical and physical order differ.  Returns
    the context and the block table."""
    import torch
    from llm_inference_lab_b200.parts.base import GroupView, StepContext
    dev = torch.device("cuda:0")
    B, T = len(q_lens), sum(q_lens)
    kv = [p + n for p, n in zip(pos0, q_lens)]
    width = max(-(-k // page_size) for k in kv)
    order = list(shuffle) if shuffle is not None else list(range(num_pages))
    table = -np.ones((B, width), dtype=np.int32)
    at = 0
    for r in range(B):
        for b in range(-(-kv[r] // page_size)):
            table[r, b] = order[at]
            at += 1
    row_req = np.concatenate([np.full(n, r, dtype=np.int32) for r, n in enumerate(q_lens)])
    row_pos = np.concatenate([np.arange(p, p + n, dtype=np.int32) for p, n in zip(pos0, q_lens)])
    row_slot = np.array([table[r, p // page_size] * page_size + p % page_size for r, p in zip(row_req, row_pos)],
                        dtype=np.int32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)  # noqa: E731
    group = GroupView(page_size, 0, t(row_slot), t(table))
    ctx = StepContext(dtype=dtype or torch.float32, device=dev, n_tokens=T, n_requests=B,
                      token_ids=t(np.zeros(T)), row_req=t(row_req), row_pos=t(row_pos),
                      q_start=t(np.concatenate([[0], np.cumsum(q_lens)])), kv_len=t(kv), pos0=t(pos0),
                      state_slot=t(slots), groups=[group], q_lens=list(q_lens), kv_lens=kv, state_slots=list(slots),
                      max_q_len=max(q_lens), max_kv_len=max(kv))
    return ctx, table


def random_config(rng):
    """A random Ritizen configuration and page size: one to five layers in any order of the three mixers, key and
    value sizes that are multiples of 8 or only of 2 and differ from one another, any number of heads and groups,
    chunks from one position to longer than the sequences, one to five taps, widths and feed-forwards that are
    multiples of 8 or only of 2, layers that borrow the keys and values of an earlier attention layer."""
    def size(lo, hi):
        return int(rng.choice([8, 8, 16, 2])) * int(rng.integers(lo, hi))

    def att():
        G = int(rng.choice([1, 1, 2, 3]))
        dim = min(size(1, 12), 160)
        return attention(G * int(rng.choice([1, 2, 4, 5])), G, dim, dim if rng.random() < 0.4 else min(size(1, 12), 160),
                         scale=float(rng.uniform(0.5, 2.0)) * dim ** -0.5)

    width = size(3, 16)
    layers, owners = [], []
    for i in range(int(rng.integers(1, 6))):
        ff = size(2, 20) if rng.random() < 0.7 else None
        kind = rng.choice(["attention", "attention", "parallel", "mamba2"])
        if kind == "attention":
            if owners and rng.random() < 0.4:
                src = int(rng.choice(owners))
                m = layers[src]["mixer"]
                layer = attention(m["heads"], m["kv_heads"], m["dim"], m["vdim"], scale=m["scale"] * 1.3, kv_from=src, ff=ff)
            else:
                layer = att()
                layer["mlp"] = None if ff is None else {"kind": "dense", "ff": ff}
                owners.append(i)
        elif kind == "parallel":
            heads = int(rng.choice([1, 2, 3, 6]))
            layer = parallel(att(), int(rng.choice([1, 3, 8, 16, 33, 64, 500])), heads, min(size(1, 10), 96), size(1, 8),
                             [float(d) for d in rng.uniform(0.3, 1.0, size=heads)],
                             scales=(float(rng.uniform(0.2, 1.5)), float(rng.uniform(0.2, 1.5))), ff=ff)
        else:
            groups = int(rng.choice([1, 1, 2, 3]))
            heads, vdim, parts = groups * int(rng.choice([1, 2, 4])), size(1, 8), int(rng.choice([1, 1, 2]))
            if (heads * vdim) % parts:
                parts = 1
            layer = mamba2(heads, vdim, min(size(1, 12), 128), groups, int(rng.integers(1, 6)), parts, ff=ff)
        layers.append(layer)
    cfg = config(layers, vocab=int(rng.integers(30, 400)), width=width, max_positions=int(rng.choice([160, 260])),
                 eps=float(rng.choice([1e-6, 1e-5])))
    return cfg, int(rng.choice([16, 16, 4, 8, 32, 64]))
