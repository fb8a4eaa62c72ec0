"""A plain, slow NumPy implementation of the Sogulix design: whole sequences, no cache, one
function per mechanism, 64-bit floats.  It shares no code with the engine; the tests hold the
engine against it.

Notation: x[t] is the residual stream at token t, h a mixer's input, W_name the matrix stored
[out, in] and applied as W h.  Positions count from 0.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np


# ---------------------------------------------------------------------------------------------
# reading a model folder (safetensors: 8-byte length, JSON header, data)
# ---------------------------------------------------------------------------------------------
def read_folder(folder):
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    with open(os.path.join(folder, "model.safetensors"), "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n))
        data = fh.read()
    w = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = data[lo:hi]
        if info["dtype"] == "BF16":
            a = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            a = a.view(np.float32).astype(np.float64)
        elif info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif info["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(info["dtype"])
        w[name] = a.reshape(info["shape"])
    return cfg, w


# ---------------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_around_zero(x, weight, eps):
    """RMS norm whose stored weight lies around zero: the gain is 1 + weight."""
    return unit_rms(x, eps) * (1.0 + weight)


def norm_plain_weight(x, weight, eps):
    return unit_rms(x, eps) * weight


def token_shift(h, mix):
    """h[t] + (h[t-1] - h[t]) * mix, with zeros before the first token; h[t-1] is the unshifted one."""
    prev = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (prev - h) * mix


def rotate_half_pairs(v, positions, base, dims):
    """Rotary encoding on the first `dims` entries of the last axis; entry i pairs with i + dims/2.
    v is [tokens, ..., d]; positions [tokens]."""
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = positions[:, None].astype(np.float64) * freq[None, :]
    shape = (v.shape[0],) + (1,) * (v.ndim - 2) + (half,)
    cs, sn = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    out = v.copy()
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * cs - b * sn
    out[..., half:dims] = b * cs + a * sn
    return out


def gated_feed_forward(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ---------------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------------
DECAY_RATE = np.exp(-0.5)


def general_delta(h, w, p, mixer, eps):
    """Generalized delta rule, token by token, state S [heads, key channel, value channel]."""
    H, D = mixer["heads"], mixer["dim"]
    T = h.shape[0]
    r = (h @ w[p + "r"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, D)
    decay = np.exp(-DECAY_RATE * sigmoid(np.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).reshape(T, H, D)
    rate = sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).reshape(T, H, D)
    unit = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    S = np.zeros((H, D, D))
    o = np.zeros((T, H, D))
    for t in range(T):
        for n in range(H):
            old = S[n]
            u = unit[t, n]
            S[n] = decay[t, n][:, None] * old - np.outer(rate[t, n] * u, u @ old) + np.outer(k[t, n], v[t, n])
            o[t, n] = S[n].T @ r[t, n]
    o = unit_rms(o, eps).reshape(T, H * D) * w[p + "norm"]
    o = o * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def latent_attention(h, w, p, mixer, eps):
    """Attention whose keys and values are read from a low-rank latent, with a rotated key part
    shared by all heads, a sliding window and a learned sink in the softmax's denominator."""
    H, D, R, V, C = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    T = h.shape[0]
    pos = np.arange(T)
    cq = norm_plain_weight(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(T, H, D + R)
    q_flat, q_rot = q[..., :D], q[..., D:]
    dkv = h @ w[p + "dkv"].T
    c = norm_plain_weight(dkv[:, :C], w[p + "dkv.norm"], eps)
    k_rot = dkv[:, C:]
    base, dims = mixer["rot"]["base"], mixer["rot"]["dims"]
    q_rot = rotate_half_pairs(q_rot, pos, base, dims)
    k_rot = rotate_half_pairs(k_rot, pos, base, dims)
    k_flat = (c @ w[p + "uk"].T).reshape(T, H, D)
    val = (c @ w[p + "uv"].T).reshape(T, H, V)
    window = mixer["mask"]["size"] if mixer.get("mask") else T      # no mask entry: every earlier token is seen
    out = np.zeros((T, H, V))
    for n in range(H):
        s = (q_flat[:, n] @ k_flat[:, n].T + q_rot[:, n] @ k_rot.T) * mixer["scale"]
        i, j = pos[:, None], pos[None, :]
        seen = (i - j >= 0) & (i - j < window)
        s = np.where(seen, s, -np.inf)
        sink = w[p + "sink"][n]
        m = np.maximum(s.max(axis=1), sink)
        e = np.exp(s - m[:, None])
        den = e.sum(axis=1) + np.exp(sink - m)
        out[:, n] = (e / den[:, None]) @ val[:, n]
    return out.reshape(T, H * V) @ w[p + "o"].T


MIXERS = {"general_delta": general_delta, "latent_attention": latent_attention}


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def layer(x, w, i, spec, cfg):
    eps, m, p = cfg["norm"]["eps"], cfg["residual_mult"], f"l{i}."
    h = token_shift(norm_around_zero(x, w[p + "norm1"], eps), w[p + "shift"])
    total = MIXERS[spec["type"]](h, w, p + "mix.", spec["mixer"], eps) * w[p + "ls1"]
    if spec.get("mlp") is not None:
        if spec["mlp"]["kind"] != "dense":
            raise ValueError(spec["mlp"]["kind"])
        total = total + gated_feed_forward(norm_around_zero(x, w[p + "norm2"], eps), w, p + "mlp.") * w[p + "ls2"]
    return x + m * total


def run_order(cfg):
    """Layer indices in the order they run, with the indices of the runs that open a pass."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n)), []
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order, opens = list(range(start)), []
    for _ in range(times):
        opens.append(len(order))
        order += list(range(start, stop))
    order += list(range(stop, n))
    return order, opens


def forward(cfg, w, tokens, return_layers=False):
    """Logits [tokens, vocab] of one sequence (and the residual stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x = norm_around_zero(w["embed"][np.asarray(tokens)], w["embed.norm"], eps)
    x0 = x
    order, opens = run_order(cfg)
    after = []
    for run, i in enumerate(order):
        if run in opens:
            x = np.concatenate([x, x0], axis=1) @ w["loop.in"].T
        x = layer(x, w, i, cfg["layers"][i], cfg)
        after.append(x)
    logits = norm_around_zero(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(after)) if return_layers else logits


def greedy(cfg, w, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]
