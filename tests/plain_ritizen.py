"""A plain, slow NumPy implementation of the Ritizen design: whole sequences, no cache, one
function per mechanism, 64-bit floats.  It shares no code with the engine; the tests hold the
engine against it.

Notation: x[t] is the residual stream at token t (positions count from 0), h a mixer's input,
W_name the matrix stored [out, in] and applied as W h.  A layer adds the *normed output* of each
sublayer to the stream, x <- x + norm(sublayer(x)); the sublayers read x itself.
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
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
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


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def softmax_over_visible(scores, visible):
    """Rows of `scores` [.., queries, keys] turned into weights over the keys marked in `visible`."""
    s = np.where(visible, scores, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(axis=-1, keepdims=True)


# ---------------------------------------------------------------------------------------------
# masks: which key j a query i sees
# ---------------------------------------------------------------------------------------------
def causal_mask(n):
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    return j <= i


def chunk_mask(n, size):
    """Causal inside chunks of `size` positions counted from position 0."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    return (j <= i) & (i // size == j // size)


# ---------------------------------------------------------------------------------------------
# softmax attention with grouped heads, norms over the whole projection, and an output gate
# ---------------------------------------------------------------------------------------------
def keys_and_values(h, w, p, m, eps, bias):
    """(k after its norm [T, G, dim], v [T, G, vdim]) of the layer whose tensors start with `p`."""
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    k = h @ w[p + "k"].T
    v = h @ w[p + "v"].T
    if bias:
        k, v = k + w[p + "k.b"], v + w[p + "v.b"]
    k = rms_norm(k, w[p + "k.norm"], eps)        # one root mean square over all heads' rows
    return k.reshape(-1, G, D), v.reshape(-1, G, V)


def softmax_attention(h, w, p, m, eps, visible, bias, gate, kv=None):
    """h [T, width] -> [T, width].  `gate`: "head" (one number per head) or "element".  `kv`: keys and
    values of another layer to use instead of this layer's own."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = h @ w[p + "q"].T
    if bias:
        q = q + w[p + "q.b"]
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(T, H, D)
    k, v = kv if kv is not None else keys_and_values(h, w, p, m, eps, bias)
    out = np.zeros((T, H, V))
    for head in range(H):
        g = head // (H // G)
        scores = (q[:, head] @ k[:, g].T) * m["scale"]
        out[:, head] = softmax_over_visible(scores, visible) @ v[:, g]
    z = sigmoid(h @ w[p + "g"].T)
    if gate == "head":
        out = out * z[:, :, None]
        out = out.reshape(T, H * V)
    else:
        out = out.reshape(T, H * V) * z
    return out @ w[p + "o"].T


# ---------------------------------------------------------------------------------------------
# linear attention with a fixed decay per head
# ---------------------------------------------------------------------------------------------
def decayed_linear_attention(h, w, p, m, eps):
    """S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t; heads normed together, gated, projected."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ w[p + "q"].T).reshape(T, H, D)
    k = silu(h @ w[p + "k"].T).reshape(T, H, D)
    v = silu(h @ w[p + "v"].T).reshape(T, H, V)
    out = np.zeros((T, H, V))
    for head in range(H):
        S = np.zeros((D, V))
        for t in range(T):
            S = m["decay"][head] * S + np.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    o = rms_norm(out.reshape(T, H * V), w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ---------------------------------------------------------------------------------------------
# two mixers side by side
# ---------------------------------------------------------------------------------------------
def parallel_mixer(h, w, p, m, eps):
    left = softmax_attention(h, w, p + "left.", m["left"], eps, chunk_mask(h.shape[0], m["left"]["mask"]["size"]),
                             bias=True, gate="element")
    right = decayed_linear_attention(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ---------------------------------------------------------------------------------------------
# state-space mixer (scalar decay per head and token)
# ---------------------------------------------------------------------------------------------
def causal_conv(u, taps, bias):
    """u [T, C], taps [C, K] (last column meets the current token), zeros before the start."""
    T, K = u.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, u.shape[1])), u], axis=0)
    out = np.zeros_like(u)
    for j in range(K):
        out += padded[j:j + T] * taps[:, j]
    return out + bias


def state_space_mixer(h, w, p, m, eps):
    Hn, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, T = Hn * V, h.shape[0]
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, Hn, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    rate = np.exp(w[p + "A_log"])
    y = np.zeros((T, Hn, V))
    for head in range(Hn):
        g = head // (Hn // G)
        S = np.zeros((N, V))
        for t in range(T):
            S = np.exp(-rate[head] * dt[t, head]) * S + dt[t, head] * np.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + w[p + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


# ---------------------------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------------------------
def dense_feed_forward(h, w, p):
    return gelu_tanh(h @ w[p + "up"].T + w[p + "up.b"]) @ w[p + "down"].T + w[p + "down.b"]


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def forward(cfg, w, ids, return_layers=False):
    """Logits [T, vocab] of one sequence (and, if asked, the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    ids = np.asarray(ids, dtype=np.int64)
    T = len(ids)
    x = w["embed"][ids] + w["pos"][:T]
    kept = {}              # layer -> its keys and values, for layers that borrow them
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = keys_and_values(x, w, p, m, eps, bias=False)
            a = softmax_attention(x, w, p, m, eps, causal_mask(T), bias=False, gate="head",
                                  kv=kept[i] if src is None else kept[src])
        elif layer["type"] == "parallel":
            a = parallel_mixer(x, w, p, m, eps)
        elif layer["type"] == "mamba2":
            a = state_space_mixer(x, w, p, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(a, w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(dense_feed_forward(x, w, f"l{i}.mlp."), w[f"l{i}.norm2"], eps)
        after.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, np.stack(after)) if return_layers else logits
