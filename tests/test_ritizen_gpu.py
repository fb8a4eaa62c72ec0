"""Ritizen on the GPU against the plain implementation (tests/plain_ritizen.py): each mechanism
alone, then whole models under every way of cutting a trace, then generation through the scheduler."""
import os

import numpy as np
import pytest

import plain_ritizen as pr
from helpers import (error_stats, make_model_folder, run_trace_inprocess, run_trace_program, tokens_needed,
                     trace_mixed, trace_portions, trace_tail_decode, trace_whole)
from ritizen_helpers import (SMALL, SPREAD, attention, config, make_ctx, mamba2, parallel, plain_logits,
                             random_config, sequences)

pytestmark = pytest.mark.gpu

F32_MAX = 2e-4      # largest error over the largest logit, 32-bit engine against the 64-bit plain model
BF16_MAX, BF16_RMS = 0.10, 0.04


def _torch():
    import torch
    return torch


def _t(a, dtype=None):
    torch = _torch()
    t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    return t if dtype is None else t.to(dtype)


def _np(t):
    return t.double().cpu().numpy()


# ---------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------
def test_stream_operators_against_numpy():
    """Learned positions, the sum x += norm(product) from whole and from split-K partial products with a bias,
    the rounded copy, the weighted sum of two products, and the activation."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(0)
    T, H, V, P = 13, 52, 30, 40
    for dtype in (torch.float32, torch.bfloat16):
        table, ptab = _t(rng.standard_normal((V, H)), dtype), _t(rng.standard_normal((P, H)), dtype)
        ids = torch.from_numpy(rng.integers(0, V, size=T).astype(np.int32)).cuda()
        pos = torch.from_numpy(rng.integers(0, P, size=T).astype(np.int32)).cuda()
        x = ops.embed_position(ids, pos, table, ptab)
        want = _np(table)[ids.cpu().numpy()] + _np(ptab)[pos.cpu().numpy()]
        assert x.dtype == torch.float32 and np.abs(_np(x) - want).max() < 1e-6
        w, bias = _t(1 + 0.2 * rng.standard_normal(H), dtype), _t(rng.standard_normal(H), dtype)
        whole, parts = _t(rng.standard_normal((T, H))), _t(rng.standard_normal((3, T, H)))
        for a, b in ((whole, None), (parts, None), (parts, bias), (whole, bias)):
            y = x.clone()
            copy = ops.stream_norm_add(y, a, w, 1e-5, bias=b, copy=True)
            prod = _np(a) if a.dim() == 2 else _np(a).sum(0)
            if b is not None:
                prod = prod + _np(b)
            ref = _np(x) + pr.rms_norm(prod, _np(w), 1e-5)
            assert np.abs(_np(y) - ref).max() < 1e-5
            assert copy.dtype == dtype and torch.equal(copy, y.to(dtype))
            assert ops.stream_norm_add(x.clone(), a, w, 1e-5, bias=b) is None
        assert torch.equal(ops.stream_round(x, dtype), x.to(dtype))
        s = ops.weighted_sum(parts, 0.6, whole, 1.1)
        assert np.abs(_np(s) - (0.6 * _np(parts).sum(0) + 1.1 * _np(whole))).max() < 1e-5
        z = _t(3 * rng.standard_normal((7, 33)), dtype)
        ref = pr.gelu_tanh(_np(z))
        assert np.abs(_np(ops.gelu_tanh_(z.clone())) - ref).max() < (1e-6 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("tokens,n_out,k", [(3, 200, 64), (70, 96, 328), (300, 520, 128), (4100, 512, 2112),
                                            (9, 50, 36), (200, 30, 100)])
def test_gelu_in_the_products_epilogue(tokens, n_out, k):
    """The activation as the epilogue of the up product (both orientations of the tensor-core kernel, the
    kernel on pairs of SMs, and the plain kernel for rows of no 16-byte multiple and in 32-bit) against the
    product followed by the activation kernel, and against NumPy."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(tokens)
    for dtype in (torch.bfloat16, torch.float32):
        x, w, b = _t(rng.standard_normal((tokens, k)), dtype), _t(rng.standard_normal((n_out, k)) / np.sqrt(k), dtype), \
            _t(rng.standard_normal(n_out), dtype)
        fused = ops.linear(x, w, b, act="gelu_tanh")
        ref = pr.gelu_tanh(_np(x) @ _np(w).T + _np(b))
        assert fused.dtype == dtype and np.abs(_np(fused) - ref).max() < (2e-2 if dtype == torch.bfloat16 else 3e-5)
        two = ops.gelu_tanh_(ops.linear(x, w, b, out_f32=True)).to(dtype)     # one rounding, as in the epilogue
        assert torch.equal(fused, two)
    with pytest.raises(ops.KernelError):
        ops.linear(x, w, b, act="relu")


@pytest.mark.parametrize("dims", [(3, 1, 16, 24), (2, 2, 40, 8), (6, 3, 64, 64)])
def test_whole_projection_norms_cache_store_and_gates(dims):
    """q and k normed over all heads at once (not head by head), heads stored with zero padding, k and v in the
    rows' page slots only, rows of padding skipped; both kinds of gate; partial products and a bias."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    H, G, D, V = dims
    head = ops.padded_head(D, V)
    rng = np.random.default_rng(sum(dims))
    T, page, pages = 9, 4, 12
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        width = H * D + G * (D + V) + H * V
        parts = _t(rng.standard_normal((2, T, width)))
        bias = _t(rng.standard_normal(H * D + G * (D + V)), dtype)
        wq, wk = _t(1 + 0.3 * rng.standard_normal(H * D), dtype), _t(1 + 0.3 * rng.standard_normal(G * D), dtype)
        slots = torch.tensor([5, 4, 47, -1, 0, 13, 22, 9, 30], dtype=torch.int32, device="cuda:0")
        ck = torch.full((pages, G, page, head), 7.0, dtype=dtype, device="cuda:0")
        cv = torch.full((pages, G, page, head), 7.0, dtype=dtype, device="cuda:0")
        q = ops.qk_norm_store(parts, bias, wq, wk, slots, ck, cv, H, G, D, V, head, 1e-5)
        proj = _np(parts).sum(0)
        qkv = proj[:, : H * D + G * (D + V)] + _np(bias)
        want_q = pr.rms_norm(qkv[:, : H * D], _np(wq), 1e-5).reshape(T, H, D)
        want_k = pr.rms_norm(qkv[:, H * D: H * D + G * D], _np(wk), 1e-5).reshape(T, G, D)
        want_v = qkv[:, H * D + G * D:].reshape(T, G, V)
        got_q = _np(q).reshape(T, H, head)
        assert np.abs(got_q[:, :, :D] - want_q).max() < tol and np.all(got_q[:, :, D:] == 0)
        written = set()
        for t, slot in enumerate(slots.cpu().numpy()):
            if slot < 0:
                continue
            pg, off = slot // page, slot % page
            written.add((pg, off))
            assert np.abs(_np(ck[pg, :, off, :D]) - want_k[t]).max() < tol and torch.all(ck[pg, :, off, D:] == 0)
            assert np.abs(_np(cv[pg, :, off, :V]) - want_v[t]).max() < tol and torch.all(cv[pg, :, off, V:] == 0)
        for pg in range(pages):
            for off in range(page):
                if (pg, off) not in written:
                    assert torch.all(ck[pg, :, off] == 7.0) and torch.all(cv[pg, :, off] == 7.0)
        # a layer that borrows keys and values has the q part only, and writes nothing
        q_only = ops.qk_norm_store(parts[:, :, : H * D + 3].contiguous(), None, wq, None, None, None, None, H, G, D, V,
                                   head, 1e-5, has_kv=False)
        assert np.abs(_np(q_only).reshape(T, H, head)[:, :, :D]
                      - pr.rms_norm(proj[:, : H * D], _np(wq), 1e-5).reshape(T, H, D)).max() < tol
        attn = _t(rng.standard_normal((T, H * head)), dtype)
        gate_at = H * D + G * (D + V)
        z = pr.sigmoid(proj[:, gate_at:])
        a = _np(attn).reshape(T, H, head)[:, :, :V]
        per_entry = ops.head_gate(attn, parts, gate_at, False, H, V, head, 0.6)
        assert np.abs(_np(per_entry) - 0.6 * (a * z.reshape(T, H, V)).reshape(T, H * V)).max() < tol
        wide = torch.zeros((T, H * V + 8), dtype=dtype, device="cuda:0")
        per_head = ops.head_gate(attn, parts, gate_at, True, H, V, head, out=wide[:, 8:])
        assert np.abs(_np(per_head) - (a * z[:, :H, None]).reshape(T, H * V)).max() < tol and torch.all(wide[:, :8] == 0)


def _plain_masked_attention(q, k, v, positions, visible_from, scale):
    """q [n, H, D] at `positions`; k [L, G, D], v [L, G, V]; a row at position p sees visible_from(p) <= j <= p."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((n, H, v.shape[2]))
    for i, p in enumerate(positions):
        lo = visible_from(p)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo: p + 1, g] @ q[i, h]) * scale
            e = np.exp(s - s.max())
            out[i, h] = (e / e.sum()) @ v[lo: p + 1, g]
    return out


def _fill_cache(rng, table, n_keys, G, head, page, pages, dtype, scale=1.0):
    torch = _torch()
    k = scale * rng.standard_normal((n_keys, G, head))
    v = scale * rng.standard_normal((n_keys, G, head))
    ck = torch.full((pages, G, page, head), float("nan"), dtype=dtype, device="cuda:0")
    cv = torch.full((pages, G, page, head), float("nan"), dtype=dtype, device="cuda:0")
    for j in range(n_keys):
        pg, off = table[0, j // page], j % page
        ck[pg, :, off] = _t(k[j], dtype)
        cv[pg, :, off] = _t(v[j], dtype)
    return ck, cv


@pytest.mark.parametrize("head,dtype", [(24, "float32"), (48, "bfloat16"), (64, "bfloat16"), (128, "bfloat16")])
@pytest.mark.parametrize("chunk", [0, 10, 64])
def test_attention_kernels_with_chunks_random(head, dtype, chunk):
    """Portions (one of more than 64 rows, which the tcgen05 kernel takes at heads of 64 and 128) and single
    tokens of requests in one launch, pages in shuffled order, chunks that end inside pages and tiles."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(head + chunk)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    H, G, page, pages = 4, 2, 8, 64
    q_lens, pos0 = [90, 1, 9, 1, 30], [37, 70, 0, 0, 3]
    ctx, table = make_ctx(q_lens, pos0, [0, 1, 2, 3, 4], page, pages, rng.permutation(pages), dtype=tdt)
    ck = torch.full((pages, G, page, head), float("nan"), dtype=tdt, device="cuda:0")
    cv = ck.clone()
    keys = {}
    for r, (n, p0) in enumerate(zip(q_lens, pos0)):
        k, v = rng.standard_normal((p0 + n, G, head)), rng.standard_normal((p0 + n, G, head))
        for j in range(p0 + n):
            ck[table[r, j // page], :, j % page] = _t(k[j], tdt)
            cv[table[r, j // page], :, j % page] = _t(v[j], tdt)
        keys[r] = (_np(ck)[table[r, np.arange(p0 + n) // page], :, np.arange(p0 + n) % page],
                   _np(cv)[table[r, np.arange(p0 + n) // page], :, np.arange(p0 + n) % page])
    q = _t(rng.standard_normal((sum(q_lens), H * head)), tdt)
    out = _np(ops.attention(q, ck, cv, ctx, ctx.groups[0], H, G, head, 0, 0.2, chunk=chunk)).reshape(-1, H, head)
    at = 0
    for r, (n, p0) in enumerate(zip(q_lens, pos0)):
        want = _plain_masked_attention(_np(q[at: at + n]).reshape(n, H, head), keys[r][0], keys[r][1],
                                       range(p0, p0 + n), (lambda p: p // chunk * chunk) if chunk else (lambda p: 0), 0.2)
        assert np.abs(out[at: at + n] - want).max() < (1e-5 if dtype == "float32" else 3e-2), (r, chunk)
        at += n


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("head,dtype", [(24, "float32"), (48, "bfloat16"), (64, "bfloat16")])
def test_chunk_edges_and_far_keys(head, dtype, decode):
    """One key made to stand out (it and the query point the same way, scaled up; its value is marked): a row
    finds it from the key's own position to the last position of the key's chunk and not from the next
    chunk's first position on; without chunks a key hundreds of places back is found.  In long portions
    and for single decoded tokens, the marked key at a page's border, a chunk's border and elsewhere."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(5)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    H, G, page, pages, n_keys = 2, 1, 8, 64, 420
    for chunk in (0, 10, 64):
        for key_at in (0, 7, 8, 9, 10, 63, 64, 100, 319):
            ctx_all, table = make_ctx([n_keys], [0], [0], page, pages, rng.permutation(pages), dtype=tdt)
            ck, cv = _fill_cache(rng, table, n_keys, G, head, page, pages, tdt, scale=0.05)
            pg, off = table[0, key_at // page], key_at % page
            ck[pg, :, off] = 0
            ck[pg, :, off, 3] = 6.0
            cv[pg, :, off] = 0
            cv[pg, :, off, 5] = 1.0
            last_in = n_keys - 1 if chunk == 0 else min(n_keys - 1, (key_at // chunk + 1) * chunk - 1)
            probes = sorted({p for p in (key_at, key_at + 1, last_in - 1, last_in, last_in + 1, last_in + 2, n_keys - 1)
                             if key_at <= p < n_keys})
            for p in probes:
                first = p if decode else max(0, p - 80)
                ctx, _ = make_ctx([p + 1 - first], [first], [0], page, pages, dtype=tdt)
                ctx.groups[0].block_table = ctx_all.groups[0].block_table
                q = torch.zeros((p + 1 - first, H * head), dtype=tdt, device="cuda:0")
                q.view(-1, H, head)[:, :, 3] = 6.0
                out = ops.attention(q, ck, cv, ctx, ctx.groups[0], H, G, head, 0, 1.0, chunk=chunk)
                out = _np(out).reshape(-1, H, head)
                for i, pos in enumerate(range(first, p + 1)):
                    if pos < key_at:
                        continue
                    seen = out[i, :, 5]
                    assert (np.all(seen > 0.9) if pos <= last_in else np.all(seen < 0.3)), (chunk, key_at, pos, seen)


def _plain_recurrence(q, k, v, a, s, S0):
    """S <- a_t S + (s_t k_t) v_t^T; o_t = S^T q_t.  q, k [T, N], v [T, V], a, s [T]."""
    S = S0.copy()
    out = np.zeros((q.shape[0], v.shape[1]))
    for t in range(q.shape[0]):
        S = a[t] * S + s[t] * np.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out, S


@pytest.mark.parametrize("H,G,N,V", [(3, 3, 20, 12), (4, 2, 40, 56), (1, 1, 5, 33), (2, 1, 130, 7)])
def test_decay_scan_against_plain(H, G, N, V):
    """The recurrence alone: requests of unequal lengths side by side in portions of changing size down to
    single tokens, state slots that hold stale numbers of other requests, a fixed decay per head (with the
    kernel's own SiLU of q, k, v) and a decay and key scale per token with q and k shared by groups."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(H * N + V)
    lengths = [45, 7, 23]
    slots = [4, 0, 2]
    for per_token in (False, True):
        data = {}
        for r, L in enumerate(lengths):
            data[r] = dict(q=rng.standard_normal((L, G * N)), k=rng.standard_normal((L, G * N)) * 0.5,
                           v=rng.standard_normal((L, H * V)), a=rng.uniform(0.3, 1.0, size=(L, H)),
                           s=rng.uniform(0.1, 2.0, size=(L, H)))
        a_head = rng.uniform(0.5, 1.0, size=H)
        want = {}
        for r, L in enumerate(lengths):
            d = data[r]
            outs = []
            for h in range(H):
                g = h // (H // G)
                qq, kk, vv = d["q"][:, g * N:(g + 1) * N], d["k"][:, g * N:(g + 1) * N], d["v"][:, h * V:(h + 1) * V]
                if per_token:
                    o, _ = _plain_recurrence(qq, kk, vv, d["a"][:, h], d["s"][:, h], np.zeros((N, V)))
                else:
                    o, _ = _plain_recurrence(pr.silu(qq), pr.silu(kk), pr.silu(vv), np.full(L, a_head[h]), np.ones(L),
                                             np.zeros((N, V)))
                outs.append(o)
            want[r] = np.concatenate(outs, axis=1)
        state = torch.full((5, H, N, V), 3.0, device="cuda:0")
        state[slots] = 0
        done = [0, 0, 0]
        cuts = ([16, 1, 3], [1, 2, 17], [2, 1, 1], [17, 3, 2], [9, 0, 0])
        for cut in cuts:
            live = [r for r in range(3) if cut[r] > 0 and done[r] < lengths[r]]
            q_lens = [min(cut[r], lengths[r] - done[r]) for r in live]
            ctx, _ = make_ctx(q_lens, [done[r] for r in live], [slots[r] for r in live])
            cat = lambda key: _t(np.concatenate([data[r][key][done[r]: done[r] + n] for r, n in zip(live, q_lens)]))  # noqa: E731
            qk = torch.cat([cat("q"), cat("k")], dim=1)
            if per_token:
                out = ops.decay_scan(qk[:, : G * N], qk[:, G * N:], cat("v"), state, ctx, H, G, N, V, a_tok=cat("a"),
                                     s_tok=cat("s"))
            else:
                out = ops.decay_scan(qk[:, : G * N], qk[:, G * N:], cat("v"), state, ctx, H, G, N, V, a_head=_t(a_head),
                                     silu=True)
            exp = np.concatenate([want[r][done[r]: done[r] + n] for r, n in zip(live, q_lens)])
            assert np.abs(_np(out) - exp).max() < 2e-4 * max(1.0, np.abs(exp).max()), (per_token, cut)
            for r, n in zip(live, q_lens):
                done[r] += n
        assert torch.all(state[1] == 3.0) and torch.all(state[3] == 3.0)
        # a call that may not write leaves the state as it is
        before = state.clone()
        ctx, _ = make_ctx([3], [0], [4])
        z = _t(rng.standard_normal((3, 2 * G * N)))
        ops.decay_scan(z[:, : G * N], z[:, G * N:], _t(rng.standard_normal((3, H * V))), state, ctx, H, G, N, V,
                       a_head=_t(a_head), write=False)
        assert torch.equal(before, state)


def _mixer(kind_spec, std, dtype, seed, scales=None):
    """A mixer built from random weights, with the weights as 64-bit arrays under the plain model's names."""
    torch = _torch()
    from llm_inference_lab_b200.parts import lookup
    from llm_inference_lab_b200.weights.random_init import random_tensor
    klass = lookup("mixer", kind_spec.kind)
    weights = {}
    for spec in klass.tensors(kind_spec):
        weights[spec.name] = random_tensor(spec, seed, std, 0.1, scales or {}).to(dtype).cuda()
    plain = {name: _np(t) for name, t in weights.items()}
    return klass(kind_spec, weights, dtype, torch.device("cuda:0")), plain


@pytest.mark.parametrize("taps,groups,parts", [(4, 1, 1), (2, 2, 4), (1, 1, 2), (3, 4, 1)])
def test_state_space_part_against_plain(taps, groups, parts):
    """The mixer alone in 32-bit: a sequence in one step, and in portions down to single tokens and shorter
    than the convolution's reach, two requests side by side on state slots that were used before."""
    torch = _torch()
    from llm_inference_lab_b200.parts import CacheView, PartSpec
    rng = np.random.default_rng(taps)
    m = {"heads": 4, "vdim": 8, "state": 12, "groups": groups, "conv": taps, "norm_groups": parts}
    spec = PartSpec("state_space", {"hidden": 40, "heads": 4, "vdim": 8, "state": 12, "groups": groups, "taps": taps,
                                    "norm_groups": parts, "eps": 1e-5}, prefix="m.")
    mixer, w = _mixer(spec, 0.2, torch.float32, 3, {"dt_bias": 5.0, "A_log": 5.0})
    seqs = [rng.standard_normal((37, 40)), rng.standard_normal((11, 40))]
    want = [pr.state_space_mixer(h, w, "m.", m, 1e-5) for h in seqs]
    channels = 4 * 8 + 2 * groups * 12
    view = CacheView(None, parts=[CacheView(None, state=torch.full((3, 4, 12, 8), 9.0, device="cuda:0")),
                                  CacheView(None, state=torch.full((3, max(taps - 1, 0), channels), 9.0, device="cuda:0"))])
    for cuts in ([[37, 11]], [[5, 1], [1, 2], [2, 1], [1, 1], [20, 6], [8, 0]]):
        for part in view.parts:
            part.state[[2, 0]] = 0
        done = [0, 0]
        for cut in cuts:
            live = [r for r in range(2) if cut[r] > 0]
            ctx, _ = make_ctx([cut[r] for r in live], [done[r] for r in live], [[2, 0][r] for r in live])
            x = _t(np.concatenate([seqs[r][done[r]: done[r] + cut[r]] for r in live]))
            out = _np(mixer.forward(x, ctx, view))
            if out.ndim == 3:
                out = out.sum(0)
            exp = np.concatenate([want[r][done[r]: done[r] + cut[r]] for r in live])
            assert np.abs(out - exp).max() < 1e-4 * max(1.0, np.abs(exp).max()), cut
            for r in live:
                done[r] += cut[r]
        assert all(torch.all(part.state[1] == 9.0) for part in view.parts)


@pytest.mark.parametrize("heads,dim,vdim", [(3, 20, 12), (1, 64, 24), (2, 8, 40)])
def test_decay_linear_attention_part_against_plain(heads, dim, vdim):
    torch = _torch()
    from llm_inference_lab_b200.parts import CacheView, PartSpec
    rng = np.random.default_rng(heads)
    decay = tuple(float(d) for d in rng.uniform(0.5, 1.0, size=heads))
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    spec = PartSpec("decay_linear_attention", {"hidden": 40, "heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
                                               "eps": 1e-5}, prefix="m.")
    mixer, w = _mixer(spec, 0.3, torch.float32, 4)
    h = rng.standard_normal((29, 40))
    want = pr.decayed_linear_attention(h, w, "m.", m, 1e-5)
    view = CacheView(None, state=torch.zeros((2, heads, dim, vdim), device="cuda:0"))
    at = 0
    for n in (6, 1, 1, 2, 19):
        ctx, _ = make_ctx([n], [at], [1])
        out = _np(mixer.forward(_t(h[at: at + n]), ctx, view))
        out = out.sum(0) if out.ndim == 3 else out
        assert np.abs(out - want[at: at + n]).max() < 1e-4 * max(1.0, np.abs(want).max())
        at += n


def test_side_by_side_takes_any_mixers():
    """Mixers that cannot share products (here another design's recurrent mixer beside the linear attention) run
    one after the other and are summed with their constants; each keeps its own part of the cache."""
    torch = _torch()
    from llm_inference_lab_b200.parts import CacheView, PartSpec
    rng = np.random.default_rng(2)
    lin = PartSpec("decay_linear_attention", {"hidden": 40, "heads": 2, "dim": 16, "vdim": 8, "decay": (0.9, 0.6),
                                              "eps": 1e-5}, prefix="a.")
    other = PartSpec("general_delta", {"hidden": 40, "heads": 2, "dim": 16, "eps": 1e-5, "decay_rate": 0.6,
                                       "decay_rank": 8}, prefix="b.")
    both = PartSpec("side_by_side", {"hidden": 40, "parts": ((lin, 0.5), (other, 2.0))}, prefix="")
    mixer, _ = _mixer(both, 0.2, torch.float32, 6)
    assert not mixer.shared and mixer.decode_graph_safe

    def views():
        return [CacheView(None, state=torch.zeros((1, 2, 16, 8), device="cuda:0")),
                CacheView(None, state=torch.zeros((1, 2, 16, 16), device="cuda:0"))]

    h = _t(rng.standard_normal((12, 40)))
    ctx, _ = make_ctx([12], [0], [0])
    apart = views()
    a, b = (m.forward(h, ctx, v) for (m, _), v in zip(mixer.mixers, apart))
    want = 0.5 * (_np(a).sum(0) if a.dim() == 3 else _np(a)) + 2.0 * (_np(b).sum(0) if b.dim() == 3 else _np(b))
    together = CacheView(None, parts=views())
    got = mixer.forward(h, ctx, together)
    assert got.dim() == 2 and np.abs(_np(got) - want).max() < 1e-5
    assert all(torch.equal(x.state, y.state) for x, y in zip(apart, together.parts))


# ---------------------------------------------------------------------------------------------
# whole models under every cut
# ---------------------------------------------------------------------------------------------
def _engine(folder, dtype, opt, steps, **kw):
    from llm_inference_lab_b200.engine import Engine
    page = opt["page_size"]
    unit = max(64, page)
    pool = tokens_needed(steps, unit)
    return Engine(folder, dtype, max_tokens=pool, page_size=page, max_requests=4, max_batch_tokens=max(pool, 64),
                  max_seq_len=pool, **kw)


def _check(got, want, dtype, label):
    """32-bit: every position within F32_MAX.  bfloat16: the rms error over all positions within BF16_RMS and
    all but one position in a hundred within BF16_MAX (a sublayer's output is divided by its root mean square,
    so where it is nearly zero its direction hangs on the last bits of bfloat16 products)."""
    worst, rms, where = error_stats(got, want)
    if dtype == "float32":
        assert worst < F32_MAX, (label, worst, where)
        return
    peak = max(float(np.abs(v).max()) for v in want.values())
    over = [key for key, row in got.items() if np.abs(row - want[key[0]][key[1]]).max() > BF16_MAX * peak]
    assert rms < BF16_RMS and len(over) <= max(1, len(got) // 100), (label, worst, rms, over[:5])


ONE_LAYER = {
    "attention": config([attention(4, 2, 16, 16, ff=None)], vocab=53, width=32),
    "attention+ff": config([attention(3, 1, 24, 8, ff=48)], vocab=53, width=40),
    "borrowed": config([attention(2, 2, 32, 16), attention(2, 2, 32, 16, kv_from=0)], vocab=53, width=32),
    "mamba2": config([mamba2(2, 16, 8, 2, 5, 1)], vocab=53, width=32),
    "mamba2+ff": config([mamba2(3, 8, 24, 1, 4, 3, ff=40)], vocab=53, width=24),
    "parallel": config([parallel(attention(2, 1, 16, 16), 12, 2, 24, 8, (0.7, 0.97))], vocab=53, width=32),
    "parallel+ff": config([parallel(attention(4, 4, 8, 24), 5, 1, 16, 16, (0.9,), scales=(0.2, 2.0), ff=56)],
                          vocab=53, width=48),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_layer_models(tmp_path, name, dtype):
    rng = np.random.default_rng(3)
    cfg = ONE_LAYER[name]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 21, dtype, std=0.08, scales=SPREAD)
    seqs = sequences(rng, cfg["vocab"], [45, 1, 30])
    want = plain_logits(folder, seqs)
    for label, steps in (("whole", trace_whole(seqs)), ("tail", trace_tail_decode(seqs, tail=25)),
                         ("portions", trace_portions(seqs))):
        eng = _engine(folder, dtype, dict(page_size=8), steps)
        _check(run_trace_inprocess(eng, steps), want, dtype, (name, label))
        assert eng.cache.live_requests == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SMALL))
def test_models_under_every_cut(tmp_path, name, dtype):
    """Whole prompts; the tail decoded token by token, long enough for every chunk to pass over decoded tokens;
    portions of 2 to 11 tokens; up to four live requests with portions beside single tokens, in a pool so
    small that pages and state slots are used again."""
    cfg, opt = SMALL[name]
    rng = np.random.default_rng(opt["seed"])
    folder = make_model_folder(str(tmp_path / "m"), cfg, opt["seed"], dtype, std=0.08, scales=SPREAD)
    seqs = sequences(rng, cfg["vocab"], [150, 3, 61, 90, 1, 77, 40])
    want = plain_logits(folder, seqs)
    traces = {"whole": trace_whole(seqs), "tail": trace_tail_decode(seqs, tail=70), "portions": trace_portions(seqs),
              "mixed": trace_mixed(seqs, np.random.default_rng(1), max_live=4)}
    for label, steps in traces.items():
        eng = _engine(folder, dtype, opt, steps)
        got = run_trace_inprocess(eng, steps)
        assert len(got) == sum(len(v) for v in seqs.values())
        _check(got, want, dtype, (name, label))
        assert eng.cache.live_requests == 0 and all(f == eng.num_pages for f in eng.free_pages())


def test_long_portions_and_long_decoding(tmp_path):
    """Heads of 64 and 128 with portions of more than a hundred tokens (the tcgen05 attention) beside single
    tokens, and a tail of 150 decoded tokens that crosses a chunk's edge."""
    cfg, opt = SMALL["D"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, opt["seed"], "bfloat16", std=0.08, scales=SPREAD)
    seqs = sequences(np.random.default_rng(9), cfg["vocab"], [400, 130, 260])
    want = plain_logits(folder, seqs)
    for label, steps in (("whole", trace_whole(seqs)), ("tail", trace_tail_decode(seqs, tail=150)),
                         ("mixed", trace_mixed(seqs, np.random.default_rng(2), max_live=3, max_portion=140))):
        eng = _engine(folder, "bfloat16", opt, steps)
        _check(run_trace_inprocess(eng, steps), want, "bfloat16", label)


@pytest.mark.parametrize("trial", range(int(os.environ.get("LAB_RANDOM_RITIZEN", "6"))))
def test_random_configurations_and_traces(tmp_path, trial):
    """Random configurations (layer orders, sizes that are no multiples of 8 or 16, key sizes that differ from
    value sizes, chunks of 1 to 500 positions, 1 to 5 taps, borrowed keys and values, page sizes 4 to 64) under
    mixed batches with pages and slots used again, in both storage types.  `LAB_RANDOM_RITIZEN=N` runs N."""
    rng = np.random.default_rng(1000 + trial)
    cfg, page = random_config(rng)
    seqs = sequences(rng, cfg["vocab"], [int(n) for n in rng.integers(1, 150, size=6)])
    steps = trace_mixed(seqs, np.random.default_rng(trial), max_live=4, max_portion=int(rng.choice([9, 40, 140])))
    want = None
    for dtype in ("float32", "bfloat16"):
        folder = make_model_folder(str(tmp_path / dtype), cfg, trial, dtype, std=0.08, scales=SPREAD)
        if want is None or dtype == "bfloat16":
            want = plain_logits(folder, seqs)
        eng = _engine(folder, dtype, dict(page_size=page), steps)
        got = run_trace_inprocess(eng, steps)
        worst, rms, where = error_stats(got, want)
        if dtype == "float32":
            assert worst < F32_MAX, (trial, cfg, worst, where)
        else:
            depth = len(cfg["layers"])
            assert rms < BF16_RMS * (1 + 0.25 * max(0, depth - 3)), (trial, cfg, worst, rms, where)
        assert eng.cache.live_requests == 0


def test_cuts_agree_in_32_bit(tmp_path):
    """In 32-bit no sum's order depends on how a prompt was cut or on what else is in the batch."""
    cfg, opt = SMALL["A"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 5, "float32", std=0.08, scales=SPREAD)
    seqs = sequences(np.random.default_rng(2), cfg["vocab"], [70, 33, 9])
    results = []
    for steps in (trace_whole(seqs), trace_portions(seqs), trace_mixed(seqs, np.random.default_rng(3), max_live=3)):
        results.append(run_trace_inprocess(_engine(folder, "float32", opt, steps), steps))
    for other in results[1:]:
        for key, row in results[0].items():
            assert np.abs(row - other[key]).max() <= 1e-5, key


def test_trace_program_and_a_failed_step(tmp_path):
    """bin/trace_run on a Ritizen folder; and a step that fails leaves every part's state and the pages as they
    were."""
    from llm_inference_lab_b200.engine import Entry
    cfg, opt = SMALL["B"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 8, "float32", std=0.08, scales=SPREAD)
    seqs = sequences(np.random.default_rng(4), cfg["vocab"], [50, 20, 35, 8, 41])
    want = plain_logits(folder, seqs)
    steps = trace_mixed(seqs, np.random.default_rng(6), max_live=4)
    out = str(tmp_path / "out")
    os.makedirs(out)
    got = run_trace_program(folder, "float32", steps, out, tokens_needed(steps, 64))
    _check(got, want, "float32", "program")
    ids = seqs["s0"]
    eng = _engine(folder, "float32", opt, trace_whole(seqs))
    assert len(eng.state_tensors) == 3      # the linear attention's state, the state-space mixer's two
    eng.step([Entry(0, ids[:20], [])])
    states = [t.clone() for t in eng.state_tensors]
    with pytest.raises(Exception):
        eng.step([Entry(0, ids[20:30], []), Entry(1, [cfg["vocab"] + 5], [0])])     # refused before it runs
    head = eng.model.head
    try:
        old = head.forward
        head.forward = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("injected"))   # fails after the layers ran
        with pytest.raises(RuntimeError):
            eng.step([Entry(0, ids[20:30], [9])])
    finally:
        head.forward = old
    assert all(bool((a == b).all()) for a, b in zip(states, eng.state_tensors))
    logits = eng.step([Entry(0, ids[20:], [len(ids) - 21])]).cpu().numpy()
    assert np.abs(logits[0] - want["s0"][-1]).max() < F32_MAX * max(1.0, np.abs(want["s0"]).max())


# ---------------------------------------------------------------------------------------------
# generation through the scheduler
# ---------------------------------------------------------------------------------------------
def _greedy(cfg, w, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(pr.forward(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_scheduler(tmp_path, name):
    """More requests than state slots, prompts cut under a small token budget: greedy tokens in 32-bit equal
    the plain model's."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.kernels import ops
    from llm_inference_lab_b200.sampling import SamplingConfig
    cfg, opt = SMALL[name]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 17, "float32", std=0.08, scales=SPREAD)
    pcfg, w = pr.read_folder(folder)
    rng = np.random.default_rng(7)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], size=n)] for n in (5, 40, 1, 23, 12, 31)]
    llm = LLM(folder, "float32", page_size=opt["page_size"], kv_tokens=512, max_requests=3, max_batch_tokens=24,
              max_seq_len=128, device="cuda:0")
    results = llm.generate(prompts, SamplingConfig(max_new_tokens=12, ignore_eos=True))
    ops.take_device_errors()
    for prompt, res in zip(prompts, results):
        assert res.finish_reason == "length"
        assert res.tokens == _greedy(pcfg, w, prompt, 12)
    assert llm.engine.cache.live_requests == 0


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16")])
def test_decode_steps_from_cuda_graphs(tmp_path, name, dtype):
    """Decode steps replayed from CUDA graphs although the model keeps fixed-size state (its parts keep it on
    the device): batches padded with requests of length zero, a batch that shrinks as requests finish, the
    state put back after the warm-up run of every capture.  32-bit: the plain model's tokens; bfloat16: the
    tokens of the same engine stepping eagerly."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.kernels import ops
    from llm_inference_lab_b200.sampling import SamplingConfig
    cfg, opt = SMALL[name]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 23, dtype, std=0.08, scales=SPREAD)
    rng = np.random.default_rng(5)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], size=n)] for n in (7, 30, 2, 19, 11)]
    sampling = [SamplingConfig(max_new_tokens=n, ignore_eos=True) for n in (20, 5, 14, 9, 17)]

    def run(graph):
        llm = LLM(folder, dtype, page_size=opt["page_size"], kv_tokens=1024, max_requests=8, max_batch_tokens=64,
                  max_seq_len=128, device="cuda:0", cuda_graph=graph)
        assert llm.cuda_graph == graph
        out = [r.tokens for r in llm.generate(prompts, sampling)]
        ops.take_device_errors()
        assert llm.engine.cache.live_requests == 0
        if graph:
            assert llm.graphs.replays >= 10 and llm.graphs.captures >= 3
        return out

    got = run(True)
    if dtype == "float32":
        pcfg, w = pr.read_folder(folder)
        assert got == [_greedy(pcfg, w, p, s.max_new_tokens) for p, s in zip(prompts, sampling)]
    else:
        assert got == run(False)


def test_command_line_generates(tmp_path):
    import json
    import subprocess
    import sys
    cfg, opt = SMALL["C"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 19, "float32", std=0.08, scales=SPREAD)
    pcfg, w = pr.read_folder(folder)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, "-m", "llm_inference_lab_b200.cli", "--model-dir", folder, "--dtype", "f32",
                           "--prompt-ids", "3,14,15,9,2,6", "--max-new-tokens", "6", "--kv-tokens", "256"],
                          cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["generated_ids"] == _greedy(pcfg, w, [3, 14, 15, 9, 2, 6], 6)
