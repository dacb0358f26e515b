"""Plain restatement of the Vulosun family in numpy float64: one function per mechanism, whole sequences only, no cache, no step
function, nothing shared with the product path.  Tests compare the native library against it.

A Vulosun layer wraps each sublayer in two layer norms (weight and bias): x += ln_b(mixer(ln_a(x))), then the same around the
feed-forward.  Mixers: "attention" (softmax attention, grouped K/V heads, an RMS norm with a weight over the WHOLE query and key
projection, interleaved rotary pairs, one sigmoid gate per head); "attention_2" (differential attention: every head has two score
maps over the same values, combined as a1 - lambda a2, unit RMS per head, constant factor, gate per head; projections with biases,
rotary frequencies divided by a constant, tokens see only their own chunk of positions, and the keys and values may be an earlier
layer's); "parallel" (the weighted sum of softmax attention with a per-head q/k norm, split-half rotary pairs and a sink in the
denominator, and of a linear recurrence S <- decay S + k v^T over SiLU-activated q, k, v whose concatenated heads are RMS-normed,
gated and projected).  Feed-forward: SiLU-gated dense, or routed squared-ReLU experts (sigmoid scores, group-limited choice, scaled
unrenormalised weights) plus a shared expert."""
from __future__ import annotations

import numpy as np


def to_float(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def layer_norm(x, w, b, eps):
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if w is None else y * w


def logistic(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * logistic(z)


def frequencies(dims, base, divide=1.0):
    return np.array([float(base) ** (-2.0 * i / dims) / divide for i in range(dims // 2)])


def rotate(v, positions, freqs, interleaved):
    """v [T, ..., n]: pair i of the last axis -- entries (2i, 2i+1) when interleaved, (i, i + len(freqs)) otherwise -- turns by
    positions[t] * freqs[i]; entries beyond 2 len(freqs) stay."""
    out = np.array(v, np.float64)
    T, half = v.shape[0], len(freqs)
    pos = np.asarray(positions, np.float64).reshape((T,) + (1,) * (v.ndim - 2))
    for i in range(half):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        ang = pos * freqs[i]
        out[..., a] = v[..., a] * np.cos(ang) - v[..., b] * np.sin(ang)
        out[..., b] = v[..., b] * np.cos(ang) + v[..., a] * np.sin(ang)
    return out


def first_visible(i, chunk):
    """first key position a query at position i sees: the start of its chunk of `chunk` positions (0: everything before it)"""
    return (i // chunk) * chunk if chunk > 0 else 0


def softmax_rows(scores, lo_of, sink=None):
    """scores [T, T] -> weights with row i limited to keys lo_of(i) .. i; sink: one more exp() in the denominator without a value"""
    T = scores.shape[0]
    w = np.zeros_like(scores)
    for i in range(T):
        lo = lo_of(i)
        s = scores[i, lo:i + 1]
        m = s.max() if sink is None else max(s.max(), sink)
        e = np.exp(s - m)
        w[i, lo:i + 1] = e / (e.sum() + (0.0 if sink is None else np.exp(sink - m)))
    return w


def rot_freqs(m):
    rot = m.get("rot")
    if not rot or not rot.get("dims"):
        return np.zeros(0)
    return frequencies(int(rot["dims"]), rot["base"], float((rot.get("scaling") or {}).get("factor", 1.0)))


def gated_attention(h, T, m, eps, book=None):
    """mixer "attention": q/k norm over the whole projection, interleaved rotation, causal softmax, one gate per head"""
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos, fr = np.arange(n), rot_freqs(m)
    q = rms_norm(h @ T["q"].T, T["q.norm"], eps).reshape(n, H, D)
    k = rms_norm(h @ T["k"].T, T["k.norm"], eps).reshape(n, G, D)
    v = (h @ T["v"].T).reshape(n, G, V)
    q, k = rotate(q, pos, fr, True), rotate(k, pos, fr, True)
    gate = logistic(h @ T["g"].T)
    out = np.zeros((n, H, V))
    for a in range(H):
        g = a // (H // G)
        w = softmax_rows(q[:, a] @ k[:, g].T * m["scale"], lambda i: 0)
        out[:, a] = (w @ v[:, g]) * gate[:, a:a + 1]
        if book is not None:
            book.setdefault("weights", {})[a] = w
    return out.reshape(n, H * V) @ T["o"].T


def differential_keys_values(h, T, m):
    """rotated keys [n, G, 2, D] and values [n, G, V] of an "attention_2" layer with projections of its own"""
    n = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ T["k"].T + T["k.b"]).reshape(n, G, 2, D)
    v = (h @ T["v"].T + T["v.b"]).reshape(n, G, V)
    return rotate(k, np.arange(n), rot_freqs(m), True), v


def differential_lambda(T, diff):
    return np.exp(np.sum(T["lq1"] * T["lk1"])) - np.exp(np.sum(T["lq2"] * T["lk2"])) + diff


def differential_attention(h, T, m, eps, kv, book=None):
    """mixer "attention_2" over given keys and values (its own or an earlier layer's)"""
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    chunk = int((m.get("mask") or {}).get("size") or 0)
    k, v = kv
    q = rotate((h @ T["q"].T + T["q.b"]).reshape(n, H, 2, D), np.arange(n), rot_freqs(m), True)
    lam = differential_lambda(T, m["diff"])
    gate = logistic(h @ T["g"].T)
    out = np.zeros((n, H, V))
    for a in range(H):
        g = a // (H // G)
        maps = []
        for j in range(2):
            w = softmax_rows(q[:, a, j] @ k[:, g, j].T * m["scale"], lambda i: first_visible(i, chunk))
            maps.append(w @ v[:, g])
            if book is not None:
                book.setdefault("weights", {})[(a, j)] = w
        o = rms_norm(maps[0] - lam * maps[1], None, eps) * (1.0 - m["diff"])
        out[:, a] = o * gate[:, a:a + 1]
    return out.reshape(n, H * V) @ T["o"].T


def sink_attention(h, T, m, eps, book=None):
    """left half of "parallel": per-head q/k norm with a shared weight, split-half rotation, causal softmax with a sink"""
    n = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos, fr = np.arange(n), rot_freqs(m)
    q = rotate(rms_norm((h @ T["q"].T).reshape(n, H, D), T["q.norm"], eps), pos, fr, False)
    k = rotate(rms_norm((h @ T["k"].T).reshape(n, G, D), T["k.norm"], eps), pos, fr, False)
    v = (h @ T["v"].T).reshape(n, G, V)
    out = np.zeros((n, H, V))
    for a in range(H):
        g = a // (H // G)
        w = softmax_rows(q[:, a] @ k[:, g].T * m["scale"], lambda i: 0, sink=float(T["sink"][a]))
        out[:, a] = w @ v[:, g]
        if book is not None:
            book.setdefault("weights", {})[a] = w
    return out.reshape(n, H * V) @ T["o"].T


def decayed_recurrence(h, T, m, eps, state=None):
    """right half of "parallel": S <- decay S + k v^T, o = S^T q per head, token by token"""
    n = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ T["q"].T).reshape(n, H, D)
    k = silu(h @ T["k"].T).reshape(n, H, D)
    v = silu(h @ T["v"].T).reshape(n, H, V)
    S = np.zeros((H, D, V)) if state is None else state
    out = np.zeros((n, H, V))
    for t in range(n):
        for a in range(H):
            S[a] = m["decay"][a] * S[a] + np.outer(k[t, a], v[t, a])
            out[t, a] = S[a].T @ q[t, a]
    o = rms_norm(out.reshape(n, H * V), T["norm"], eps) * logistic(h @ T["g"].T)
    return o @ T["o"].T


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def dense_ff(h, T):
    return (silu(h @ T["gate"].T) * (h @ T["up"].T)) @ T["down"].T


def relu2_expert(h, up, down):
    return np.maximum(h @ up.T, 0.0) ** 2 @ down.T


def route(scores, top, n_groups, keep):
    """indices of the `top` largest scores among the experts of the `keep` best groups (a group's rank: the sum of its two largest
    scores); ties go to the lower index"""
    E = len(scores)
    size = E // n_groups
    rank = [np.sort(scores[g * size:(g + 1) * size])[::-1][:2].sum() for g in range(n_groups)]
    best = sorted(range(n_groups), key=lambda g: (-rank[g], g))[:keep]
    allowed = [e for e in range(E) if e // size in best]
    return sorted(allowed, key=lambda e: (-scores[e], e))[:top]


def experts_ff(h, T, ml, book=None):
    r = ml["router"]
    E, top = int(r["experts"]), int(r["top"])
    grp = r.get("groups") or {}
    n_groups, keep = int(grp.get("count", 1)), int(grp.get("keep", grp.get("count", 1)))
    s = logistic(h @ T["router"].T)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = route(s[t], top, n_groups, keep)
        if book is not None:
            book.setdefault("choices", []).append(chosen)
            book.setdefault("margin", []).append(np.min(np.abs(np.subtract.outer(s[t], s[t]))[~np.eye(E, dtype=bool)]))
        for e in chosen:
            out[t] += s[t, e] * float(r.get("scale", 1.0)) * relu2_expert(h[t], T[f"e{e}.up"], T[f"e{e}.down"])
    if ml.get("shared"):
        out += relu2_expert(h, T["shared.up"], T["shared.down"])
    return out


def forward(cfg, tensors, tokens, layer_outputs=None, book=None):
    """tensors: name -> float64 arrays.  Returns logits [n, vocab]; layer_outputs (a list) receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = tensors["embed"][np.asarray(tokens)]
    ln = lambda v, name: layer_norm(v, tensors[name], tensors[name + ".b"], eps)
    kv = {}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        h = ln(x, p + "norm1")
        T = sub(tensors, p + "mix.")
        bk = None if book is None else book.setdefault(i, {})
        if l["type"] == "attention":
            y = gated_attention(h, T, m, eps, bk)
        elif l["type"] == "attention_2":
            if m.get("kv_from") is None:
                kv[i] = differential_keys_values(h, T, m)
            y = differential_attention(h, T, m, eps, kv[i if m.get("kv_from") is None else int(m["kv_from"])], bk)
        elif l["type"] == "parallel":
            y = m["left_scale"] * sink_attention(h, sub(T, "left."), m["left"], eps, bk) + m["right_scale"] * decayed_recurrence(h, sub(T, "right."), m["right"], eps)
        else:
            raise ValueError(l["type"])
        x = x + ln(y, p + "norm1b")
        ml = l.get("mlp")
        if ml:
            h = ln(x, p + "norm2")
            T = sub(tensors, p + "mlp.")
            y = dense_ff(h, T) if ml["kind"] == "dense" else experts_ff(h, T, ml, bk)
            x = x + ln(y, p + "norm2b")
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    return ln(x, "final.norm") @ tensors["head"].T


def greedy(cfg, tensors, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(np.argmax(forward(cfg, tensors, toks)[-1])))
    return toks[len(prompt):]
