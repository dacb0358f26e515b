"""Plain restatement of the Nanotar family in numpy float64: one function per mechanism, whole sequences only, no cache, no step
function, nothing shared with the product path.  Tests compare the native library against it.

A Nanotar model keeps `streams` copies of the residual stream (hyper-connections).  Sublayer q of a layer reads the mix
u = sum_s in_q[s] x_s, computes y = f(dyt(u)) and rewrites all streams at once, x_t <- sum_s mix_q[s, t] x_s + out_q[t] y.  dyt is
the Dynamic Tanh norm tanh(alpha v) w + b.  Mixers are latent attention: keys and values are up-projections of one low-rank latent
per token plus one rotary key part shared by the heads; optional query latent, sliding window, sink in the softmax denominator;
one sigmoid gate per head.  Feed-forward: gated dense (tanh-GELU) or routed experts (sigmoid router, top-k, renormalised weights,
SiLU-gated experts, a gated shared expert).  The logits are soft-capped."""
from __future__ import annotations

import numpy as np


def dyt(v, alpha, w, b):
    return np.tanh(alpha * v) * w + b


def unit_rms(v, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def logistic(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * logistic(z)


def rotate_pairs(v, positions, dims, base):
    """v [T, ..., n]: entries (2i, 2i+1), i < dims/2, of the last axis turn by positions[t] * base^(-2i/dims); the rest stay."""
    out = np.array(v, np.float64)
    T = v.shape[0]
    pos = np.asarray(positions, np.float64).reshape((T,) + (1,) * (v.ndim - 2))
    for i in range(dims // 2):
        a = pos * float(base) ** (-2.0 * i / dims)
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * np.cos(a) - w * np.sin(a)
        out[..., 2 * i + 1] = w * np.cos(a) + u * np.sin(a)
    return out


def visible(i, window):
    """first key position that query position i sees (window 0: everything before it)"""
    return max(0, i - window + 1) if window > 0 else 0


def softmax_with_sink(scores, sink):
    """weights over the given scores when the denominator may hold one extra exp(sink) that carries no value"""
    m = np.max(scores) if sink is None else max(np.max(scores), sink)
    e = np.exp(scores - m)
    den = e.sum() + (0.0 if sink is None else np.exp(sink - m))
    return e / den


def latent_attention(h, T, mx, eps, first_pos=0, book=None):
    """h [T, width] -> [T, width].  T: tensors of the mixer by their short names; mx: the layer's `mixer` section.
    book: a list that receives (query position, head, first visible key, softmax weights of the visible keys)."""
    H, dn, dr, dv, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    n = h.shape[0]
    pos = np.arange(first_pos, first_pos + n)
    if "q_rank" in mx:
        cq = unit_rms(h @ T["dq"].T, eps) * T["dq.norm"]
        q = cq @ T["uq"].T
    else:
        q = h @ T["q"].T
    q = q.reshape(n, H, dn + dr)
    dkv = h @ T["dkv"].T
    c = unit_rms(dkv[:, :rank], eps) * T["dkv.norm"]
    rot = mx.get("rot") or {"dims": 0, "base": 1.0}
    k_rot = rotate_pairs(dkv[:, rank:], pos, rot["dims"], rot["base"])                    # [n, dr], one for all heads
    q_rot = rotate_pairs(q[:, :, dn:], pos, rot["dims"], rot["base"])
    k_plain = (c @ T["uk"].T).reshape(n, H, dn)
    val = (c @ T["uv"].T).reshape(n, H, dv)
    gate = logistic(h @ T["g"].T)                                                        # [n, H]
    window = int((mx.get("mask") or {}).get("size", 0))
    out = np.zeros((n, H, dv))
    for i in range(n):
        lo = visible(i, window)
        for a in range(H):
            s = (k_plain[lo:i + 1, a] @ q[i, a, :dn] + k_rot[lo:i + 1] @ q_rot[i, a]) * mx["scale"]
            w = softmax_with_sink(s, T["sink"][a] if "sink" in T else None)
            if book is not None:
                book.append((i, a, lo, w))
            out[i, a] = (w @ val[lo:i + 1, a]) * gate[i, a]
    return out.reshape(n, H * dv) @ T["o"].T


def gated_ff(h, gate, up, down, act):
    return (act(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router, top):
    """per token: indices of the `top` largest sigmoid scores (ties to the lower index) and their weights, which sum to one"""
    s = logistic(h @ router.T)
    idx = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    w = np.take_along_axis(s, idx, axis=-1)
    return idx, w / (w.sum(axis=-1, keepdims=True) + 1e-20)


def experts_ff(h, T, ml):
    idx, w = route(h, T["router"], ml["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(idx[t], w[t]):
            out[t] += we * gated_ff(h[t:t + 1], T[f"e{e}.gate"], T[f"e{e}.up"], T[f"e{e}.down"], silu)[0]
    if "shared" in ml:
        out += logistic(h @ T["shared.sg"].T) * gated_ff(h, T["shared.gate"], T["shared.up"], T["shared.down"], silu)
    return out


def feed_forward(h, T, ml):
    if ml["kind"] == "dense":
        return gated_ff(h, T["gate"], T["up"], T["down"], gelu_tanh)
    return experts_ff(h, T, ml)


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def hyper_update(xs, hc, f):
    """xs [streams, T, width]: one sublayer under hyper-connections.  hc: {"in" [s], "out" [s], "mix" [s from, s to]}."""
    u = np.tensordot(hc["in"], xs, axes=(0, 0))
    y = f(u)
    return np.tensordot(hc["mix"].T, xs, axes=(1, 0)) + hc["out"][:, None, None] * y[None]


def to_float(bits):
    """bfloat16 bit patterns -> float64"""
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def forward(cfg, tensors, tokens, layer_outputs=None, book=None):
    """tokens -> logits [T, vocab] of a whole sequence from position 0.  tensors: name -> float64 array.
    layer_outputs: a list that receives the sum of the streams after every layer."""
    eps = cfg["norm"]["eps"]
    x = tensors["embed"][np.asarray(tokens)]
    xs = np.stack([x] * int(cfg.get("streams", 1)))
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        n1 = lambda v: dyt(v, tensors[p + "norm1.alpha"], tensors[p + "norm1"], tensors[p + "norm1.b"])
        bk = [] if book is not None else None
        xs = hyper_update(xs, sub(tensors, p + "hc1."), lambda u: latent_attention(n1(u), sub(tensors, p + "mix."), lay["mixer"], eps, book=bk))
        if book is not None:
            book.append(bk)
        if lay.get("mlp"):
            n2 = lambda v: dyt(v, tensors[p + "norm2.alpha"], tensors[p + "norm2"], tensors[p + "norm2.b"])
            xs = hyper_update(xs, sub(tensors, p + "hc2."), lambda u: feed_forward(n2(u), sub(tensors, p + "mlp."), lay["mlp"]))
        if layer_outputs is not None:
            layer_outputs.append(xs.sum(axis=0))
    xf = dyt(xs.sum(axis=0), tensors["final.norm.alpha"], tensors["final.norm"], tensors["final.norm.b"])
    logits = xf @ tensors["head"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * np.tanh(logits / cap) if cap > 0 else logits


def greedy(cfg, tensors, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(np.argmax(forward(cfg, tensors, toks)[-1])))
    return toks[len(prompt):]
