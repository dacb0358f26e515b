"""Vulosun: reader of the family's config.json, its tensor inventory, synthetic weights.

A Vulosun model is a list of sandwich layers: x += norm1b(mixer(norm1(x))), then x += norm2b(ff(norm2(x))), all four norms layer norms
with weight and bias.  config.json lists the layers; each names its mixer --
"attention": softmax attention with grouped K/V heads, one RMS norm with a weight over the whole query projection and one over the whole
key projection, interleaved rotary pairs, one sigmoid gate per head;
"attention_2": differential attention (two score maps per head over the same values, combined as a1 - lambda a2, unit RMS per head, a
constant factor, a gate per head) with projection biases, rotary frequencies divided by a constant, a chunked causal mask, and
optionally the keys and values of an earlier layer's cache ("kv_from");
"parallel": the weighted sum of a left branch -- softmax attention with a weighted per-head q/k norm, split-half rotary pairs and a
learned sink in the denominator -- and a right branch -- a per-head linear recurrence with a fixed decay over SiLU-activated q, k, v
whose concatenated heads are RMS-normed with a weight, gated by a sigmoid and projected --
and its feed-forward: SiLU-gated dense, routed squared-ReLU experts (sigmoid scores, group-limited choice, scaled unrenormalised
weights, a shared expert), or none.  This module turns config.json into the flat description the native library takes
(seq.SeqModel); every size and constant comes from the config."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from . import safetensors_io as st
from .seq import BLOCK_SANDWICH, FF_GROUP_EXPERTS, FF_SWIGLU, MIX_RETENTION, MIX_SOFTMAX_ATTN, NORM_LAYER, ROT_HALVES, ROT_INTERLEAVED

ARCHITECTURE = "Vulosun"


def _softmax_branch(i: int, m: dict, name: str = "") -> dict:
    b = {"kind": MIX_SOFTMAX_ATTN, "name": name, "heads": int(m["heads"]), "kv_heads": int(m.get("kv_heads", m["heads"])), "dim": int(m["dim"]),
         "vdim": int(m.get("vdim", m["dim"])), "scale": float(m["scale"]), "kv_from": -1, "maps": 1}
    if b["heads"] % b["kv_heads"]:
        raise ValueError(f"layer {i}: {b['heads']} query heads do not divide into {b['kv_heads']} key/value heads")
    return b


def _rotation(i: int, b: dict, m: dict, layout: int) -> None:
    rot = m.get("rot")
    if rot and int(rot.get("dims") or 0) > 0:
        b.update(rot_dims=int(rot["dims"]), rot_base=float(rot["base"]), rot_layout=layout)
        if b["rot_dims"] > b["dim"] or b["rot_dims"] % 2:
            raise ValueError(f"layer {i}: {b['rot_dims']} rotated entries do not fit a head of {b['dim']}")
        sc = rot.get("scaling")
        if sc:
            b["rot_divide"] = float(sc["factor"])
            if b["rot_divide"] <= 0.0:
                raise ValueError(f"layer {i}: rotary frequencies divided by {b['rot_divide']}")


def _shared_cache(i: int, b: dict, m: dict) -> None:
    if m.get("kv_from") is not None:
        b["kv_from"] = int(m["kv_from"])
        if not 0 <= b["kv_from"] < i:
            raise ValueError(f"layer {i}: kv_from {b['kv_from']} is not an earlier layer")


def _mixer(i: int, kind: str, m: dict) -> list:
    if kind == "attention":
        b = _softmax_branch(i, m)
        b.update(qk_norm=3, gated=3)
        _rotation(i, b, m, ROT_INTERLEAVED)
        _shared_cache(i, b, m)
        return [b]
    if kind == "attention_2":
        b = _softmax_branch(i, m)
        b.update(maps=2, diff=float(m["diff"]), bias=1, gated=3)
        _rotation(i, b, m, ROT_INTERLEAVED)
        mask = m.get("mask")
        if mask and mask.get("size"):
            b["chunk"] = int(mask["size"])
            if b["chunk"] <= 0:
                raise ValueError(f"layer {i}: chunks of {b['chunk']} positions")
        _shared_cache(i, b, m)
        return [b]
    if kind == "parallel":
        le, ri = m["left"], m["right"]
        left = _softmax_branch(i, le, "left")
        left.update(qk_norm=2, sink=1, out_scale=float(m["left_scale"]))
        _rotation(i, left, le, ROT_HALVES)
        if len(ri["decay"]) != int(ri["heads"]):
            raise ValueError(f"layer {i}: {len(ri['decay'])} decays for {ri['heads']} heads")
        right = {"kind": MIX_RETENTION, "name": "right", "heads": int(ri["heads"]), "dim": int(ri["dim"]), "vdim": int(ri["vdim"]), "scale": 1.0,
                 "act": 1, "out_norm": 2, "gated": 2, "decay": [float(x) for x in ri["decay"]], "out_scale": float(m["right_scale"])}
        return [left, right]
    raise ValueError(f"layer {i}: unknown type {kind!r}")


def describe(cfg: dict) -> dict:
    """config.json (parsed) -> description for seq.SeqModel."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: {cfg.get('architecture')!r}")
    d = {"vocab": int(cfg["vocab"]), "width": int(cfg["width"]), "eps": float(cfg["norm"]["eps"]), "final_norm": 3, "layers": []}
    for i, l in enumerate(cfg["layers"]):
        lay = {"style": BLOCK_SANDWICH, "norm_kind": NORM_LAYER, "branches": _mixer(i, l.get("type"), l["mixer"]), "ff": 0}
        mlp = l.get("mlp")
        if mlp:
            if mlp.get("kind") == "dense":
                lay.update(ff=int(mlp["ff"]), ff_kind=FF_SWIGLU)
            elif mlp.get("kind") == "moe":
                r = mlp["router"]
                g = r.get("groups") or {}
                lay.update(ff=int(mlp["expert"]["ff"]), ff_kind=FF_GROUP_EXPERTS, experts=int(r["experts"]), top=int(r["top"]),
                           route_groups=int(g.get("count") or 1), route_keep=int(g.get("keep") or g.get("count") or 1), route_scale=float(r.get("scale", 1.0)),
                           shared_ff=int((mlp.get("shared") or {}).get("ff", 0)))
                if lay["experts"] % lay["route_groups"] or not 0 < lay["route_keep"] <= lay["route_groups"]:
                    raise ValueError(f"layer {i}: {lay['experts']} experts in {lay['route_groups']} groups, {lay['route_keep']} kept")
                if lay["top"] > lay["route_keep"] * (lay["experts"] // lay["route_groups"]):
                    raise ValueError(f"layer {i}: {lay['top']} choices from {lay['route_keep']} groups of {lay['experts'] // lay['route_groups']}")
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        d["layers"].append(lay)
    for i, lay in enumerate(d["layers"]):            # a shared cache must fit the layer that reads it
        b = lay["branches"][0]
        if b.get("kv_from", -1) >= 0:
            src = d["layers"][b["kv_from"]]["branches"]
            if len(src) != 1 or src[0]["kind"] != MIX_SOFTMAX_ATTN or src[0].get("kv_from", -1) >= 0:
                raise ValueError(f"layer {i}: kv_from {b['kv_from']} is not an attention layer with keys and values of its own")
            if any(src[0].get(k) != b.get(k) for k in ("kv_heads", "dim", "vdim", "maps")):
                raise ValueError(f"layer {i}: head sizes differ from those of layer {b['kv_from']}, whose cache it reads")
    return d


def tensor_shapes(desc: dict) -> dict:
    """name -> shape of every tensor of a checkpoint of this description (all bfloat16)."""
    W, out = desc["width"], {}
    out["embed"] = (desc["vocab"], W)

    def norm(name):
        out.update({name: (W,), name + ".b": (W,)})

    for i, l in enumerate(desc["layers"]):
        p = f"l{i}."
        for b in l["branches"]:
            bp = p + "mix." + (b["name"] + "." if b["name"] else "")
            H, D, V = b["heads"], b["dim"], b["vdim"]
            if b["kind"] == MIX_RETENTION:
                out.update({bp + "q": (H * D, W), bp + "k": (H * D, W), bp + "v": (H * V, W), bp + "g": (H * V, W), bp + "norm": (H * V,), bp + "o": (W, H * V)})
                continue
            G, M = b["kv_heads"], b.get("maps", 1)
            own = b.get("kv_from", -1) < 0
            out[bp + "q"] = (H * M * D, W)
            if own:
                out[bp + "k"] = (G * M * D, W)
                out[bp + "v"] = (G * V, W)
            if b.get("bias"):
                out[bp + "q.b"] = (H * M * D,)
                if own:
                    out.update({bp + "k.b": (G * M * D,), bp + "v.b": (G * V,)})
            if b.get("qk_norm") == 3:
                out[bp + "q.norm"] = (H * M * D,)
                if own:
                    out[bp + "k.norm"] = (G * M * D,)
            elif b.get("qk_norm") == 2:
                out[bp + "q.norm"] = (D,)
                if own:
                    out[bp + "k.norm"] = (D,)
            if M == 2:
                out.update({bp + n: (D,) for n in ("lq1", "lk1", "lq2", "lk2")})
            if b.get("sink"):
                out[bp + "sink"] = (H,)
            if b.get("gated") == 3:
                out[bp + "g"] = (H, W)
            out[bp + "o"] = (W, H * V)
        for q in ("1", "1b") + (("2", "2b") if l["ff"] else ()):
            norm(p + "norm" + q)
        if l["ff"] and l["ff_kind"] == FF_SWIGLU:
            out.update({p + "mlp.gate": (l["ff"], W), p + "mlp.up": (l["ff"], W), p + "mlp.down": (W, l["ff"])})
        elif l["ff"]:
            out[p + "mlp.router"] = (l["experts"], W)
            for e in range(l["experts"]):
                out.update({f"{p}mlp.e{e}.up": (l["ff"], W), f"{p}mlp.e{e}.down": (W, l["ff"])})
            if l.get("shared_ff"):
                out.update({p + "mlp.shared.up": (l["shared_ff"], W), p + "mlp.shared.down": (W, l["shared_ff"])})
    norm("final.norm")
    out["head"] = (desc["vocab"], W)
    return out


def synth_tensors(desc: dict, seed: int = 0, gain: float = 1.0) -> dict:
    """Random weights (bfloat16 bit patterns): matrices ~ N(0, gain^2 / fan_in), norm weights around one, small biases."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(desc).items():
        parts = name.split(".")
        leaf = parts[-1]
        if leaf == "b":
            a = 0.1 * rng.standard_normal(shape)
        elif leaf == "norm" or leaf.startswith("norm"):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            a = 0.3 * rng.standard_normal(shape)
        elif leaf == "sink":
            a = rng.standard_normal(shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        elif leaf == "router" or (leaf == "g" and shape[0] < shape[1] // 2):
            a = rng.standard_normal(shape) * 2.0 * gain / np.sqrt(shape[-1])
        else:
            a = rng.standard_normal(shape) * gain / np.sqrt(shape[-1])
        out[name] = st.f32_to_bf16_bits(np.asarray(a, np.float32))
    return out


def read_checkpoint(model_dir) -> tuple[dict, dict]:
    """(description, name -> bfloat16 bit patterns) of a folder with config.json and model.safetensors."""
    model_dir = Path(model_dir)
    desc = describe(json.loads((model_dir / "config.json").read_text()))
    return desc, st.read_as_bf16(model_dir / "model.safetensors", tensor_shapes(desc), ARCHITECTURE)


def write_checkpoint(model_dir, cfg: dict, tensors: dict) -> None:
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    (model_dir / "config.json").write_text(json.dumps(cfg, indent=1))
    st.write(model_dir / "model.safetensors", {k: ("BF16", v) for k, v in tensors.items()})


def gated_attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, rot_base=10000.0, scale=None, mlp=None) -> dict:
    """One "attention" entry of config["layers"]."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(dim ** -0.5 if scale is None else scale)}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": rot_base}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def differential_layer(heads=4, kv_heads=2, dim=16, vdim=24, diff=0.4, chunk=16, rot_dims=8, rot_base=10000.0, factor=2.0, scale=None, kv_from=None, mlp=None) -> dict:
    """One "attention_2" entry of config["layers"]."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": float(dim ** -0.5 if scale is None else scale)}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": rot_base}
        if factor:
            m["rot"]["scaling"] = {"factor": factor}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def parallel_layer(heads=4, kv_heads=2, dim=16, vdim=16, rot_dims=8, rot_base=10000.0, scale=None, r_heads=2, r_dim=16, r_vdim=24, decay=None,
                   left_scale=0.8, right_scale=1.3, mlp=None) -> dict:
    """One "parallel" entry of config["layers"]."""
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(dim ** -0.5 if scale is None else scale)}
    if rot_dims:
        left["rot"] = {"dims": rot_dims, "base": rot_base}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": [float(1.0 - 2.0 ** (-2 - 2 * h)) for h in range(r_heads)] if decay is None else list(decay)}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right": right, "right_scale": right_scale}, "mlp": mlp}


def dense_mlp(ff=40) -> dict:
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts=8, top=2, ff=24, groups=4, keep=2, scale=1.25, shared_ff=40) -> dict:
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if groups:
        m["router"]["groups"] = {"count": groups, "keep": keep}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def make_config(vocab=96, width=48, layers=None, eps=1e-5) -> dict:
    """A config.json dictionary for tests, benchmarks and examples."""
    if layers is None:
        layers = [differential_layer(mlp=dense_mlp()), parallel_layer(mlp=moe_mlp()), gated_attention_layer(mlp=moe_mlp(shared_ff=0)),
                  differential_layer(kv_from=0, mlp=moe_mlp())]
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
