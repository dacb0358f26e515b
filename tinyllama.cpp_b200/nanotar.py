"""Nanotar: reader of the family's config.json, its tensor inventory, synthetic weights.

A Nanotar model is a list of pre-norm layers over a residual stream that is kept in `streams` copies (hyper-connections): a sublayer
reads a weighted sum of the copies through a Dynamic Tanh norm (tanh(alpha x) * w + b, no statistics) and every copy is rewritten
from all of them plus its own share of the sublayer's output.  Mixers are latent attention -- keys and values are up-projections of
one low-rank latent per token plus one rotary key part shared by the heads, so the cache holds kv_rank + rot_dim numbers per token
-- in two forms: "latent_attention" (direct queries, causal, plain softmax) and "latent_attention_2" (queries through a latent of
their own, a sliding window, a learned sink per head in the softmax denominator); both end in one sigmoid gate per head.
Feed-forward: gated dense with the tanh form of GELU, or routed experts (sigmoid router, the `top` largest scores renormalised,
SiLU-gated experts, a shared expert scaled by a sigmoid gate per token), or none.  The output norm is Dynamic Tanh as well and the
logits are soft-capped.  This module turns config.json into the flat description the native library takes (seq.SeqModel); every
size and constant comes from the config."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from . import safetensors_io as st
from .seq import BLOCK_PRENORM, FF_GATED_EXPERTS, FF_GEGLU, MIX_LATENT_ATTN, NORM_DYT, ROT_INTERLEAVED

ARCHITECTURE = "Nanotar"
MIXERS = {"latent_attention": dict(q_latent=False, window=False, sink=False),
          "latent_attention_2": dict(q_latent=True, window=True, sink=True)}


def _mixer(i: int, kind: str, m: dict) -> dict:
    if kind not in MIXERS:
        raise ValueError(f"layer {i}: unknown type {kind!r}")
    f = MIXERS[kind]
    b = {"kind": MIX_LATENT_ATTN, "name": "", "heads": int(m["heads"]), "dim": int(m["dim"]), "rope_dim": int(m["rot_dim"]), "vdim": int(m["vdim"]),
         "kv_rank": int(m["kv_rank"]), "scale": float(m["scale"]), "gated": 3, "sink": int(f["sink"]), "q_rank": 0, "window": 0}
    rot = m.get("rot")
    if rot and b["rope_dim"] > 0:
        b.update(rot_dims=int(rot["dims"]), rot_base=float(rot["base"]), rot_layout=ROT_INTERLEAVED)
        if b["rot_dims"] > b["rope_dim"] or b["rot_dims"] % 2:
            raise ValueError(f"layer {i}: {b['rot_dims']} rotated entries do not fit a rotated part of {b['rope_dim']}")
    if f["q_latent"]:
        b["q_rank"] = int(m["q_rank"])
    if f["window"]:
        b["window"] = int(m["mask"]["size"])
        if b["window"] <= 0:
            raise ValueError(f"layer {i}: a window of {b['window']} tokens")
    return b


def describe(cfg: dict) -> dict:
    """config.json (parsed) -> description for seq.SeqModel."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: {cfg.get('architecture')!r}")
    d = {"vocab": int(cfg["vocab"]), "width": int(cfg["width"]), "eps": float(cfg["norm"]["eps"]), "final_norm": 2,
         "streams": int(cfg["streams"]), "logit_softcap": float(cfg.get("logit_softcap") or 0.0), "layers": []}
    if d["streams"] < 1:
        raise ValueError(f"{d['streams']} copies of the stream")
    for i, l in enumerate(cfg["layers"]):
        lay = {"style": BLOCK_PRENORM, "norm_kind": NORM_DYT, "branches": [_mixer(i, l.get("type"), l["mixer"])], "ff": 0}
        mlp = l.get("mlp")
        if mlp:
            if mlp.get("kind") == "dense":
                lay.update(ff=int(mlp["ff"]), ff_kind=FF_GEGLU)
            elif mlp.get("kind") == "moe":
                r = mlp["router"]
                lay.update(ff=int(mlp["expert"]["ff"]), ff_kind=FF_GATED_EXPERTS, experts=int(r["experts"]), top=int(r["top"]),
                           shared_ff=int((mlp.get("shared") or {}).get("ff", 0)))
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        d["layers"].append(lay)
    return d


def tensor_shapes(desc: dict) -> dict:
    """name -> shape of every tensor of a checkpoint of this description (all bfloat16)."""
    W, S, out = desc["width"], desc["streams"], {}
    out["embed"] = (desc["vocab"], W)

    def norm(name):
        out.update({name: (W,), name + ".b": (W,), name + ".alpha": ()})

    for i, l in enumerate(desc["layers"]):
        p, b = f"l{i}.", l["branches"][0]
        hd = b["dim"] + b["rope_dim"]
        if b["q_rank"]:
            out.update({p + "mix.dq": (b["q_rank"], W), p + "mix.dq.norm": (b["q_rank"],), p + "mix.uq": (b["heads"] * hd, b["q_rank"])})
        else:
            out[p + "mix.q"] = (b["heads"] * hd, W)
        out.update({p + "mix.dkv": (b["kv_rank"] + b["rope_dim"], W), p + "mix.dkv.norm": (b["kv_rank"],),
                    p + "mix.uk": (b["heads"] * b["dim"], b["kv_rank"]), p + "mix.uv": (b["heads"] * b["vdim"], b["kv_rank"]),
                    p + "mix.g": (b["heads"], W), p + "mix.o": (W, b["heads"] * b["vdim"])})
        if b["sink"]:
            out[p + "mix.sink"] = (b["heads"],)
        for q in (1, 2) if l["ff"] else (1,):
            norm(f"{p}norm{q}")
            out.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
        if l["ff"] and l["ff_kind"] == FF_GEGLU:
            out.update({p + "mlp.gate": (l["ff"], W), p + "mlp.up": (l["ff"], W), p + "mlp.down": (W, l["ff"])})
        elif l["ff"]:
            out[p + "mlp.router"] = (l["experts"], W)
            for e in range(l["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (l["ff"], W), f"{p}mlp.e{e}.up": (l["ff"], W), f"{p}mlp.e{e}.down": (W, l["ff"])})
            if l.get("shared_ff"):
                n = l["shared_ff"]
                out.update({p + "mlp.shared.gate": (n, W), p + "mlp.shared.up": (n, W), p + "mlp.shared.down": (W, n), p + "mlp.shared.sg": (1, W)})
    norm("final.norm")
    out["head"] = (desc["vocab"], W)
    return out


def synth_tensors(desc: dict, seed: int = 0, gain: float = 1.0) -> dict:
    """Random weights (bfloat16 bit patterns): matrices ~ N(0, gain^2 / fan_in), norm weights around one, hyper-connection weights
    around a plain residual sum (read the mean of the copies, keep each copy, give each the whole output)."""
    rng = np.random.default_rng(seed)
    S, out = desc["streams"], {}
    for name, shape in tensor_shapes(desc).items():
        parts = ("." + name).split(".")
        leaf = parts[-1]
        if leaf == "alpha":
            a = np.asarray(0.5 + 0.2 * rng.random())
        elif leaf == "b" and "norm" in parts[-2]:
            a = 0.1 * rng.standard_normal(shape)
        elif leaf in ("norm1", "norm2") or name == "final.norm" or name.endswith(".norm"):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif parts[-2].startswith("hc"):
            a = {"in": np.full(shape, 1.0 / S), "out": np.ones(shape), "mix": np.eye(S)}[leaf] + 0.2 * rng.standard_normal(shape)
        elif leaf == "sink":
            a = rng.standard_normal(shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        elif leaf in ("router", "sg"):
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


def latent_layer(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, q_rank=None, window=None, rot_dims=None, rot_base=10000.0, scale=None, mlp=None) -> dict:
    """One entry of config["layers"]: with q_rank and window the second form (query latent, sliding window, sink), else the first."""
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": float((dim + rot_dim) ** -0.5 if scale is None else scale),
         "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": rot_base}}
    second = q_rank is not None or window is not None
    if second:
        m.update(q_rank=int(q_rank or 16), mask={"size": int(window or 8)})
    return {"type": "latent_attention_2" if second else "latent_attention", "mixer": m, "mlp": mlp}


def dense_mlp(ff=40) -> dict:
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts=6, top=2, ff=24, shared_ff=16) -> dict:
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def make_config(vocab=96, width=48, streams=3, layers=None, eps=1e-5, logit_softcap=20.0) -> dict:
    """A config.json dictionary for tests, benchmarks and examples."""
    if layers is None:
        layers = [latent_layer(mlp=dense_mlp()), latent_layer(q_rank=16, window=8, heads=2, vdim=8, mlp=moe_mlp()), latent_layer(mlp=moe_mlp(shared_ff=0))]
    return {"architecture": ARCHITECTURE, "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps}, "logit_softcap": logit_softcap, "layers": layers}
