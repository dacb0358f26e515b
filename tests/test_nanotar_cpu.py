"""CPU-side pieces of the Nanotar family: the config reader on every constant and on absent sections, the tensor inventory, the
registry and checkpoint folder, the binding's structures against the C header, and closed forms of the restatement's own building
blocks (oracle/nanotar_ref.py)."""
import ctypes as C
import json
import re
from pathlib import Path

import numpy as np
import pytest

from oracle import nanotar_ref as R
from tinyllama_cpp_b200 import nanotar as NT, registry, seq

ROOT = Path(__file__).resolve().parent.parent


def test_describe_reads_every_constant():
    layers = [NT.latent_layer(heads=5, dim=6, rot_dim=10, vdim=14, kv_rank=22, rot_dims=4, rot_base=777.0, scale=0.21, mlp=NT.moe_mlp(experts=7, top=3, ff=28, shared_ff=36)),
              NT.latent_layer(heads=2, dim=12, rot_dim=4, vdim=8, kv_rank=18, q_rank=26, window=19, rot_base=5e5, scale=0.4, mlp=NT.dense_mlp(44)),
              NT.latent_layer(heads=3, dim=4, rot_dim=2, vdim=4, kv_rank=6)]
    cfg = NT.make_config(vocab=55, width=40, streams=4, layers=layers, eps=3e-4, logit_softcap=12.5)
    d = NT.describe(cfg)
    assert (d["vocab"], d["width"], d["eps"], d["streams"], d["logit_softcap"], d["final_norm"]) == (55, 40, 3e-4, 4, 12.5, 2)
    a, b, c = (l["branches"][0] for l in d["layers"])
    assert all(l["style"] == seq.BLOCK_PRENORM and l["norm_kind"] == seq.NORM_DYT for l in d["layers"])
    assert (a["kind"], a["heads"], a["dim"], a["rope_dim"], a["vdim"], a["kv_rank"], a["q_rank"], a["window"], a["sink"], a["gated"]) == (seq.MIX_LATENT_ATTN, 5, 6, 10, 14, 22, 0, 0, 0, 3)
    assert (a["rot_dims"], a["rot_base"], a["rot_layout"], a["scale"]) == (4, 777.0, seq.ROT_INTERLEAVED, 0.21)
    assert (b["q_rank"], b["window"], b["sink"], b["rot_dims"], b["rot_base"], b["scale"]) == (26, 19, 1, 4, 5e5, 0.4)
    l0, l1, l2 = d["layers"]
    assert (l0["ff_kind"], l0["ff"], l0["experts"], l0["top"], l0["shared_ff"]) == (seq.FF_GATED_EXPERTS, 28, 7, 3, 36)
    assert (l1["ff_kind"], l1["ff"]) == (seq.FF_GEGLU, 44) and l2["ff"] == 0
    sh = NT.tensor_shapes(d)
    assert sh["l0.mix.q"] == (80, 40) and sh["l0.mix.dkv"] == (32, 40) and sh["l0.mix.dkv.norm"] == (22,) and sh["l0.mix.uk"] == (30, 22) and sh["l0.mix.uv"] == (70, 22)
    assert sh["l0.mix.g"] == (5, 40) and sh["l0.mix.o"] == (40, 70) and "l0.mix.sink" not in sh and "l0.mix.dq" not in sh
    assert sh["l1.mix.dq"] == (26, 40) and sh["l1.mix.dq.norm"] == (26,) and sh["l1.mix.uq"] == (32, 26) and sh["l1.mix.sink"] == (2,) and "l1.mix.q" not in sh
    assert sh["l0.mlp.router"] == (7, 40) and sh["l0.mlp.e6.gate"] == (28, 40) and sh["l0.mlp.e6.down"] == (40, 28) and "l0.mlp.e7.up" not in sh
    assert sh["l0.mlp.shared.up"] == (36, 40) and sh["l0.mlp.shared.down"] == (40, 36) and sh["l0.mlp.shared.sg"] == (1, 40)
    assert sh["l1.mlp.gate"] == (44, 40) and sh["l1.mlp.down"] == (40, 44)
    assert sh["l0.hc1.in"] == (4,) and sh["l0.hc2.mix"] == (4, 4) and sh["l0.norm2.alpha"] == () and sh["l0.norm1.b"] == (40,)
    assert "l2.norm2" not in sh and "l2.hc2.in" not in sh and sh["l2.hc1.out"] == (4,)
    assert sh["final.norm"] == (40,) and sh["final.norm.b"] == (40,) and sh["final.norm.alpha"] == () and sh["head"] == (55, 40)
    with pytest.raises(ValueError):
        NT.describe(dict(cfg, architecture="Other"))
    for path, value in ((("layers", 0, "type"), "attention"), (("layers", 1, "mlp", "kind"), "gated"), (("layers", 0, "mixer", "rot", "dims"), 12),
                        (("layers", 0, "mixer", "rot", "dims"), 3), (("layers", 1, "mixer", "mask", "size"), 0), (("streams",), 0)):
        bad = json.loads(json.dumps(cfg))
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ValueError):
            NT.describe(bad)


def test_optional_sections_may_be_absent():
    cfg = NT.make_config(layers=[NT.latent_layer(rot_dim=0), NT.latent_layer(mlp=NT.moe_mlp(shared_ff=0))])
    del cfg["layers"][0]["mixer"]["rot"]
    del cfg["logit_softcap"]
    d = NT.describe(cfg)
    a = d["layers"][0]["branches"][0]
    assert d["logit_softcap"] == 0.0 and a["rope_dim"] == 0 and a.get("rot_dims", 0) == 0 and d["layers"][1]["shared_ff"] == 0
    sh = NT.tensor_shapes(d)
    assert sh["l0.mix.dkv"] == (20, 48) and "l1.mlp.shared.sg" not in sh


def test_registry_and_checkpoint_folder(tmp_path):
    cfg = NT.make_config()
    t = NT.synth_tensors(NT.describe(cfg), 1)
    NT.write_checkpoint(tmp_path / "m", cfg, t)
    assert registry.family_of(tmp_path / "m") == "Nanotar" and "Nanotar" in registry.STEPWISE
    desc, back = NT.read_checkpoint(tmp_path / "m")
    assert set(back) == set(NT.tensor_shapes(desc)) and all(np.array_equal(back[k], t[k]) for k in t)
    assert back["l0.norm1.alpha"].shape == ()


def test_binding_structures_follow_the_header():
    """Field names and order of the ctypes structures are those of include/gten_b200_seq.h; so are the enumerators."""
    hdr = (ROOT / "include" / "gten_b200_seq.h").read_text()

    def fields(struct):
        body = hdr[:hdr.index("} " + struct + ";")].rsplit("typedef struct {", 1)[1]
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                names.append(re.sub(r"\[.*\]", "", part.strip().split()[-1].lstrip("*")))
        return names
    assert fields("gtb_seq_branch") == [f[0] for f in seq.BranchC._fields_]
    assert fields("gtb_seq_layer") == [f[0] for f in seq.LayerC._fields_]
    assert fields("gtb_seq_config") == [f[0] for f in seq.ConfigC._fields_]
    enums = dict(re.findall(r"(GTB_[A-Z0-9_]+) = (\d+)", hdr))
    for name, value in (("MIX_LATENT_ATTN", seq.MIX_LATENT_ATTN), ("BLOCK_PRENORM", seq.BLOCK_PRENORM), ("FF_GATED_EXPERTS", seq.FF_GATED_EXPERTS),
                        ("NORM_DYT", seq.NORM_DYT), ("NORM_RMS", seq.NORM_RMS), ("MIX_SOFTMAX_ATTN", seq.MIX_SOFTMAX_ATTN), ("FF_EXPERTS", seq.FF_EXPERTS)):
        assert int(enums["GTB_" + name]) == value
    assert C.sizeof(seq.BranchC) % 8 == 0


def test_restatement_norm_and_hyper_connections():
    v = np.array([-3.0, 0.0, 0.5])
    assert np.allclose(R.dyt(v, 2.0, np.array([1.0, 2.0, 3.0]), np.array([0.1, 0.2, 0.3])), np.tanh(2 * v) * [1, 2, 3] + [0.1, 0.2, 0.3])
    assert np.allclose(R.unit_rms(np.array([[3.0, 4.0]]), 0.0), [[3 / np.sqrt(12.5), 4 / np.sqrt(12.5)]])
    rng = np.random.default_rng(0)
    xs = rng.standard_normal((2, 3, 4))
    hc = {"in": np.array([0.25, 0.75]), "out": np.array([2.0, -1.0]), "mix": np.array([[1.0, 0.5], [0.0, 3.0]])}      # [from, to]
    out = R.hyper_update(xs, hc, lambda u: u + 1.0)
    y = 0.25 * xs[0] + 0.75 * xs[1] + 1.0
    assert np.allclose(out[0], 1.0 * xs[0] + 0.0 * xs[1] + 2.0 * y) and np.allclose(out[1], 0.5 * xs[0] + 3.0 * xs[1] - 1.0 * y)


def test_restatement_latent_attention_is_attention_over_expanded_keys():
    """With one head, no rotated part and no gate effect removed, the mixer equals a textbook softmax attention whose keys and values are
    uk c and uv c; a window of one token leaves only the token itself; a sink that dwarfs the scores empties the output."""
    rng = np.random.default_rng(1)
    n, W_, dn, dv, rank = 7, 10, 4, 5, 6
    h = rng.standard_normal((n, W_))
    T = {"q": rng.standard_normal((dn, W_)), "dkv": rng.standard_normal((rank, W_)), "dkv.norm": rng.standard_normal(rank), "uk": rng.standard_normal((dn, rank)),
         "uv": rng.standard_normal((dv, rank)), "g": np.zeros((1, W_)), "o": np.eye(dv)}
    mx = {"heads": 1, "dim": dn, "rot_dim": 0, "vdim": dv, "kv_rank": rank, "scale": 0.3}
    got = R.latent_attention(h, T, mx, 1e-6)
    c = R.unit_rms(h @ T["dkv"].T, 1e-6) * T["dkv.norm"]
    k, v, q = c @ T["uk"].T, c @ T["uv"].T, h @ T["q"].T
    want = np.zeros((n, dv))
    for i in range(n):
        s = np.exp(0.3 * k[:i + 1] @ q[i])
        want[i] = 0.5 * (s / s.sum()) @ v[:i + 1]                # the gate's logit is zero: one half
    assert np.allclose(got, want)
    T2 = dict(T, dq=rng.standard_normal((3, W_)), uq=rng.standard_normal((dn, 3)), sink=np.array([-50.0]))
    T2["dq.norm"] = np.ones(3)
    one = R.latent_attention(h, T2, dict(mx, q_rank=3, mask={"size": 1}), 1e-6)
    assert np.allclose(one, 0.5 * v)
    T2["sink"] = np.array([60.0])
    assert np.abs(R.latent_attention(h, T2, dict(mx, q_rank=3, mask={"size": 4}), 1e-6)).max() < 1e-12


def test_restatement_experts():
    h = np.array([[1.0, 0.0, 0.0]])
    router = np.array([[0.0, 0, 0], [1.0, 0, 0], [2.0, 0, 0], [0.5, 0, 0]])
    idx, w = R.route(h, router, 2)
    s = 1 / (1 + np.exp(-np.array([0.0, 1.0, 2.0, 0.5])))
    assert idx.tolist() == [[2, 1]] and np.allclose(w, [[s[2] / (s[2] + s[1]), s[1] / (s[2] + s[1])]])
    idx, _ = R.route(h, np.zeros((4, 3)), 2)
    assert idx.tolist() == [[0, 1]]                              # ties go to the lower index
    T = {"router": router, "shared.sg": np.array([[0.0, 0, 0]])}
    for e in range(4):
        T[f"e{e}.gate"], T[f"e{e}.up"], T[f"e{e}.down"] = np.full((2, 3), float(e)), np.ones((2, 3)), np.ones((3, 2))
    T["shared.gate"], T["shared.up"], T["shared.down"] = np.ones((2, 3)), np.ones((2, 3)), np.ones((3, 2))
    y = R.experts_ff(h, T, {"kind": "moe", "router": {"experts": 4, "top": 2}, "shared": {"ff": 2}})
    silu = lambda z: z / (1 + np.exp(-z))
    want = 2 * (w[0, 0] * silu(2.0) + w[0, 1] * silu(1.0)) + 0.5 * 2 * silu(1.0)
    assert np.allclose(y, want)
    assert np.allclose(R.gelu_tanh(np.array([0.0, 10.0, -10.0])), [0.0, 10.0, 0.0], atol=1e-6)


def test_logits_are_soft_capped():
    cfg = NT.make_config(vocab=30, width=16, streams=2, layers=[NT.latent_layer(heads=2, dim=4, rot_dim=2, vdim=4, kv_rank=6)], logit_softcap=1.5)
    t = NT.synth_tensors(NT.describe(cfg), 3, gain=4.0)
    W = {k: R.to_float(v) for k, v in t.items()}
    a = R.forward(cfg, W, [1, 2, 3, 4])
    raw = R.forward(dict(cfg, logit_softcap=0.0), W, [1, 2, 3, 4])
    assert np.abs(a).max() < 1.5 and np.allclose(a, 1.5 * np.tanh(raw / 1.5))
    assert R.greedy(cfg, W, [1, 2], 3) == R.greedy(dict(cfg, logit_softcap=0.0), W, [1, 2], 3)       # the cap is monotonic
