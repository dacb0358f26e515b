"""CPU-side pieces of the Vulosun family: the config reader on every constant and on absent sections, the tensor inventory, the
registry and checkpoint folder, and closed forms of the restatement's own building blocks (oracle/vulosun_ref.py)."""
import numpy as np
import pytest

from oracle import vulosun_ref as R
from tinyllama_cpp_b200 import registry, seq, vulosun as VU


def test_describe_reads_every_constant():
    layers = [VU.differential_layer(heads=6, kv_heads=3, dim=10, vdim=14, diff=0.35, chunk=12, rot_dims=6, rot_base=777.0, factor=3.5, scale=0.21, mlp=VU.dense_mlp(44)),
              VU.parallel_layer(heads=4, kv_heads=1, dim=12, vdim=20, rot_dims=4, rot_base=55.0, scale=0.3, r_heads=3, r_dim=8, r_vdim=10, decay=[0.5, 0.9, 0.99],
                                left_scale=0.7, right_scale=1.9, mlp=VU.moe_mlp(experts=9, top=2, ff=20, groups=3, keep=2, scale=2.5, shared_ff=28)),
              VU.gated_attention_layer(heads=2, kv_heads=2, dim=6, vdim=8, rot_dims=6, rot_base=31.0, scale=0.9),
              VU.differential_layer(heads=6, kv_heads=3, dim=10, vdim=14, diff=0.1, chunk=5, rot_dims=6, rot_base=777.0, factor=3.5, kv_from=0)]
    d = VU.describe(VU.make_config(vocab=70, width=36, layers=layers, eps=2e-4))
    assert (d["vocab"], d["width"], d["eps"], d["final_norm"]) == (70, 36, 2e-4, 3)
    assert all(l["style"] == seq.BLOCK_SANDWICH and l["norm_kind"] == seq.NORM_LAYER for l in d["layers"])
    a = d["layers"][0]["branches"][0]
    assert (a["kind"], a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["maps"], a["diff"], a["chunk"], a["bias"], a["gated"]) == (seq.MIX_SOFTMAX_ATTN, 6, 3, 10, 14, 2, 0.35, 12, 1, 3)
    assert (a["rot_dims"], a["rot_base"], a["rot_divide"], a["rot_layout"], a["scale"], a["kv_from"]) == (6, 777.0, 3.5, seq.ROT_INTERLEAVED, 0.21, -1)
    assert (d["layers"][0]["ff"], d["layers"][0]["ff_kind"]) == (44, seq.FF_SWIGLU)
    le, ri = d["layers"][1]["branches"]
    assert (le["name"], le["heads"], le["kv_heads"], le["dim"], le["vdim"], le["qk_norm"], le["sink"], le["out_scale"], le["rot_layout"], le["rot_dims"]) == ("left", 4, 1, 12, 20, 2, 1, 0.7, seq.ROT_HALVES, 4)
    assert (ri["kind"], ri["name"], ri["heads"], ri["dim"], ri["vdim"], ri["decay"], ri["act"], ri["out_norm"], ri["gated"], ri["out_scale"], ri["scale"]) == \
        (seq.MIX_RETENTION, "right", 3, 8, 10, [0.5, 0.9, 0.99], 1, 2, 2, 1.9, 1.0)
    l1 = d["layers"][1]
    assert (l1["ff_kind"], l1["ff"], l1["experts"], l1["top"], l1["route_groups"], l1["route_keep"], l1["route_scale"], l1["shared_ff"]) == (seq.FF_GROUP_EXPERTS, 20, 9, 2, 3, 2, 2.5, 28)
    g = d["layers"][2]["branches"][0]
    assert (g["qk_norm"], g["gated"], g["maps"], g.get("chunk", 0), g.get("bias", 0), g["rot_layout"]) == (3, 3, 1, 0, 0, seq.ROT_INTERLEAVED) and d["layers"][2]["ff"] == 0
    assert d["layers"][3]["branches"][0]["kv_from"] == 0 and d["layers"][3]["branches"][0]["chunk"] == 5
    sh = VU.tensor_shapes(d)
    assert sh["l0.mix.q"] == (6 * 2 * 10, 36) and sh["l0.mix.k"] == (3 * 2 * 10, 36) and sh["l0.mix.v"] == (3 * 14, 36) and sh["l0.mix.k.b"] == (60,) and sh["l0.mix.lq2"] == (10,)
    assert sh["l0.mix.g"] == (6, 36) and sh["l1.mix.right.g"] == (30, 36) and sh["l1.mix.right.norm"] == (30,) and sh["l1.mix.left.sink"] == (4,) and sh["l1.mix.left.k.norm"] == (12,)
    assert sh["l2.mix.q.norm"] == (12,) and sh["l2.mix.k.norm"] == (12,) and sh["l1.mlp.shared.down"] == (36, 28) and sh["l1.mlp.e8.up"] == (20, 36)
    assert "l3.mix.k" not in sh and "l3.mix.v.b" not in sh and "l3.mix.q.b" in sh and "l2.norm2" not in sh and sh["l1.norm2b.b"] == (36,) and sh["final.norm.b"] == (36,)


def test_optional_sections_may_be_absent_and_bad_values_are_refused():
    cfg = VU.make_config(layers=[VU.differential_layer(rot_dims=0, chunk=0), VU.parallel_layer(rot_dims=0, mlp=VU.moe_mlp(groups=0, shared_ff=0))])
    d = VU.describe(cfg)
    a = d["layers"][0]["branches"][0]
    assert a.get("rot_dims", 0) == 0 and a.get("chunk", 0) == 0 and d["layers"][1]["route_groups"] == 1 and d["layers"][1]["route_keep"] == 1 and d["layers"][1]["shared_ff"] == 0
    assert "l1.mlp.shared.up" not in VU.tensor_shapes(d)
    for bad in (lambda c: c["layers"][0]["mixer"].__setitem__("kv_from", 0), lambda c: c["layers"][0].__setitem__("type", "attention_3"),
                lambda c: c["layers"][1]["mixer"]["right"].__setitem__("decay", [0.5]), lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3),
                lambda c: c["layers"][1]["mlp"]["router"].__setitem__("groups", {"count": 3, "keep": 1}), lambda c: c.__setitem__("architecture", "Other")):
        c2 = VU.make_config(layers=[VU.differential_layer(), VU.parallel_layer(mlp=VU.moe_mlp())])
        bad(c2)
        with pytest.raises(ValueError):
            VU.describe(c2)
    c3 = VU.make_config(layers=[VU.differential_layer(), VU.parallel_layer(), VU.differential_layer(kv_from=1)])       # a cache that is not a differential layer's
    with pytest.raises(ValueError):
        VU.describe(c3)


def test_registry_and_checkpoint_folder(tmp_path):
    cfg = VU.make_config()
    t = VU.synth_tensors(VU.describe(cfg), 1)
    VU.write_checkpoint(tmp_path / "m", cfg, t)
    assert registry.family_of(tmp_path / "m") == "Vulosun" and "Vulosun" in registry.STEPWISE
    desc, back = VU.read_checkpoint(tmp_path / "m")
    assert set(back) == set(VU.tensor_shapes(desc)) and all(np.array_equal(back[k], t[k]) for k in t)


def test_enumerators_follow_the_header():
    import re
    from pathlib import Path
    hdr = (Path(__file__).resolve().parent.parent / "include" / "gten_b200_seq.h").read_text()
    enums = dict(re.findall(r"(GTB_[A-Z0-9_]+) = (\d+)", hdr))
    for name, value in (("BLOCK_SANDWICH", seq.BLOCK_SANDWICH), ("NORM_LAYER", seq.NORM_LAYER), ("FF_SWIGLU", seq.FF_SWIGLU), ("FF_GROUP_EXPERTS", seq.FF_GROUP_EXPERTS),
                        ("MIX_RETENTION", seq.MIX_RETENTION), ("ROT_HALVES", seq.ROT_HALVES), ("ROT_INTERLEAVED", seq.ROT_INTERLEAVED)):
        assert int(enums["GTB_" + name]) == value, name
    for field in ("chunk", "maps", "diff", "bias", "act", "rot_divide"):
        assert field in [f[0] for f in seq.BranchC._fields_]
    for field in ("route_groups", "route_keep", "route_scale"):
        assert field in [f[0] for f in seq.LayerC._fields_]


def test_restatement_norms_and_rotation():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 12)) * 3 + 2
    y = R.layer_norm(x, np.ones(12), np.zeros(12), 0.0)
    assert np.allclose(y.mean(-1), 0.0) and np.allclose((y * y).mean(-1), 1.0)
    assert np.allclose(R.layer_norm(x, 2 * np.ones(12), np.full(12, 0.5), 0.0), 2 * y + 0.5)
    assert np.allclose((R.rms_norm(x, None, 0.0) ** 2).mean(-1), 1.0)
    v = rng.standard_normal((6, 2, 8))
    for inter in (True, False):
        f = R.frequencies(4, 100.0)
        r1 = R.rotate(v, np.arange(6), f, inter)
        assert np.allclose(np.linalg.norm(r1, axis=-1), np.linalg.norm(v, axis=-1)) and np.allclose(r1[..., 4:], v[..., 4:]) and np.allclose(r1[0], v[0])
        assert np.allclose(R.rotate(r1, np.arange(6), f, inter), R.rotate(v, 2 * np.arange(6), f, inter))
    r_i, r_h = R.rotate(v, np.arange(6), R.frequencies(4, 100.0), True), R.rotate(v, np.arange(6), R.frequencies(4, 100.0), False)
    assert not np.allclose(r_i, r_h)                                                      # the two layouts pair other entries
    assert np.allclose(R.rotate(v[..., [0, 2, 1, 3, 4, 5, 6, 7]], np.arange(6), R.frequencies(4, 100.0), False)[..., [0, 2, 1, 3, 4, 5, 6, 7]], r_i)
    assert np.allclose(R.frequencies(6, 50.0, 4.0) * 4.0, R.frequencies(6, 50.0)) and np.isclose(R.frequencies(6, 50.0)[1], 50.0 ** (-2 / 6))
    assert [R.first_visible(i, 4) for i in (0, 3, 4, 9)] == [0, 0, 4, 8] and R.first_visible(9, 0) == 0


def test_restatement_softmax_sink_and_recurrence():
    rng = np.random.default_rng(1)
    s = rng.standard_normal((5, 5))
    w = R.softmax_rows(s, lambda i: 0)
    assert np.allclose(w.sum(-1), 1.0) and np.allclose(np.triu(w, 1), 0.0)
    ws = R.softmax_rows(s, lambda i: 0, sink=0.3)
    assert np.isclose(ws[4].sum(), np.exp(s[4]).sum() / (np.exp(s[4]).sum() + np.exp(0.3)))
    wc = R.softmax_rows(s, lambda i: R.first_visible(i, 2))
    assert np.isclose(wc[2, 2], 1.0) and wc[3, 1] == 0.0 and wc[3, 2] > 0.0 and np.isclose(wc[4, 4], 1.0)
    # the recurrence equals the explicit sum over the past with powers of the decay
    m = {"heads": 2, "dim": 3, "vdim": 4, "decay": [0.5, 0.9]}
    T = {"q": rng.standard_normal((6, 7)), "k": rng.standard_normal((6, 7)), "v": rng.standard_normal((8, 7)), "g": rng.standard_normal((8, 7)),
         "norm": np.ones(8), "o": np.eye(8)}
    h = rng.standard_normal((9, 7))
    got = R.decayed_recurrence(h, T, m, 0.0)
    q, k, v = (R.silu(h @ T[n].T).reshape(9, 2, -1) for n in "qkv")
    raw = np.zeros((9, 2, 4))
    for t in range(9):
        for j in range(t + 1):
            for a in range(2):
                raw[t, a] += m["decay"][a] ** (t - j) * (q[t, a] @ k[j, a]) * v[j, a]
    assert np.allclose(got, R.rms_norm(raw.reshape(9, 8), None, 0.0) * R.logistic(h @ T["g"].T))
    # carried state: two halves equal the whole
    st = np.zeros((2, 3, 4))
    halves = np.concatenate([R.decayed_recurrence(h[:4], T, m, 0.0, st), R.decayed_recurrence(h[4:], T, m, 0.0, st)])
    assert np.allclose(halves, got)


def test_restatement_router_groups():
    s = np.array([0.9, 0.1, 0.5, 0.6, 0.8, 0.05, 0.3, 0.3])
    assert R.route(s, 2, 1, 1) == [0, 4]                                    # no groups: the largest scores
    # four groups of two: ranks 1.0, 1.1, 0.85, 0.6 -> groups 1 and 0 are kept, expert 4 (0.8) cannot be chosen
    assert R.route(s, 3, 4, 2) == [0, 3, 2]
    assert R.route(s, 2, 8, 3) == [0, 4] and R.route(s, 1, 8, 1) == [0]      # groups of one rank by their only score
    assert R.route(np.array([0.5, 0.5, 0.5, 0.5]), 2, 2, 1) == [0, 1]        # ties go to the lower index
    rng = np.random.default_rng(2)
    T = {"router": rng.standard_normal((4, 6)), "shared.up": rng.standard_normal((5, 6)), "shared.down": rng.standard_normal((6, 5))}
    for e in range(4):
        T[f"e{e}.up"], T[f"e{e}.down"] = rng.standard_normal((3, 6)), rng.standard_normal((6, 3))
    h = rng.standard_normal((2, 6))
    ml = {"router": {"experts": 4, "top": 4, "scale": 2.0}, "shared": {"ff": 5}}
    sc = R.logistic(h @ T["router"].T)
    want = sum(2.0 * sc[:, e:e + 1] * R.relu2_expert(h, T[f"e{e}.up"], T[f"e{e}.down"]) for e in range(4)) + R.relu2_expert(h, T["shared.up"], T["shared.down"])
    assert np.allclose(R.experts_ff(h, T, ml), want)


def test_restatement_differential_attention_reduces_to_plain_attention():
    """With lambda = 0 (diff = 0 and equal lambda vectors) the second map drops out: one softmax attention per head, unit RMS, gate."""
    rng = np.random.default_rng(3)
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "diff": 0.0, "scale": 0.5}
    Wd = 10
    T = {"q": rng.standard_normal((16, Wd)), "q.b": rng.standard_normal(16), "k": rng.standard_normal((8, Wd)), "k.b": rng.standard_normal(8), "v": rng.standard_normal((6, Wd)),
         "v.b": rng.standard_normal(6), "g": rng.standard_normal((2, Wd)), "o": np.eye(12)}
    T["lq1"] = T["lq2"] = rng.standard_normal(4)
    T["lk1"] = T["lk2"] = rng.standard_normal(4)
    assert np.isclose(R.differential_lambda(T, 0.0), 0.0) and np.isclose(R.differential_lambda(T, 0.25), 0.25)
    h = rng.standard_normal((7, Wd))
    got = R.differential_attention(h, T, m, 0.0, R.differential_keys_values(h, T, m)).reshape(7, 2, 6)
    q = (h @ T["q"].T + T["q.b"]).reshape(7, 2, 2, 4)[:, :, 0]
    k = (h @ T["k"].T + T["k.b"]).reshape(7, 1, 2, 4)[:, 0, 0]
    v = h @ T["v"].T + T["v.b"]
    for a in range(2):
        w = R.softmax_rows(q[:, a] @ k.T * 0.5, lambda i: 0)
        assert np.allclose(got[:, a], R.rms_norm(w @ v, None, 0.0) * R.logistic(h @ T["g"].T)[:, a:a + 1])
