"""`bench.py --workload reninex`: prefill and decode throughput of the Reninex family at layer sizes that resemble a real model
(random weights), beside TinyLlama at the same layer shape and layer count.  `bench.py --workload robopel`: the same for the Robopel
family, beside Reninex (the closest existing model: same library, same width and layer count).  `bench.py --workload nanotar`: the Nanotar
family beside Robopel (the closest existing model: softmax attention with a window, a sink and an output gate, routed experts) at the same
widths and layer count.  `bench.py --workload vulosun`: the Vulosun family beside Robopel (the closest existing model: sequential sublayers
with norms on their outputs, softmax attention with a sink, a gate and a shared cache, squared-ReLU experts) at the same widths and layer
count.  Timed with CUDA events on each library's own stream,
after warm-up; the weights of one pass (hundreds of MB) are larger than L2, so every pass streams them from HBM."""
from __future__ import annotations

import json
import time

import numpy as np

SIZES = {
    # name: width, ff, left (heads, kv, dim), right (heads, dim, vdim)
    "w2048": dict(width=2048, ff=5632, l_heads=32, l_kv=4, l_dim=64, l_vdim=64, r_heads=16, r_dim=128, r_vdim=128, rot_dims=64),
    "w1024": dict(width=1024, ff=2816, l_heads=16, l_kv=4, l_dim=64, l_vdim=64, r_heads=8, r_dim=128, r_vdim=128, rot_dims=64),
}


def _events(torch, stream, fn, iters, warmup):
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for a, b in ev:
            a.record(stream)
            fn()
            b.record(stream)
        torch.cuda.synchronize()
    return float(np.median([a.elapsed_time(b) for a, b in ev]))


def matmul_params(desc) -> int:
    """Weights that every token multiplies (per pass over the layer runs), head included."""
    W, n = desc["width"], 0
    runs = run_count(desc)
    for i, l in enumerate(desc["layers"]):
        per = 0
        for b in l["branches"]:
            kvh = b.get("kv_heads", b["heads"])
            per += W * (b["heads"] * b["dim"] + kvh * (b["dim"] + b["vdim"]) + (b["heads"] * b["vdim"] if b.get("gated") else 0) + b["heads"] * b["vdim"])
        per += 3 * W * l["ff"]
        n += per * runs[i]
    lp = desc.get("loop")
    if lp:
        n += lp["times"] * 2 * W * W
    return n + desc["vocab"] * W


def run_count(desc):
    lp = desc.get("loop")
    return [lp["times"] if lp and lp["start"] <= i < lp["stop"] else 1 for i in range(len(desc["layers"]))]


def mixer_flops(desc, T) -> float:
    """Sigmoid attention (causal, T keys) and retention (state update + read) FLOPs of a T-token prompt."""
    f, runs = 0.0, run_count(desc)
    for i, l in enumerate(desc["layers"]):
        for b in l["branches"]:
            if b["kind"] == 1:
                f += runs[i] * 2.0 * b["heads"] * (b["dim"] + b["vdim"]) * T * (T + 1) / 2
            else:
                f += runs[i] * 4.0 * b["heads"] * b["dim"] * b["vdim"] * T
    return f


def reninex_section(torch, name, layers, T, iters, warmup, peaks):
    from . import reninex, seq
    cfg = reninex.make_config(vocab=32000, n_layers=layers, taps=4, bigram=(65521, 31, 17), loop=None, **SIZES[name])
    desc = reninex.describe(cfg)
    t0 = time.time()
    rng = np.random.default_rng(0)
    tensors = {}
    for k, shape in reninex.tensor_shapes(desc).items():          # cheap random bf16 patterns of the right scale
        n = int(np.prod(shape)) if shape else 1
        leaf = k.split(".")[-1]
        if leaf in ("norm1", "norm"):
            a = np.full(n, 0x3F80, np.uint16)
        else:
            std = 0.3 if leaf.startswith("canon") else (1.0 if k in ("embed", "bigram") else 1.0 / np.sqrt(shape[-1]))
            a = reninex.st.f32_to_bf16_bits((rng.standard_normal(n, np.float32) * np.float32(std)))
        tensors[k] = a.reshape(shape)
    n_slots = 8
    m = seq.SeqModel(desc, seq.BF16, n_slots, T + 64, max_rows=T).load(tensors)
    stream = torch.cuda.ExternalStream(seq.stream_handle(), device=torch.device("cuda", 0))
    prompt = rng.integers(0, 32000, T).astype(np.int32)
    out = {"size": name, "layers": layers, "params_matmul": matmul_params(desc), "weight_bytes": m.weight_bytes(), "setup_s": round(time.time() - t0, 1)}

    def prefill():
        m.reset(0)
        m.step([(0, prompt)], [T - 1])
    l0 = seq.launch_count()
    prefill()
    out["prefill_launches"] = seq.launch_count() - l0
    ms = _events(torch, stream, prefill, iters, warmup)
    flops = 2.0 * T * matmul_params(desc) - 2.0 * (T - 1) * desc["vocab"] * desc["width"] + mixer_flops(desc, T)
    out["prefill"] = {"T": T, "ms": ms, "tokens_per_s": T / ms * 1e3, "tflops": flops / ms * 1e-9, "frac_of_bf16_peak": flops / ms * 1e-9 / peaks["tflops"],
                      "note": "includes the host->device copy of the prompt and the device->host copy of the last row's logits"}
    # decode at context T: 1 and 8 sequences, device-side greedy loop (CUDA-graph replay per step)
    for s in range(n_slots):
        m.reset(s)
    m.step_greedy([(s, prompt[: T - 40]) for s in range(1)])
    for s in range(1, n_slots):
        m.step_greedy([(s, prompt[: T - 40])])
    state_bytes = m.state_bytes_per_slot() * (T - 40) / (T + 64)
    for nseq in (1, 8):
        slots = list(range(nseq))
        steps = 8

        def dec():
            for s in slots:
                pass
            m.decode(slots, steps)
        # positions advance: rewind by re-prefilling is too slow, so time short bursts that stay inside max_ctx
        m.decode(slots, 2)
        t_ms = []
        with torch.cuda.stream(stream):
            for _ in range(3):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                dec()
                b.record(stream)
                torch.cuda.synchronize()
                t_ms.append(a.elapsed_time(b) / steps)
        ms = float(np.median(t_ms))
        by = m.weight_bytes() - 2 * desc["vocab"] * desc["width"] - (2 * 65522 * desc["width"]) + nseq * state_bytes
        out[f"decode_{nseq}"] = {"ms_per_step": ms, "tokens_per_s": nseq / ms * 1e3, "bytes_per_step": by, "gbs": by / ms * 1e-6,
                                 "frac_of_hbm_peak": by / ms * 1e-6 / peaks["hbm_gbs"]}
    m.close()
    return out


ROBOPEL_SIZES = {
    # width, dense ff, minGRU width, attention (heads, kv, dim), window, pool, experts x ff (top of experts + identity)
    "w2048": dict(width=2048, ff=5632, gru=2048, heads=32, kv=4, dim=64, window=1024, pool=16, experts=16, identity=2, top=2, eff=1408),
    "w1024": dict(width=1024, ff=2816, gru=1024, heads=16, kv=4, dim=64, window=512, pool=8, experts=16, identity=2, top=2, eff=704),
}


def robopel_config(name, vocab=32000):
    """Four layers in the family's usual order: minGRU + dense, attention + experts, minGRU + experts, attention on layer 1's cache + dense."""
    from . import robopel as RP
    z = ROBOPEL_SIZES[name]
    att = dict(heads=z["heads"], kv_heads=z["kv"], dim=z["dim"], vdim=z["dim"], window=z["window"], pool=z["pool"], rot_dims=z["dim"], rot_base=500000.0,
               scaling=(8.0, 1.0, 4.0, 8192), softcap=30.0)
    moe = lambda: RP.moe_mlp(experts=z["experts"], identity=z["identity"], top=z["top"], ff=z["eff"])
    layers = [RP.mingru_layer(z["gru"], mlp=RP.dense_mlp(z["ff"])), RP.attention_layer(mlp=moe(), **att), RP.mingru_layer(z["gru"], mlp=moe()),
              RP.attention_layer(kv_from=1, mlp=RP.dense_mlp(z["ff"]), **att)]
    return RP.make_config(vocab=vocab, width=z["width"], layers=layers, embed_scale=float(z["width"]) ** 0.5, eps=1e-6)


def robopel_counts(desc, T):
    """(weights every token multiplies, FLOPs of the mixers' own arithmetic for a T-token prompt, bytes of weights a decode step of one
    sequence reads) -- routed experts count `top` experts per token."""
    from .seq import FF_EXPERTS, MIX_MINGRU
    W, params, mix, dec = desc["width"], 0, 0.0, 0
    for l in desc["layers"]:
        b = l["branches"][0]
        if b["kind"] == MIX_MINGRU:
            per = 4 * W * b["dim"]
            mix += 10.0 * b["dim"] * T
        else:
            hv = b["heads"] * b["vdim"]
            per = W * (b["heads"] * b["dim"] + 2 * hv) + (W * b["kv_heads"] * (b["dim"] + b["vdim"]) if b["kv_from"] < 0 else 0)
            win, pool = b.get("window", 0), b.get("pool", 0)
            keys = sum(min(i + 1, win) + ((i - win + 1) // pool if pool and i - win + 1 >= pool else 0) for i in range(T)) if win else T * (T + 1) / 2
            mix += 2.0 * b["heads"] * (b["dim"] + b["vdim"]) * keys
        if l["ff"]:
            per += (W * (l["experts"] + l["identity"]) + l["top"] * 2 * W * l["ff"]) if l.get("ff_kind") == FF_EXPERTS else 2 * W * l["ff"]
        params += per
    return params + desc["vocab"] * W, mix, 2 * (params + desc["vocab"] * W)


def robopel_section(torch, name, T, iters, warmup, peaks):
    from . import robopel as RP, seq
    cfg = robopel_config(name)
    desc = RP.describe(cfg)
    t0 = time.time()
    rng = np.random.default_rng(0)
    tensors = {}
    for k, shape in RP.tensor_shapes(desc).items():              # cheap random bf16 patterns of the right scale
        n = int(np.prod(shape))
        leaf = k.split(".")[-1]
        if leaf in ("norm1", "norm2") or k == "final.norm" or leaf in ("correction", "b"):
            a = np.zeros(n, np.uint16)
        elif k.endswith("q.norm") or k.endswith("k.norm"):
            a = np.full(n, 0x3F80, np.uint16)
        elif leaf == "act":
            a = RP.st.f32_to_bf16_bits(np.array([0.6, 0.3, 0.2, 0.05], np.float32))
        else:
            std = 1.0 / desc["embed_scale"] if k == "embed" else (1.0 if leaf == "sink" else 1.0 / np.sqrt(shape[-1]))
            a = RP.st.f32_to_bf16_bits(rng.standard_normal(n, np.float32) * np.float32(std))
        tensors[k] = a.reshape(shape)
    n_slots = 8
    m = seq.SeqModel(desc, seq.BF16, n_slots, T + 64, max_rows=T).load(tensors)
    stream = torch.cuda.ExternalStream(seq.stream_handle(), device=torch.device("cuda", 0))
    prompt = rng.integers(0, desc["vocab"], T).astype(np.int32)
    params, mix, dec_bytes = robopel_counts(desc, T)
    out = {"size": name, "layers": len(desc["layers"]), "params_matmul_per_token": params, "weight_bytes": m.weight_bytes(), "setup_s": round(time.time() - t0, 1)}

    def prefill():
        m.reset(0)
        m.step([(0, prompt)], [T - 1])
    l0 = seq.launch_count()
    prefill()
    out["prefill_launches"] = seq.launch_count() - l0
    ms = _events(torch, stream, prefill, iters, warmup)
    flops = 2.0 * T * params - 2.0 * (T - 1) * desc["vocab"] * desc["width"] + mix
    out["prefill"] = {"T": T, "ms": ms, "tokens_per_s": T / ms * 1e3, "tflops": flops / ms * 1e-9, "frac_of_bf16_peak": flops / ms * 1e-9 / peaks["tflops"],
                      "note": "includes the host->device copy of the prompt and the device->host copy of the last row's logits; experts count top per token"}
    for s in range(n_slots):
        m.reset(s)
        m.step_greedy([(s, prompt[: T - 40])])
    state_bytes = m.state_bytes_per_slot() * (T - 40) / (T + 64)
    for nseq in (1, 8):
        slots, steps = list(range(nseq)), 8
        m.decode(slots, 2)
        t_ms = []
        with torch.cuda.stream(stream):
            for _ in range(3):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                m.decode(slots, steps)
                b.record(stream)
                torch.cuda.synchronize()
                t_ms.append(a.elapsed_time(b) / steps)
        ms = float(np.median(t_ms))
        by = dec_bytes                                             # layers (top experts per routed layer) + head; the embedding is one row per sequence
        out[f"decode_{nseq}"] = {"ms_per_step": ms, "tokens_per_s": nseq / ms * 1e3, "bytes_per_step_one_sequence": by, "gbs": by / ms * 1e-6,
                                 "frac_of_hbm_peak": by / ms * 1e-6 / peaks["hbm_gbs"],
                                 "note": "bytes: weights one sequence's step reads (top experts per routed layer); further sequences add their experts and state"}
    out["state_bytes_per_slot_at_T"] = state_bytes
    m.close()
    return out


NANOTAR_SIZES = {
    # width, dense ff, heads x (plain + rotated | value), latent ranks, window of the second form, experts x ff (top) + shared ff, stream copies
    "w2048": dict(width=2048, ff=5632, heads=16, dim=96, rot=32, vdim=128, kv_rank=512, q_rank=768, window=1024, experts=16, top=2, eff=1408, sff=1408, streams=2),
    "w1024": dict(width=1024, ff=2816, heads=8, dim=96, rot=32, vdim=128, kv_rank=256, q_rank=384, window=512, experts=16, top=2, eff=704, sff=704, streams=2),
}


def nanotar_config(name, vocab=32000):
    """Four layers: causal latent attention + dense, windowed form (query latent, sink) + experts, causal + experts, windowed + dense."""
    from . import nanotar as NT
    z = NANOTAR_SIZES[name]
    att = dict(heads=z["heads"], dim=z["dim"], rot_dim=z["rot"], vdim=z["vdim"], kv_rank=z["kv_rank"], rot_base=500000.0)
    moe = lambda: NT.moe_mlp(experts=z["experts"], top=z["top"], ff=z["eff"], shared_ff=z["sff"])
    layers = [NT.latent_layer(mlp=NT.dense_mlp(z["ff"]), **att), NT.latent_layer(q_rank=z["q_rank"], window=z["window"], mlp=moe(), **att),
              NT.latent_layer(mlp=moe(), **att), NT.latent_layer(q_rank=z["q_rank"], window=z["window"], mlp=NT.dense_mlp(z["ff"]), **att)]
    return NT.make_config(vocab=vocab, width=z["width"], streams=z["streams"], layers=layers, eps=1e-6, logit_softcap=30.0)


def nanotar_counts(desc, T):
    """(weights every token multiplies, FLOPs of the attention's own arithmetic for a T-token prompt, bytes of weights a decode step of one
    sequence reads) -- routed experts count `top` experts per token; keys and values count one up-projection per token."""
    from .seq import FF_GATED_EXPERTS
    W, params, mix = desc["width"], 0, 0.0
    for l in desc["layers"]:
        b = l["branches"][0]
        H, hd = b["heads"], b["dim"] + b["rope_dim"]
        per = W * ((b["q_rank"] or H * hd) + b["kv_rank"] + b["rope_dim"] + H) + b["q_rank"] * H * hd + b["kv_rank"] * H * (b["dim"] + b["vdim"]) + W * H * b["vdim"]
        win = b.get("window", 0)
        keys = sum(min(i + 1, win) for i in range(T)) if win else T * (T + 1) / 2
        mix += 2.0 * H * (hd + b["vdim"]) * keys
        if l["ff"]:
            per += (W * (l["experts"] + 1) + l["top"] * 3 * W * l["ff"] + 3 * W * l.get("shared_ff", 0)) if l.get("ff_kind") == FF_GATED_EXPERTS else 3 * W * l["ff"]
        params += per
    return params + desc["vocab"] * W, mix, 2 * (params + desc["vocab"] * W)


def nanotar_section(torch, name, T, iters, warmup, peaks):
    from . import nanotar as NT, seq
    cfg = nanotar_config(name)
    desc = NT.describe(cfg)
    t0 = time.time()
    rng = np.random.default_rng(0)
    S, tensors = desc["streams"], {}
    for k, shape in NT.tensor_shapes(desc).items():              # cheap random bf16 patterns of the right scale
        n = int(np.prod(shape)) if shape else 1
        parts = ("." + k).split(".")
        leaf = parts[-1]
        if leaf == "alpha":
            a = NT.st.f32_to_bf16_bits(np.full(n, 0.5, np.float32))
        elif leaf == "b" and "norm" in parts[-2]:
            a = np.zeros(n, np.uint16)
        elif leaf in ("norm1", "norm2", "norm"):
            a = np.full(n, 0x3F80, np.uint16)
        elif parts[-2].startswith("hc"):
            a = NT.st.f32_to_bf16_bits({"in": np.full(shape, 1.0 / S), "out": np.ones(shape), "mix": np.eye(S)}[leaf].astype(np.float32).reshape(-1))
        else:
            std = 1.0 if k == "embed" or leaf == "sink" else 1.0 / np.sqrt(shape[-1])
            a = NT.st.f32_to_bf16_bits(rng.standard_normal(n, np.float32) * np.float32(std))
        tensors[k] = a.reshape(shape)
    n_slots = 8
    m = seq.SeqModel(desc, seq.BF16, n_slots, T + 64, max_rows=T).load(tensors)
    stream = torch.cuda.ExternalStream(seq.stream_handle(), device=torch.device("cuda", 0))
    prompt = rng.integers(0, desc["vocab"], T).astype(np.int32)
    params, mix, dec_bytes = nanotar_counts(desc, T)
    out = {"size": name, "layers": len(desc["layers"]), "params_matmul_per_token": params, "weight_bytes": m.weight_bytes(), "setup_s": round(time.time() - t0, 1)}

    def prefill():
        m.reset(0)
        m.step([(0, prompt)], [T - 1])
    l0 = seq.launch_count()
    prefill()
    out["prefill_launches"] = seq.launch_count() - l0
    ms = _events(torch, stream, prefill, iters, warmup)
    flops = 2.0 * T * params - 2.0 * (T - 1) * desc["vocab"] * desc["width"] + mix
    out["prefill"] = {"T": T, "ms": ms, "tokens_per_s": T / ms * 1e3, "tflops": flops / ms * 1e-9, "frac_of_bf16_peak": flops / ms * 1e-9 / peaks["tflops"],
                      "note": "includes the host->device copy of the prompt and the device->host copy of the last row's logits; experts count top per token"}

    def chunked():                                                # the same prompt in four portions: every portion expands the latents before it again
        m.reset(0)
        for i in range(0, T, T // 4):
            m.step([(0, prompt[i:i + T // 4])], [T // 4 - 1])
    out["prefill_in_4_portions_ms"] = _events(torch, stream, chunked, max(3, iters // 2), 2)
    for s in range(n_slots):
        m.reset(s)
        m.step_greedy([(s, prompt[: T - 40])])
    state_bytes = m.state_bytes_per_slot() * (T - 40) / (T + 64)
    for nseq in (1, 8):
        slots, steps = list(range(nseq)), 8
        m.decode(slots, 2)
        t_ms = []
        with torch.cuda.stream(stream):
            for _ in range(3):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                m.decode(slots, steps)
                b.record(stream)
                torch.cuda.synchronize()
                t_ms.append(a.elapsed_time(b) / steps)
        ms = float(np.median(t_ms))
        by = dec_bytes
        out[f"decode_{nseq}"] = {"ms_per_step": ms, "tokens_per_s": nseq / ms * 1e3, "bytes_per_step_one_sequence": by, "gbs": by / ms * 1e-6,
                                 "frac_of_hbm_peak": by / ms * 1e-6 / peaks["hbm_gbs"],
                                 "note": "bytes: weights one sequence's step reads (top experts per routed layer); further sequences add their experts and cached latents"}
    out["state_bytes_per_slot_at_T"] = state_bytes
    m.close()
    return out


VULOSUN_SIZES = {
    # width, dense ff; gated attention heads / kv x dim | vdim; differential heads / kv x (2 x dim) | vdim and its chunk; parallel: left heads / kv x dim | vdim,
    # right heads x dim | vdim; experts x ff (top, groups, kept) + shared ff
    "w2048": dict(width=2048, ff=5632, heads=32, kv=4, dim=64, vdim=64, d_heads=16, d_kv=4, d_dim=64, d_vdim=128, chunk=1024, l_heads=16, l_kv=4, l_dim=64, l_vdim=64,
                  r_heads=8, r_dim=128, r_vdim=128, experts=16, top=2, groups=4, keep=2, eff=1408, sff=1408),
    "w1024": dict(width=1024, ff=2816, heads=16, kv=4, dim=64, vdim=64, d_heads=8, d_kv=4, d_dim=64, d_vdim=128, chunk=512, l_heads=8, l_kv=4, l_dim=64, l_vdim=64,
                  r_heads=4, r_dim=128, r_vdim=128, experts=16, top=2, groups=4, keep=2, eff=704, sff=704),
}


def vulosun_config(name, vocab=32000):
    """Four layers: differential attention + dense, parallel (sink attention | decayed recurrence) + experts, gated attention + experts,
    differential attention on layer 0's cache + dense."""
    from . import vulosun as VU
    z = VULOSUN_SIZES[name]
    dif = dict(heads=z["d_heads"], kv_heads=z["d_kv"], dim=z["d_dim"], vdim=z["d_vdim"], diff=0.5, chunk=z["chunk"], rot_dims=32, rot_base=10000.0, factor=8.0)
    moe = lambda: VU.moe_mlp(experts=z["experts"], top=z["top"], ff=z["eff"], groups=z["groups"], keep=z["keep"], scale=2.0, shared_ff=z["sff"])
    layers = [VU.differential_layer(mlp=VU.dense_mlp(z["ff"]), **dif),
              VU.parallel_layer(heads=z["l_heads"], kv_heads=z["l_kv"], dim=z["l_dim"], vdim=z["l_vdim"], rot_dims=32, rot_base=100000.0, r_heads=z["r_heads"], r_dim=z["r_dim"],
                                r_vdim=z["r_vdim"], decay=[float(1.0 - 2.0 ** (-3 - h)) for h in range(z["r_heads"])], left_scale=1.0, right_scale=0.8, mlp=moe()),
              VU.gated_attention_layer(heads=z["heads"], kv_heads=z["kv"], dim=z["dim"], vdim=z["vdim"], rot_dims=z["dim"], rot_base=250000.0, mlp=moe()),
              VU.differential_layer(kv_from=0, mlp=VU.dense_mlp(z["ff"]), **dif)]
    return VU.make_config(vocab=vocab, width=z["width"], layers=layers, eps=1e-6)


def vulosun_counts(desc, T):
    """(weights every token multiplies, FLOPs of the mixers' own arithmetic for a T-token prompt, bytes of weights a decode step of one
    sequence reads) -- routed experts count `top` experts per token, attention the keys a row really sees."""
    from .seq import FF_GROUP_EXPERTS, MIX_RETENTION
    W, params, mix = desc["width"], 0, 0.0
    for l in desc["layers"]:
        per = 0
        for b in l["branches"]:
            H, D, V = b["heads"], b["dim"], b["vdim"]
            if b["kind"] == MIX_RETENTION:
                per += W * (2 * H * D + 3 * H * V)
                mix += 4.0 * H * D * V * T                        # state update and read per token
                continue
            M, G = b.get("maps", 1), b["kv_heads"]
            per += W * (H * M * D + H * V) + (W * G * (M * D + V) if b.get("kv_from", -1) < 0 else 0) + (W * H if b.get("gated") == 3 else 0)
            ch = b.get("chunk", 0)
            keys = sum(i % ch + 1 for i in range(T)) if ch else T * (T + 1) / 2
            mix += 2.0 * H * M * (D + V) * keys
        if l["ff"]:
            per += (W * l["experts"] + l["top"] * 2 * W * l["ff"] + 2 * W * l.get("shared_ff", 0)) if l.get("ff_kind") == FF_GROUP_EXPERTS else 3 * W * l["ff"]
        params += per
    return params + desc["vocab"] * W, mix, 2 * (params + desc["vocab"] * W)


def vulosun_section(torch, name, T, iters, warmup, peaks):
    from . import vulosun as VU, seq
    cfg = vulosun_config(name)
    desc = VU.describe(cfg)
    t0 = time.time()
    rng = np.random.default_rng(0)
    tensors = {}
    for k, shape in VU.tensor_shapes(desc).items():              # cheap random bf16 patterns of the right scale
        n = int(np.prod(shape))
        leaf = k.split(".")[-1]
        if leaf == "b":
            a = np.zeros(n, np.uint16)
        elif leaf.startswith("norm"):
            a = np.full(n, 0x3F80, np.uint16)
        else:
            std = 1.0 if k == "embed" or leaf == "sink" else (0.1 if leaf in ("lq1", "lk1", "lq2", "lk2") else 1.0 / np.sqrt(shape[-1]))
            a = VU.st.f32_to_bf16_bits(rng.standard_normal(n, np.float32) * np.float32(std))
        tensors[k] = a.reshape(shape)
    n_slots = 8
    m = seq.SeqModel(desc, seq.BF16, n_slots, T + 64, max_rows=T).load(tensors)
    stream = torch.cuda.ExternalStream(seq.stream_handle(), device=torch.device("cuda", 0))
    prompt = rng.integers(0, desc["vocab"], T).astype(np.int32)
    params, mix, dec_bytes = vulosun_counts(desc, T)
    out = {"size": name, "layers": len(desc["layers"]), "params_matmul_per_token": params, "weight_bytes": m.weight_bytes(), "setup_s": round(time.time() - t0, 1)}

    def prefill():
        m.reset(0)
        m.step([(0, prompt)], [T - 1])
    l0 = seq.launch_count()
    prefill()
    out["prefill_launches"] = seq.launch_count() - l0
    ms = _events(torch, stream, prefill, iters, warmup)
    flops = 2.0 * T * params - 2.0 * (T - 1) * desc["vocab"] * desc["width"] + mix
    out["prefill"] = {"T": T, "ms": ms, "tokens_per_s": T / ms * 1e3, "tflops": flops / ms * 1e-9, "frac_of_bf16_peak": flops / ms * 1e-9 / peaks["tflops"],
                      "note": "includes the host->device copy of the prompt and the device->host copy of the last row's logits; experts count top per token"}

    def chunked():                                                # the same prompt in four portions
        m.reset(0)
        for i in range(0, T, T // 4):
            m.step([(0, prompt[i:i + T // 4])], [T // 4 - 1])
    out["prefill_in_4_portions_ms"] = _events(torch, stream, chunked, max(3, iters // 2), 2)
    for s in range(n_slots):
        m.reset(s)
        m.step_greedy([(s, prompt[: T - 40])])
    state_bytes = m.state_bytes_per_slot() * (T - 40) / (T + 64)
    for nseq in (1, 8):
        slots, steps = list(range(nseq)), 8
        m.decode(slots, 2)
        l0 = seq.launch_count()
        t_ms = []
        with torch.cuda.stream(stream):
            for _ in range(3):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                m.decode(slots, steps)
                b.record(stream)
                torch.cuda.synchronize()
                t_ms.append(a.elapsed_time(b) / steps)
        ms = float(np.median(t_ms))
        by = dec_bytes
        out[f"decode_{nseq}"] = {"ms_per_step": ms, "tokens_per_s": nseq / ms * 1e3, "bytes_per_step_one_sequence": by, "gbs": by / ms * 1e-6,
                                 "frac_of_hbm_peak": by / ms * 1e-6 / peaks["hbm_gbs"],
                                 "note": "bytes: weights one sequence's step reads (top experts per routed layer); further sequences add their experts, keys and state"}
    out["state_bytes_per_slot_at_T"] = state_bytes
    m.close()
    return out


def run_vulosun(args, root, clock_sampler) -> None:
    """`--workload vulosun`: Vulosun at two sizes, Robopel at the same widths and layer count in the same call."""
    import torch
    from . import build, seq
    build.build(target="seq")
    torch.cuda.set_device(0)
    peaks = _peaks(root)
    seq.init(0)
    T = 2048
    iters = max(3, min(args.steps if args.steps != 512 else 5, 20))
    warm = max(args.warmup if args.warmup != 16 else 3, 3)
    res = {"vulosun": [], "robopel_same_width": [], "peaks": peaks}
    only = getattr(args, "sizes", None)
    with clock_sampler(0) as clk:
        for name in VULOSUN_SIZES:
            if not only or name in only:
                res["vulosun"].append(vulosun_section(torch, name, T, iters, warm, peaks))
        for name in ROBOPEL_SIZES:
            if not only or name in only:
                res["robopel_same_width"].append(robopel_section(torch, name, T, iters, warm, peaks))
    head = res["vulosun"][0]
    print(json.dumps({"metric": "vulosun_prefill_tokens_per_s", "value": head["prefill"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
                      "steps": iters, "warmup": warm, "ms_per_step": head["prefill"]["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "bf16 operands, fp32 accumulation; fp32 stream, norms, scores, recurrent state, router", "data": "synthetic",
                      "config": {"workload": f"Vulosun {head['size']} x {head['layers']} layers, random weights: prefill of {T} tokens; decode at that context",
                                 "l2": "weights of a pass exceed L2"},
                      "detail": res, "gpu_launches": head["prefill_launches"], "clocks": clk.summary()}), flush=True)


def _peaks(root):
    p = root / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d.get("bf16_tflops", 1590.0)), "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}


def run_nanotar(args, root, clock_sampler) -> None:
    """`--workload nanotar`: Nanotar at two sizes, Robopel at the same widths and layer count in the same call."""
    import torch
    from . import build, seq
    build.build(target="seq")
    torch.cuda.set_device(0)
    peaks = _peaks(root)
    seq.init(0)
    T = 2048
    iters = max(3, min(args.steps if args.steps != 512 else 5, 20))
    warm = max(args.warmup if args.warmup != 16 else 3, 3)
    res = {"nanotar": [], "robopel_same_width": [], "peaks": peaks}
    with clock_sampler(0) as clk:
        for name in NANOTAR_SIZES:
            res["nanotar"].append(nanotar_section(torch, name, T, iters, warm, peaks))
        for name in ROBOPEL_SIZES:
            res["robopel_same_width"].append(robopel_section(torch, name, T, iters, warm, peaks))
    head = res["nanotar"][0]
    print(json.dumps({"metric": "nanotar_prefill_tokens_per_s", "value": head["prefill"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
                      "steps": iters, "warmup": warm, "ms_per_step": head["prefill"]["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "bf16 operands, fp32 accumulation; fp32 stream copies, norms, scores, router", "data": "synthetic",
                      "config": {"workload": f"Nanotar {head['size']} x {head['layers']} layers, random weights: prefill of {T} tokens; decode at that context",
                                 "l2": "weights of a pass exceed L2"},
                      "detail": res, "gpu_launches": head["prefill_launches"], "clocks": clk.summary()}), flush=True)


def tinyllama_section(torch, layers, T, iters, warmup, peaks):
    """The closest existing model at the same layer shape (width 2048, ff 5632) and layer count: FP16 weights."""
    from . import capi, weights as W
    capi.init(0)
    cfg = W.mini_config(n_layers=layers, n_vocab=32000)
    stream = torch.cuda.ExternalStream(capi.stream_handle(), device=torch.device("cuda", 0))
    out = {"layers": layers}
    for wname, wdt in (("fp16", W.F16), ("q8", W.Q8)):
        eng = capi.Engine(cfg, T + 64, wdt).load(W.synth_weights(cfg, wdt, seed=1))
        prompt = W.synth_prompt(7, T, cfg.n_vocab)
        per_layer = 2 * cfg.n_embd * cfg.n_embd + 2 * cfg.kv_dim * cfg.n_embd + 3 * cfg.n_ffn * cfg.n_embd
        flops = 2.0 * T * layers * per_layer + 2.0 * cfg.n_vocab * cfg.n_embd + layers * 2.0 * cfg.n_heads * 2 * cfg.d_head * T * (T + 1) / 2
        ms = _events(torch, stream, lambda: eng.prefill_fast(prompt), iters, warmup)
        out[f"prefill_{wname}"] = {"T": T, "ms": ms, "tokens_per_s": T / ms * 1e3, "tflops": flops / ms * 1e-9,
                                   "frac_of_bf16_peak": flops / ms * 1e-9 / peaks["tflops"], "path": "gtb_engine_prefill_fast (tcgen05 GEMMs, mma.sync attention)"}
        eng.prefill_fast(prompt[: T - 40])
        steps = 8
        t_ms = []
        with torch.cuda.stream(stream):
            eng.decode(2)
            for _ in range(3):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                eng.decode(steps)
                b.record(stream)
                torch.cuda.synchronize()
                t_ms.append(a.elapsed_time(b) / steps)
        ms = float(np.median(t_ms))
        by = cfg.decode_bytes(wdt, T - 30)
        out[f"decode_{wname}"] = {"ms_per_step": ms, "tokens_per_s": 1e3 / ms, "bytes_per_step": by, "gbs": by / ms * 1e-6,
                                  "frac_of_hbm_peak": by / ms * 1e-6 / peaks["hbm_gbs"], "path": "persistent exact kernel" if eng.uses_megakernel() else "one kernel per phase"}
        if wdt == W.Q8:
            eng.set_option("fast_decode", 1)
            t_ms = []
            with torch.cuda.stream(stream):
                eng.decode(2)
                for _ in range(3):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                    eng.decode(steps)
                    b.record(stream)
                    torch.cuda.synchronize()
                    t_ms.append(a.elapsed_time(b) / steps)
            ms = float(np.median(t_ms))
            out["decode_q8_order_free"] = {"ms_per_step": ms, "tokens_per_s": 1e3 / ms, "gbs": by / ms * 1e-6, "frac_of_hbm_peak": by / ms * 1e-6 / peaks["hbm_gbs"]}
        eng.close()
    return out


def run_robopel(args, root, clock_sampler) -> None:
    """`--workload robopel`: Robopel at two sizes, Reninex at the same widths and layer count in the same call."""
    import torch
    from . import build, seq
    build.build(target="seq")
    torch.cuda.set_device(0)
    p = root / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        peaks = {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d.get("bf16_tflops", 1590.0)), "source": "measured (MEASURED_PEAKS.json)"}
    else:
        peaks = {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}
    seq.init(0)
    T = 2048
    iters = max(3, min(args.steps if args.steps != 512 else 5, 20))
    warm = max(args.warmup if args.warmup != 16 else 3, 3)
    res = {"robopel": [], "reninex_same_width": [], "peaks": peaks}
    with clock_sampler(0) as clk:
        for name in ROBOPEL_SIZES:
            res["robopel"].append(robopel_section(torch, name, T, iters, warm, peaks))
        for name in SIZES:
            res["reninex_same_width"].append(reninex_section(torch, name, 4, T, iters, warm, peaks))
    head = res["robopel"][0]
    print(json.dumps({"metric": "robopel_prefill_tokens_per_s", "value": head["prefill"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
                      "steps": iters, "warmup": warm, "ms_per_step": head["prefill"]["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "bf16 operands, fp32 accumulation; fp32 stream, scores, state", "data": "synthetic",
                      "config": {"workload": f"Robopel {head['size']} x {head['layers']} layers, random weights: prefill of {T} tokens; decode at that context",
                                 "l2": "weights of a pass exceed L2"},
                      "detail": res, "gpu_launches": head["prefill_launches"], "clocks": clk.summary()}), flush=True)


def run(args, root, clock_sampler) -> None:
    import torch
    from . import build
    build.build(target="seq")
    torch.cuda.set_device(0)
    p = root / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        peaks = {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d.get("bf16_tflops", 1590.0)), "source": "measured (MEASURED_PEAKS.json)"}
    else:
        peaks = {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}
    from . import seq
    seq.init(0)
    layers, T = 4, 2048
    iters = max(3, min(args.steps if args.steps != 512 else 5, 20))
    res = {"reninex": [], "peaks": peaks}
    with clock_sampler(0) as clk:
        for name in SIZES:
            res["reninex"].append(reninex_section(torch, name, layers, T, iters, max(args.warmup if args.warmup != 16 else 3, 3), peaks))
        try:
            res["tinyllama_same_shape"] = tinyllama_section(torch, layers, T, iters, 3, peaks)
        except Exception as e:            # the TinyLlama library is a separate build target
            res["tinyllama_same_shape"] = {"unavailable": f"{type(e).__name__}: {e}"}
    head = res["reninex"][0]
    print(json.dumps({"metric": "reninex_prefill_tokens_per_s", "value": head["prefill"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
                      "steps": iters, "warmup": 3, "ms_per_step": head["prefill"]["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "bf16 operands, fp32 accumulation; fp32 stream, scores, state", "data": "synthetic",
                      "config": {"workload": f"Reninex {head['size']} x {layers} layers, random weights: prefill of {T} tokens; decode at that context",
                                 "l2": "weights of a pass exceed L2"},
                      "detail": res, "gpu_launches": head["prefill_launches"], "clocks": clk.summary()}), flush=True)
