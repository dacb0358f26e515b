"""Batched (tcgen05) prefill against the CPU checker.

The batched path sums each dot product in a different order than ops.h:224-391 and feeds the tensor cores fp16
operands (dequantised Q8/Q4 values rounded to 11 bits; FP16 models: the fp16 values themselves), so parity here is a
STATED TOLERANCE, not bit equality:

* the tcgen05 GEMM itself is exact on integer-valued inputs (every product and partial sum is representable);
* the yardstick for everything else is the reference ITSELF: its two documented builds (README.md:18 scalar,
  README.md:25 AVX) associate the same sums differently and, because every op re-encodes its output as Q8 blocks, end
  up a few percent apart after a few layers (tests/golden/order_sensitivity.npz, generated from the unmodified sources
  by tests/golden/make_order_sensitivity.py).  The batched path's licence to differ from the AVX build is the same
  one -- summation order -- so its distance to the AVX build must stay within SLACK x the scalar build's distance,
  per layer (worst activation row, relative L2) and for the logits of the last prompt row (+ a small floor, ABS);
* the K/V cache written by the batched path feeds the order-exact decode path: logits of the NEXT row, computed by
  the exact kernels on top of that cache, stay within the same bound (catches any cache-layout mistake).

The exact path (gtb_engine_prefill / gtb_engine_logits) remains the bit-checked one (tests/test_gpu_parity.py).
"""
from pathlib import Path

import numpy as np
import pytest

import oracle
from oracle import F16, Q4, Q8
from tinyllama_cpp_b200 import weights as W

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"

SLACK = 2.0           # x the reference's own scalar-vs-AVX distance
ABS = 5e-3            # floor (a layer where the two reference builds happen to agree almost exactly), never more than half the spread
SENS = np.load(GOLD / "order_sensitivity.npz")


@pytest.fixture(scope="module")
def capi():
    from tinyllama_cpp_b200 import capi
    capi.init(0)
    return capi


def rel(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("bn", [128, 256, 512])        # 512 = the CTA-pair kernel (256 x 256 tiles, tcgen05 cta_group::2)
@pytest.mark.parametrize("shape", [(128, 256, 64), (1, 256, 128), (200, 2560, 2048), (333, 2048, 5632), (2048, 512, 2048)])
def test_tcgen05_gemm_exact_on_integers(capi, shape, bn):
    """Small integers: every product and every partial sum is exact in fp32, so any summation order gives the same bits."""
    m, n, k = shape
    rng = np.random.default_rng(m * 31 + n + k + bn)
    a = rng.integers(-3, 4, (m, k)).astype(np.float16)
    w = rng.integers(-3, 4, (n, k)).astype(np.float16)
    got = capi.pf_gemm_f32(a, w, bn)
    want = a.astype(np.float32) @ w.astype(np.float32).T
    assert np.array_equal(got, want), (shape, bn, np.abs(got - want).max())


def test_tcgen05_gemm_random(capi):
    rng = np.random.default_rng(3)
    m, n, k = 300, 1024, 2048
    a = rng.standard_normal((m, k)).astype(np.float16)
    w = (0.02 * rng.standard_normal((n, k))).astype(np.float16)
    got = capi.pf_gemm_f32(a, w, 256)
    want = a.astype(np.float64) @ w.astype(np.float64).T
    assert rel(got, want) < 1e-5        # measured 2.5e-6: the tensor-core accumulator keeps fewer guard bits than an fp32 FMA chain


@pytest.mark.parametrize("wdt", [Q8, Q4, F16])
@pytest.mark.parametrize("n_prompt", [100, 64, 7])
def test_batched_prefill_mini(capi, checker, wdt, n_prompt):
    _mini_case(capi, checker, wdt, n_prompt, {})


@pytest.mark.parametrize("opts", [{"pf_attn2": 1}, {"pf_2cta": 1}, {"pf_pdl": 0, "pf_fused": 0}], ids=["two-sweep-attn", "cta-pairs", "unfused-no-pdl"])
def test_batched_prefill_variants(capi, checker, opts):
    """The optional code paths meet the same bound: two-sweep attention (also reproduces the fp16 rounding of the block
    scales of the probability rows; the default online-softmax sweep applies them unrounded), the CTA-pair GEMM kernel,
    and the unfused epilogues without programmatic dependent launch."""
    _mini_case(capi, checker, Q8, 100, opts)


def _mini_case(capi, checker, wdt, n_prompt, opts):
    cfg = W.mini_config(n_layers=3, n_vocab=300)
    wl = list(W.synth_weights(cfg, wdt, seed=21))
    max_ctx = 192
    cm = checker.model(cfg, max_ctx if wdt != F16 else 2 * max_ctx, wdt).load(wl)     # FP16 P rows: 2 n <= max_ctx
    e = capi.Engine(cfg, max_ctx, wdt).load(wl)
    for k, v in opts.items():
        e.set_option(k, v)
    prompt = W.synth_prompt(5, n_prompt, cfg.n_vocab)
    want_logits = cm.logits(prompt, 0)
    e.set_option("capture_acv", 1)
    e.prefill_fast(prompt)
    got_logits = e.read_logits()
    rows = sorted({0, 1, n_prompt // 2, n_prompt - 2, n_prompt - 1} & set(range(n_prompt)))
    worst = {}
    for row in rows:
        if cm.lib.prefix == "orc_":           # the plain-C port keeps the activations of one row per forward pass
            cm.capture_row(row)
            cm.logits(prompt, 0)
        for layer in range(cfg.n_layers):
            for name, aid in oracle.LAYER_ACVS.items():
                if name == "attn_res" and layer == cfg.n_layers - 1:
                    continue                      # the last residual add belongs to the exact final-norm phase
                err = rel(e.pf_acv(layer, aid, row), cm.acv(layer, aid, row))
                worst[(layer, name)] = max(worst.get((layer, name), 0.0), err)
        assert np.array_equal(e.pf_acv(0, oracle.A_EMB, row), cm.acv(0, oracle.A_EMB, row))     # the embedding gather is exact
    wn = {Q8: "q8", Q4: "q4", F16: "f16"}[wdt]
    sens_acv = SENS[f"mini_{wn}_{n_prompt}_acv"].max(axis=1)          # the reference's own spread, worst activation per layer
    sens_logits = float(SENS[f"mini_{wn}_{n_prompt}_logits"])
    ours = [max(v for (l, _), v in worst.items() if l == layer) for layer in range(cfg.n_layers)]
    lerr = rel(got_logits, want_logits)
    print(f"\nwdt={wn} T={n_prompt} {opts}: logits rel {lerr:.2e} (reference scalar-vs-AVX {sens_logits:.2e}); per layer "
          + ", ".join(f"{o:.1e} ({s:.1e})" for o, s in zip(ours, sens_acv)))
    # whether an early layer already shows a flipped code is luck (T=7: the two reference builds agree to 1e-3 in layer 0,
    # to 2e-2 one layer later), so every layer is held to the reference's worst layer
    for layer in range(cfg.n_layers):
        assert ours[layer] <= SLACK * sens_acv.max() + min(ABS, 0.5 * sens_acv.max()), (layer, ours[layer], sens_acv)
    LOGIT_REL = SLACK * sens_logits + min(ABS, 0.5 * sens_logits)
    assert lerr <= LOGIT_REL, (lerr, sens_logits)
    # the next row through the ORDER-EXACT kernels, on top of the K/V cache the batched path wrote
    nxt = int(np.argmax(want_logits))
    toks = np.concatenate([prompt, [nxt]]).astype(np.int32)
    e.set_option("capture_acv", 0)
    got_next = e.logits(toks, n_prompt)
    want_next = cm.logits(toks, n_prompt)
    assert rel(got_next, want_next) <= LOGIT_REL, rel(got_next, want_next)
    e.close(); cm.close()


def test_batched_prefill_then_decode_runs_in_megakernel(capi):
    """After the batched prefill the device-side greedy loop continues from position T (tokens are well-formed ids)."""
    cfg = W.mini_config(n_layers=2, n_vocab=300)
    e = capi.Engine(cfg, 256, Q4).load(W.synth_weights(cfg, Q4, seed=3))
    prompt = W.synth_prompt(2, 130, cfg.n_vocab)
    e.prefill_fast(prompt)
    assert e.position() == 130
    e.decode(8)
    assert e.position() == 138
    toks = e.read_tokens(0, 139)
    assert np.array_equal(toks[:130], prompt)
    assert ((toks[130:] >= 0) & (toks[130:] < cfg.n_vocab)).all()
    # same prompt through the exact path: the first generated token agrees unless the top-2 margin is inside the tolerance
    e2 = capi.Engine(cfg, 256, Q4).load(W.synth_weights(cfg, Q4, seed=3))
    e2.prefill(prompt)
    lg = e2.read_logits()
    top2 = np.sort(lg)[-2:]
    if top2[1] - top2[0] > 0.05:
        assert e2.read_tokens(130, 1)[0] == toks[130]
    e.close(); e2.close()


@pytest.mark.parametrize("n_prompt", [1, 2, 33, 129, 190])
def test_batched_prefill_ragged_lengths(capi, checker, n_prompt):
    """Lengths that are not multiples of the 128-row GEMM tile / 64-row attention tile / 32-key block, the single-row
    prompt and the longest prompt max_ctx allows (n < max_ctx); bound = the worst spread the reference shows on this model."""
    cfg = W.mini_config(n_layers=2, n_vocab=300)
    wl = list(W.synth_weights(cfg, Q4, seed=12))
    max_ctx = 191
    cm = checker.model(cfg, 256, Q4).load(wl)                  # Q8 P rows: the reference needs ceil(n/32)*34 <= max_ctx
    e = capi.Engine(cfg, max_ctx, Q4).load(wl)
    prompt = W.synth_prompt(31, n_prompt, cfg.n_vocab)
    want = cm.logits(prompt, 0)
    e.prefill_fast(prompt)
    assert e.position() == n_prompt
    bound = SLACK * max(float(SENS[k]) for k in SENS.files if k.startswith("mini_") and k.endswith("_logits")) + ABS
    err = rel(e.read_logits(), want)
    assert err <= bound, (n_prompt, err, bound)
    e.close(); cm.close()


def test_batched_prefill_argument_errors(capi):
    cfg = W.mini_config(n_layers=1, n_vocab=64)
    e = capi.Engine(cfg, 32, Q8)
    with pytest.raises(capi.GtbError, match="not loaded"):
        e.prefill_fast(np.zeros(4, np.int32))
    e.load(W.synth_weights(cfg, Q8, seed=2))
    with pytest.raises(capi.GtbError, match="argument check failed"):
        e.prefill_fast(np.zeros(32, np.int32))              # n must leave room for the first generated token
    with pytest.raises(capi.GtbError, match="argument check failed"):
        e.prefill_fast(np.zeros(0, np.int32))
    e.close()


def test_fused_epilogues_equal_unfused_kernels(capi):
    """RoPE/KV-append and SiLU*up run inside the GEMM epilogues; the stand-alone kernels share their arithmetic, so both
    routes must give the same bits (logits, K/V cache via the next exact row)."""
    cfg = W.mini_config(n_layers=2, n_vocab=300)
    wl = list(W.synth_weights(cfg, Q4, seed=8))
    prompt = W.synth_prompt(9, 150, cfg.n_vocab)
    outs = []
    for fused in (1, 0):
        e = capi.Engine(cfg, 192, Q4).load(wl)
        e.set_option("pf_fused", fused)
        e.prefill_fast(prompt)
        lg = e.read_logits()
        nxt = e.logits(np.concatenate([prompt, [int(np.argmax(lg))]]).astype(np.int32), 150)
        outs.append((lg, nxt))
        e.close()
    assert np.array_equal(outs[0][0].view(np.uint32), outs[1][0].view(np.uint32))
    assert np.array_equal(outs[0][1].view(np.uint32), outs[1][1].view(np.uint32))


def test_batched_prefill_f16_two_sweep_attention(capi, checker):
    """FP16 activations: the two-sweep attention rounds p = e / sum to fp16 like ops.h:996 does; same bound."""
    _mini_case(capi, checker, F16, 64, {"pf_attn2": 1})


def test_batched_prefill_full_size_q8_2048_vs_golden(capi):
    """BASELINE.json config 4 at full size: the reference's logits after a 2048-token Q8 prefill (committed golden)."""
    f = GOLD / "prefill_q8.npz"
    if not f.exists():
        pytest.skip("prefill_q8.npz not generated")
    gold = np.load(f)
    cfg = W.TINYLLAMA
    e = capi.Engine(cfg, 2176, Q8).load(W.synth_weights(cfg, Q8, seed=1))
    prompt = gold["tokens"][:2048]
    e.prefill_fast(prompt)
    got = e.read_logits()
    err = rel(got, gold["logits"])
    sens = float(SENS["full_q8_2048_logits"]) if "full_q8_2048_logits" in SENS.files else None
    print(f"\nfull-size Q8 prefill 2048: logits rel L2 error {err:.2e} (reference scalar-vs-AVX: {sens}); "
          f"top-1 {int(np.argmax(got))} vs reference {int(np.argmax(gold['logits']))}")
    assert err <= (SLACK * sens + ABS if sens is not None else 0.25)
    e.close()
