"""ctypes binding of libgten_b200_seq.so (include/gten_b200_seq.h): layer-list sequence models.

No compute lives here and there is no fallback: a missing library or a missing CUDA device raises."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libgten_b200_seq.so"

BF16, F32 = 0, 1
MIX_SIGMOID_ATTN, MIX_RETENTION, MIX_MINGRU, MIX_SOFTMAX_ATTN, MIX_LATENT_ATTN = 1, 2, 3, 4, 5
BLOCK_PARALLEL, BLOCK_POSTNORM, BLOCK_PRENORM, BLOCK_SANDWICH = 0, 1, 2, 3
FF_GEGLU, FF_POLYNORM, FF_EXPERTS, FF_GATED_EXPERTS, FF_SWIGLU, FF_GROUP_EXPERTS = 0, 1, 2, 3, 4, 5
NORM_RMS, NORM_DYT, NORM_LAYER = 0, 1, 2
ROT_HALVES, ROT_INTERLEAVED = 0, 1
MODE_BY_NAME = {"bfloat16": BF16, "bf16": BF16, "float32": F32, "fp32": F32}


class SeqError(RuntimeError):
    pass


class BranchC(C.Structure):
    _fields_ = [("kind", C.c_int), ("name", C.c_char * 16), ("heads", C.c_int), ("kv_heads", C.c_int), ("dim", C.c_int), ("vdim", C.c_int),
                ("scale", C.c_float), ("qk_norm", C.c_int), ("rot_dims", C.c_int), ("rot_base", C.c_float), ("out_norm", C.c_int),
                ("gated", C.c_int), ("out_scale", C.c_float), ("decay", C.POINTER(C.c_float)), ("rot_layout", C.c_int),
                ("rot_factor", C.c_float), ("rot_low", C.c_float), ("rot_high", C.c_float), ("rot_original", C.c_float), ("softcap", C.c_float),
                ("window", C.c_int), ("pool", C.c_int), ("sink", C.c_int), ("kv_from", C.c_int),
                ("rope_dim", C.c_int), ("kv_rank", C.c_int), ("q_rank", C.c_int),
                ("chunk", C.c_int), ("maps", C.c_int), ("diff", C.c_float), ("bias", C.c_int), ("act", C.c_int), ("rot_divide", C.c_float)]


class LayerC(C.Structure):
    _fields_ = [("n_branches", C.c_int), ("branch", BranchC * 2), ("ff", C.c_int), ("style", C.c_int), ("ff_kind", C.c_int),
                ("experts", C.c_int), ("top", C.c_int), ("identity", C.c_int), ("norm_kind", C.c_int), ("shared_ff", C.c_int),
                ("route_groups", C.c_int), ("route_keep", C.c_int), ("route_scale", C.c_float)]


class ConfigC(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("vocab", "width", "n_layers")] + [("eps", C.c_float)] + \
               [(n, C.c_int) for n in ("taps", "bigram_buckets", "bigram_mul_prev", "bigram_mul_cur", "loop_start", "loop_stop", "loop_times",
                                       "mode", "n_slots", "max_ctx", "max_rows")] + [("embed_scale", C.c_float), ("final_norm", C.c_int), ("streams", C.c_int),
                                                                                     ("logit_softcap", C.c_float)]


SYMBOLS = ["gtb_seq_create", "gtb_seq_destroy", "gtb_seq_set_tensor", "gtb_seq_finalize", "gtb_seq_n_runs", "gtb_seq_slot_reset",
           "gtb_seq_slot_position", "gtb_seq_step", "gtb_seq_step_greedy", "gtb_seq_decode", "gtb_seq_topk", "gtb_seq_last_logits",
           "gtb_seq_set_option", "gtb_seq_read_capture", "gtb_seq_weight_bytes", "gtb_seq_state_bytes_per_slot", "gtb_seq_selftest_gemm"]

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise SeqError(f"{LIB_PATH} is missing: build it with tinyllama.cpp_b200/build.py --target seq")
        L = C.CDLL(str(LIB_PATH))
        vp, i, sz = C.c_void_p, C.c_int, C.c_size_t
        L.gtb_last_error.restype = C.c_char_p
        L.gtb_launch_count.restype = C.c_int64
        L.gtb_stream.restype = vp
        sigs = {
            "gtb_init": [i], "gtb_sync": [],
            "gtb_seq_create": [C.POINTER(vp), C.POINTER(ConfigC), C.POINTER(LayerC)], "gtb_seq_destroy": [vp],
            "gtb_seq_set_tensor": [vp, C.c_char_p, vp, C.POINTER(C.c_int64), i], "gtb_seq_finalize": [vp],
            "gtb_seq_n_runs": [vp, C.POINTER(i)], "gtb_seq_slot_reset": [vp, i], "gtb_seq_slot_position": [vp, i, C.POINTER(i)],
            "gtb_seq_step": [vp, i, vp, vp, vp, i, vp, vp], "gtb_seq_step_greedy": [vp, i, vp, vp, vp, vp],
            "gtb_seq_decode": [vp, i, vp, i, i, vp], "gtb_seq_topk": [vp, i, i, vp, vp], "gtb_seq_last_logits": [vp, i, vp],
            "gtb_seq_set_option": [vp, C.c_char_p, i], "gtb_seq_read_capture": [vp, i, i, vp],
            "gtb_seq_selftest_gemm": [vp, vp, vp, i, i, i, i, i, i, C.POINTER(C.c_float)],
            "gtb_seq_weight_bytes": [vp, C.POINTER(sz)], "gtb_seq_state_bytes_per_slot": [vp, C.POINTER(sz)],
        }
        for name, args in sigs.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = C.c_int
        _lib = L
    return _lib


def check(rc: int):
    if rc != 0:
        raise SeqError(f"gtb error {rc}: {lib().gtb_last_error().decode()}")


def init(device: int = 0):
    check(lib().gtb_init(device))


def sync():
    check(lib().gtb_sync())


def launch_count() -> int:
    return int(lib().gtb_launch_count())


def stream_handle() -> int:
    return int(lib().gtb_stream() or 0)


def _hp(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, np.int32)


def selftest_gemm(a_bits: np.ndarray, w_bits: np.ndarray, c0: np.ndarray | None = None, ld_extra: int = 0, iters: int = 1, cold: bool = False):
    """The tcgen05 bf16 product on host operands (bfloat16 bit patterns): returns (A . W^T (+ c0), mean milliseconds of `iters` runs)."""
    a, w = np.ascontiguousarray(a_bits, np.uint16), np.ascontiguousarray(w_bits, np.uint16)
    (m, k), n = a.shape, w.shape[0]
    c = np.zeros((m, n), np.float32) if c0 is None else np.ascontiguousarray(c0, np.float32).copy()
    ms = C.c_float()
    check(lib().gtb_seq_selftest_gemm(_hp(a), _hp(w), _hp(c), m, n, k, ld_extra, 2 if cold else int(c0 is not None), iters, C.byref(ms)))
    return c, ms.value


class SeqModel:
    """A described model resident on the GPU: weights, n_slots sequences of state, the step function."""

    def __init__(self, desc: dict, mode: int, n_slots: int, max_ctx: int, max_rows: int = 0):
        """desc: the flat description a model family's config reader produces (see reninex.describe, robopel.describe, nanotar.describe,
        vulosun.describe)."""
        self.desc, self.mode, self.n_slots, self.max_ctx = desc, mode, n_slots, max_ctx
        self.vocab, self.width = desc["vocab"], desc["width"]
        layers = (LayerC * len(desc["layers"]))()
        self._keep = []
        for lc, l in zip(layers, desc["layers"]):
            lc.n_branches = len(l["branches"])
            lc.ff = l["ff"]
            lc.style, lc.ff_kind = l.get("style", BLOCK_PARALLEL), l.get("ff_kind", FF_GEGLU)
            lc.experts, lc.top, lc.identity = l.get("experts", 0), l.get("top", 0), l.get("identity", 0)
            lc.norm_kind, lc.shared_ff = l.get("norm_kind", NORM_RMS), l.get("shared_ff", 0)
            lc.route_groups, lc.route_keep, lc.route_scale = l.get("route_groups", 0), l.get("route_keep", 0), l.get("route_scale", 1.0)
            for bc, b in zip(lc.branch, l["branches"]):
                bc.kind, bc.name = b["kind"], b["name"].encode()
                bc.heads, bc.kv_heads, bc.dim, bc.vdim = b["heads"], b.get("kv_heads", b["heads"]), b["dim"], b["vdim"]
                bc.scale, bc.qk_norm = b["scale"], int(b.get("qk_norm", 0))
                bc.rot_dims, bc.rot_base = b.get("rot_dims", 0), b.get("rot_base", 10000.0)
                bc.out_norm, bc.gated, bc.out_scale = int(b.get("out_norm", 0)), int(b.get("gated", 0)), b.get("out_scale", 1.0)
                bc.rot_layout = b.get("rot_layout", ROT_HALVES)
                bc.rot_factor, bc.rot_low, bc.rot_high, bc.rot_original = (b.get("rot_" + k, 0.0) for k in ("factor", "low", "high", "original"))
                bc.softcap, bc.window, bc.pool = b.get("softcap", 0.0), b.get("window", 0), b.get("pool", 0)
                bc.sink, bc.kv_from = int(b.get("sink", 0)), b.get("kv_from", -1)
                bc.rope_dim, bc.kv_rank, bc.q_rank = b.get("rope_dim", 0), b.get("kv_rank", 0), b.get("q_rank", 0)
                bc.chunk, bc.maps, bc.diff = b.get("chunk", 0), b.get("maps", 1), b.get("diff", 0.0)
                bc.bias, bc.act, bc.rot_divide = int(b.get("bias", 0)), int(b.get("act", 0)), b.get("rot_divide", 0.0)
                if b.get("decay") is not None:
                    arr = (C.c_float * len(b["decay"]))(*b["decay"])
                    self._keep.append(arr)
                    bc.decay = C.cast(arr, C.POINTER(C.c_float))
        bg, lp = desc.get("bigram"), desc.get("loop")
        cfg = ConfigC(desc["vocab"], desc["width"], len(desc["layers"]), desc["eps"], desc.get("taps", 0),
                      bg["buckets"] if bg else 0, bg["mul_prev"] if bg else 0, bg["mul_cur"] if bg else 0,
                      lp["start"] if lp else 0, lp["stop"] if lp else 0, lp["times"] if lp else 0, mode, n_slots, max_ctx, max_rows,
                      desc.get("embed_scale", 1.0), int(desc.get("final_norm", 0)), int(desc.get("streams", 0)), float(desc.get("logit_softcap", 0.0)))
        self.h = C.c_void_p()
        check(lib().gtb_seq_create(C.byref(self.h), C.byref(cfg), layers))
        n = C.c_int()
        check(lib().gtb_seq_n_runs(self.h, C.byref(n)))
        self.n_runs = n.value

    def close(self):
        if self.h:
            lib().gtb_seq_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_tensor(self, name: str, bf16_bits: np.ndarray):
        a = np.ascontiguousarray(bf16_bits, np.uint16)
        shape = (C.c_int64 * max(a.ndim, 1))(*a.shape)
        check(lib().gtb_seq_set_tensor(self.h, name.encode(), _hp(a.reshape(-1)) if a.size else None, shape, a.ndim))

    def load(self, tensors: dict) -> "SeqModel":
        """tensors: name -> bfloat16 bit patterns (uint16 arrays)."""
        for name, a in tensors.items():
            self.set_tensor(name, a)
        check(lib().gtb_seq_finalize(self.h))
        return self

    def set_option(self, name: str, value: int):
        check(lib().gtb_seq_set_option(self.h, name.encode(), int(value)))

    def reset(self, slot: int):
        check(lib().gtb_seq_slot_reset(self.h, slot))

    def position(self, slot: int) -> int:
        p = C.c_int()
        check(lib().gtb_seq_slot_position(self.h, slot, C.byref(p)))
        return p.value

    def step(self, segments, want=()) -> np.ndarray:
        """segments: [(slot, tokens)]; want: row indices into the concatenated tokens, ascending.  Returns logits [len(want), vocab]."""
        slots = _i32([s for s, _ in segments])
        lens = _i32([len(t) for _, t in segments])
        toks = _i32(np.concatenate([np.asarray(t, np.int64) for _, t in segments]))
        w = _i32(list(want))
        out = np.empty((w.size, self.vocab), np.float32)
        check(lib().gtb_seq_step(self.h, slots.size, _hp(slots), _hp(lens), _hp(toks), w.size, _hp(w) if w.size else None, _hp(out) if w.size else None))
        return out

    def step_greedy(self, segments) -> np.ndarray:
        """Feeds the segments and returns the greedy next token of each (the slot keeps it for decode())."""
        slots = _i32([s for s, _ in segments])
        lens = _i32([len(t) for _, t in segments])
        toks = _i32(np.concatenate([np.asarray(t, np.int64) for _, t in segments]))
        nxt = np.empty(slots.size, np.int32)
        check(lib().gtb_seq_step_greedy(self.h, slots.size, _hp(slots), _hp(lens), _hp(toks), _hp(nxt)))
        return nxt

    def decode(self, slots, n_steps: int, eos_id: int = -1) -> np.ndarray:
        """n greedy steps of the slots on the device; returns tokens [len(slots), n_steps]."""
        s = _i32(list(slots))
        out = np.empty((s.size, n_steps), np.int32)
        check(lib().gtb_seq_decode(self.h, s.size, _hp(s), n_steps, eos_id, _hp(out)))
        return out

    def topk(self, seg: int, k: int):
        v, ids = np.empty(k, np.float32), np.empty(k, np.int32)
        check(lib().gtb_seq_topk(self.h, seg, k, _hp(v), _hp(ids)))
        return v, ids

    def last_logits(self, seg: int) -> np.ndarray:
        out = np.empty(self.vocab, np.float32)
        check(lib().gtb_seq_last_logits(self.h, seg, _hp(out)))
        return out

    def read_capture(self, run: int, row: int) -> np.ndarray:
        out = np.empty(self.width, np.float32)
        check(lib().gtb_seq_read_capture(self.h, run, row, _hp(out)))
        return out

    def weight_bytes(self) -> int:
        n = C.c_size_t()
        check(lib().gtb_seq_weight_bytes(self.h, C.byref(n)))
        return n.value

    def state_bytes_per_slot(self) -> int:
        n = C.c_size_t()
        check(lib().gtb_seq_state_bytes_per_slot(self.h, C.byref(n)))
        return n.value
