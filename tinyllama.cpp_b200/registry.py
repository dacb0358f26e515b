"""Model registry: which family a checkpoint belongs to and how it is opened.

A checkpoint folder with a config.json names its family in "architecture"; a .gten file is a TinyLlama checkpoint of the
reference's converter (tinyllama.cpp:336-392).  open_model() returns an object with the family's native engine behind it."""
from __future__ import annotations

import json
from pathlib import Path


def _open_described(family, path: Path, dtype: str, n_slots: int, max_ctx: int, max_rows: int = 0, device: int = 0):
    """A family of the layer-list library: `family` is its module (read_checkpoint, tensor_shapes)."""
    from . import seq
    seq.init(device)
    desc, tensors = family.read_checkpoint(path)
    known = family.tensor_shapes(desc)
    extra = sorted(set(tensors) - set(known))
    if extra:                                   # e.g. a filter of a feed-forward that the layer does not have
        import sys
        print(f"{path}: ignoring {len(extra)} tensors the description does not use: {', '.join(extra[:4])}{' ...' if len(extra) > 4 else ''}", file=sys.stderr)
        tensors = {k: v for k, v in tensors.items() if k in known}
    if dtype not in seq.MODE_BY_NAME:
        raise ValueError(f"dtype {dtype!r}: this family runs in bfloat16 or float32")
    return seq.SeqModel(desc, seq.MODE_BY_NAME[dtype], n_slots, max_ctx, max_rows).load(tensors)


def _open_tinyllama(path: Path, dtype: str, n_slots: int, max_ctx: int, max_rows: int = 0, device: int = 0):
    from . import capi, weights as W
    capi.init(device)
    if dtype not in W.WDTYPE_BY_NAME:
        raise ValueError(f"dtype {dtype!r}: this family runs its checkpoint formats fp16, q8, q4")
    e = capi.Engine(W.TINYLLAMA, max_ctx, W.WDTYPE_BY_NAME[dtype]).load_gten(path)
    if n_slots > 1:
        e.batch_create(n_slots)
    return e


def _open_reninex(path: Path, dtype: str, n_slots: int, max_ctx: int, **kw):
    from . import reninex
    return _open_described(reninex, path, dtype, n_slots, max_ctx, **kw)


def _open_robopel(path: Path, dtype: str, n_slots: int, max_ctx: int, **kw):
    from . import robopel
    return _open_described(robopel, path, dtype, n_slots, max_ctx, **kw)


def _open_nanotar(path: Path, dtype: str, n_slots: int, max_ctx: int, **kw):
    from . import nanotar
    return _open_described(nanotar, path, dtype, n_slots, max_ctx, **kw)


def _open_vulosun(path: Path, dtype: str, n_slots: int, max_ctx: int, **kw):
    from . import vulosun
    return _open_described(vulosun, path, dtype, n_slots, max_ctx, **kw)


FAMILIES = {"Nanotar": _open_nanotar, "Reninex": _open_reninex, "Robopel": _open_robopel, "TinyLlama": _open_tinyllama, "Vulosun": _open_vulosun}
STEPWISE = {"Nanotar", "Reninex", "Robopel", "Vulosun"}          # families of the layer-list library: slots, portion-wise step function, scheduler


def family_of(path) -> str:
    path = Path(path)
    if path.is_dir():
        cfg = path / "config.json"
        if not cfg.exists():
            raise FileNotFoundError(f"{path} has no config.json")
        arch = json.loads(cfg.read_text()).get("architecture")
        if arch not in FAMILIES:
            raise ValueError(f"{path}: architecture {arch!r} is not registered (known: {sorted(FAMILIES)})")
        return arch
    if path.suffix == ".gten":
        return "TinyLlama"
    raise ValueError(f"{path}: neither a checkpoint folder nor a .gten file")


def open_model(path, dtype: str, n_slots: int = 1, max_ctx: int = 2048, **kw):
    return FAMILIES[family_of(path)](Path(path), dtype, n_slots, max_ctx, **kw)
