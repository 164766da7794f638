"""Tiny Loletar configurations for the tests and their random weights.

The configurations differ from one another in every size and option: head counts that divide
nothing nicely, key and value sizes that differ or are equal, head sizes that are no multiple of a
warp, 1 to 4 convolution taps, full, partial and no rotation, layers that borrow an earlier layer's
keys and values (next to it and two layers back), dense, routed and no feed-forwards, routers with
and without identity experts, with one group, with all groups kept and with some closed, top-1 to
top-3, a model that starts with a recurrent layer, and one without any attention (no pages at all).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def _att(heads, kv, dim, vdim, rot, base, scale, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"dims": rot, "base": base}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _delta(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(ff, experts, identity, top, count=None, keep=None):
    router = {"experts": experts, "top": top, "identity": identity}
    if count is not None:
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


TINY = {
    # starts with a recurrent layer; a borrowed cache right after its owner; closed groups; a top-1 router without groups
    "A": {"architecture": "Loletar", "vocab": 101, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0},
          "layers": [
              {"type": "delta", "mixer": _delta(4, 2, 16, 8, 2), "mlp": _moe(24, 5, 1, 2, 3, 2)},
              {"type": "attention", "mixer": _att(6, 2, 16, 8, 6, 100.0, 0.3), "mlp": _dense(40)},
              {"type": "attention", "mixer": _att(6, 2, 16, 8, 6, 100.0, 0.3, kv_from=1), "mlp": None},
              {"type": "attention", "mixer": _att(2, 1, 8, 24, 8, 10000.0, 0.5), "mlp": _moe(16, 4, 0, 1)}]},
    # no rotation, equal key and value sizes, a cache borrowed across two recurrent layers, head sizes of 40 and 72
    "B": {"architecture": "Loletar", "vocab": 67, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
          "layers": [
              {"type": "attention", "mixer": _att(3, 3, 24, 24, None, None, 0.2), "mlp": _moe(8, 6, 2, 3, 4, 4)},
              {"type": "delta", "mixer": _delta(1, 1, 40, 40, 1), "mlp": _dense(56)},
              {"type": "delta", "mixer": _delta(2, 1, 8, 72, 4), "mlp": None},
              {"type": "attention", "mixer": _att(3, 3, 24, 24, None, None, 0.2, kv_from=0), "mlp": _dense(24)}]},
    # keys and values of one size, 64 and 128: in the bfloat16 engine prompt portions of these layers run on the
    # tensor-core attention kernel; one router output per group
    "D": {"architecture": "Loletar", "vocab": 80, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
          "layers": [
              {"type": "attention", "mixer": _att(4, 2, 64, 64, 32, 10000.0, 0.125), "mlp": _dense(48)},
              {"type": "attention", "mixer": _att(4, 2, 64, 64, 32, 10000.0, 0.125, kv_from=0), "mlp": _moe(16, 4, 1, 2, 5, 2)},
              {"type": "attention", "mixer": _att(2, 1, 128, 128, 128, 500000.0, 0.09), "mlp": None},
              {"type": "delta", "mixer": _delta(2, 2, 64, 64, 4), "mlp": _dense(40)}]},
    # recurrent layers only: no pages at all; as many identity experts as real ones, one group of two kept
    "C": {"architecture": "Loletar", "vocab": 300, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
          "layers": [
              {"type": "delta", "mixer": _delta(2, 2, 32, 16, 3), "mlp": _moe(12, 3, 3, 2, 2, 1)},
              {"type": "delta", "mixer": _delta(3, 1, 16, 16, 2), "mlp": None}]},
}


def make_weights(cfg: dict, seed: int):
    """Random tensors for a configuration, scaled so that every mechanism matters: projections large enough
    for attention to be peaked and for the router to prefer some experts, corrections that change choices."""
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.model import Model
    from socrates_b200.weights.random_init import random_tensors
    params = Model(config_from_dict(cfg).plan()).parameters()
    w = random_tensors(params, seed)
    g = torch.Generator().manual_seed(seed + 1)
    for name in list(w):
        t = w[name].float()
        if name.endswith(".router"):
            t = t * 30.0
        elif name.endswith(".correction"):
            t = 0.15 * torch.randn(t.shape, generator=g)
        elif name == "embed":
            t = t * 20.0
        elif params[name].role == "matrix":
            t = t * 4.0
        # everything is stored as bfloat16, so both engines and the plain statement read equal values
        w[name] = t.to(torch.bfloat16)
    return w


def make_folder(tmp_path, name: str, seed: int = 5):
    """(folder, config dict, weights as float64) of the tiny model `name`."""
    from safetensors.torch import save_file
    cfg = TINY[name]
    w = make_weights(cfg, seed)
    folder = Path(tmp_path) / f"loletar_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in w.items()}, str(folder / "model.safetensors"))
    return folder, cfg, {k: v.double() for k, v in w.items()}


def save_weights(folder, w):
    from safetensors.torch import save_file
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, str(Path(folder) / "model.safetensors"))
