"""Tiny Bofusun configurations for the tests, their random weights, and a harness that feeds
schedules through the engine's step function and cache manager.

The configurations differ from one another in every size and option: head counts that do not
divide anything nicely, key and value sizes that differ, 1, 2, 3 and 4 convolution taps, windows
that are no multiple of a page, a bias table with an odd number of rows, a loop of three passes
that starts at layer 0, a loop of one pass, no loop, a feed-forward on a retention layer and none
on a parallel one, partial rotation and none.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def _ret(heads, dim, vdim, rot, base, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "rot": {"dims": rot, "base": base}, "decay": decay}


def _par(heads, kv, dim, vdim, conv, scale, softcap, bias_max, window, inner, state, rank, rconv):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale,
            "bias_max": bias_max, "mask": {"size": window}}
    if softcap is not None:
        left["softcap"] = softcap
    return {"left": left, "right": {"inner": inner, "state": state, "dt_rank": rank, "conv": rconv}}


TINY = {
    # three passes over layers 0..1, starting at layer 0
    "P": ({"architecture": "Bofusun", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
           "layers": [
               {"type": "retention", "mixer": _ret(3, 8, 16, 4, 100.0, [0.9, 0.97, 0.995]),
                "mlp": {"kind": "dense", "ff": 40}},
               {"type": "parallel", "mixer": _par(4, 2, 16, 8, 2, 0.3, 5.0, 20, 11, 40, 6, 3, 4), "mlp": None},
               {"type": "retention", "mixer": _ret(2, 16, 8, 16, 10000.0, [0.5, 0.999]), "mlp": None}],
           "loop": {"start": 0, "stop": 2, "times": 3}}, 12),
    # no loop, one tap on the left (no convolution state), no cap, an odd bias table, one head
    "Q": ({"architecture": "Bofusun", "vocab": 61, "width": 32, "norm": {"eps": 1e-6},
           "layers": [
               {"type": "parallel", "mixer": _par(2, 2, 8, 8, 1, 0.5, None, 64, 37, 24, 16, 5, 3),
                "mlp": {"kind": "dense", "ff": 72}},
               {"type": "retention", "mixer": _ret(1, 16, 8, 0, 10000.0, [0.98]), "mlp": None}]}, 9),
    # a loop of one pass in the middle, two parallel layers with different windows, six query heads on one KV head
    "R": ({"architecture": "Bofusun", "vocab": 130, "width": 40, "norm": {"eps": 1e-5},
           "layers": [
               {"type": "parallel", "mixer": _par(6, 1, 8, 16, 3, 0.25, 8.0, 100, 16, 32, 33, 2, 2), "mlp": None},
               {"type": "retention", "mixer": _ret(5, 8, 8, 6, 500.0, [0.8, 0.9, 0.95, 0.99, 0.9999]),
                "mlp": {"kind": "dense", "ff": 24}},
               {"type": "parallel", "mixer": _par(2, 1, 16, 16, 4, 0.2, 3.0, 48, 50, 16, 4, 1, 1),
                "mlp": {"kind": "dense", "ff": 56}}],
           "loop": {"start": 1, "stop": 2, "times": 1}}, 20),
    # retention only (no pages at all), a feed-forward on every layer, the whole model run twice
    "S": ({"architecture": "Bofusun", "vocab": 300, "width": 24, "norm": {"eps": 1e-5},
           "layers": [
               {"type": "retention", "mixer": _ret(2, 4, 12, 2, 50.0, [0.9, 0.99]), "mlp": {"kind": "dense", "ff": 16}},
               {"type": "retention", "mixer": _ret(1, 24, 24, 24, 1e6, [0.97]), "mlp": {"kind": "dense", "ff": 32}}],
           "loop": {"start": 0, "stop": 2, "times": 2}}, 4),
}


def make_weights(cfg: dict, seed: int, rel_rows: int):
    """Random tensors for a configuration, scaled so that every mechanism matters: projections large
    enough for scores to reach the cap, distance biases and taps of order one."""
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.model import Model
    from socrates_b200.weights.random_init import random_tensors
    params = Model(config_from_dict(cfg).plan()).parameters()
    w = random_tensors(params, seed)
    g = torch.Generator().manual_seed(seed + 1)
    for name in list(w):
        t = w[name]
        if name.endswith(".rel"):
            t = torch.randn(rel_rows, t.shape[1], generator=g)
        elif name.endswith(".conv"):
            t = 0.6 * torch.randn(t.shape, generator=g)
        elif params[name].role == "matrix":
            t = t.float() * (8.0 if name.endswith((".left.q", ".left.k")) else 4.0)
        elif name.endswith(".b") and not name.endswith("dt.b"):
            t = t.float() * 5.0
        if name == "loop.step":
            t = 0.5 * torch.randn(t.shape, generator=g)
        # everything is stored as bfloat16, so both engines and the plain statement read equal values
        w[name] = t.to(torch.bfloat16)
    return w


def make_folder(tmp_path, name: str, seed: int = 3):
    """(folder, config dict, weights as float64) of the tiny model `name`."""
    from safetensors.torch import save_file
    cfg, rel_rows = TINY[name]
    w = make_weights(cfg, seed, rel_rows)
    folder = Path(tmp_path) / f"bofusun_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in w.items()}, str(folder / "model.safetensors"))
    return folder, cfg, {k: v.double() for k, v in w.items()}


class Harness:
    """The engine's model, cache manager and step function on a model folder, driven step by step."""

    def __init__(self, folder, dtype, max_rows=4, max_len=512, page=16, pages=None, graphs=False):
        from socrates_b200.cache import CacheManager
        from socrates_b200.engine.engine import build_model
        from socrates_b200.engine.runner import ModelRunner
        self.config, self.model = build_model(folder, dtype, "cuda")
        pages = pages if pages is not None else max_rows * (max_len // page)
        self.cache = CacheManager(self.model.cache_needs(), max_rows, max_len, page, pages, dtype, "cuda")
        self.runner = ModelRunner(self.model, self.cache, dtype, "cuda", max_tokens=max_len, max_seqs=max_rows,
                                  use_graphs=graphs)
        self.rows, self.free = {}, list(range(max_rows - 1, -1, -1))

    def step(self, entries, end=()):
        """entries: [(request id, tokens)]; returns {request id: float64 logits [len(tokens), vocab]}."""
        from socrates_b200.engine.runner import StepEntry
        batch = []
        for rid, tokens in entries:
            if rid not in self.rows:
                self.rows[rid] = self.free.pop()
                self.cache.assign(self.rows[rid])
            row = self.rows[rid]
            start = self.cache.lengths[row]
            assert self.cache.reserve(row, start + len(tokens)), "the pool ran out of pages"
            batch.append(StepEntry(row, list(tokens), start, list(range(len(tokens)))))
        logits = self.runner.step(batch).logits.double().cpu()
        self.runner.check_status()
        out, i = {}, 0
        for (rid, tokens), e in zip(entries, batch):
            out[rid] = logits[i:i + len(tokens)]
            i += len(tokens)
            self.cache.commit(e.row, e.start + len(tokens))
        for rid in end:
            row = self.rows.pop(rid)
            self.cache.release(row)
            self.free.append(row)
        self.cache.check()
        return out

    def run(self, rid, ids, sizes):
        """One request alone in portions of the given sizes (the last size repeats); all its logits."""
        got, i, k = [], 0, 0
        while i < len(ids):
            c = min(sizes[min(k, len(sizes) - 1)], len(ids) - i)
            got.append(self.step([(rid, ids[i:i + c])], end=[rid] if i + c == len(ids) else [])[rid])
            i, k = i + c, k + 1
        return torch.cat(got)


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest difference relative to the largest logit of the sequence."""
    return float((got - want).abs().max() / want.abs().max())
