"""Typed configuration of the Bofusun decoder, read from its config.json.

The file names the design under "architecture", gives `vocab`, `width`, `norm.eps`, a list
`layers` (each entry: `type`, the mixer's sizes under `mixer`, and `mlp` or null) and an
optional `loop` (`start`, `stop`, `times`): layers start..stop-1 run `times` times in a row
with the same weights, each pass with caches and states of its own.  Every size and every
constant a checkpoint can vary comes from there (or from a tensor's shape: the rows of the
distance-bias table); what the design fixes (1 + w gains, the key scale of retention, the
activation of the feed-forward, the halved sum of the parallel mixers) is written in `plan()`.

Layer types:
  "retention": decayed linear attention with rotated q and k (parts/retention.py).
  "parallel":  windowed softmax attention with capped scores, distance bias, short
               convolutions and a gate per head (parts/window_attention.py) beside a selective
               scan (parts/selective_scan.py), each RMS-normed and averaged (parts/combine.py).
Every branch is normed before and after (arrangement "sandwich_norm"), the embedding is normed
before it becomes the stream, and each pass over the repeated layers starts with a learned
vector and, from the second on, the embedding's output added to the stream.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Tuple

from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .qwen3 import ConfigError


def _need(d: Mapping[str, Any], keys, where: str) -> None:
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"{where} lacks required keys: {', '.join(missing)}")


def _freeze(x):
    if isinstance(x, Mapping):
        return tuple(sorted((k, _freeze(v)) for k, v in x.items()))
    if isinstance(x, (list, tuple)):
        return tuple(_freeze(v) for v in x)
    return x


@dataclass(frozen=True)
class BofusunLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]

    def __hash__(self):
        return hash((self.type, _freeze(self.mixer), _freeze(self.mlp)))


@dataclass(frozen=True)
class BofusunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[BofusunLayer, ...]
    loop: Optional[Tuple[int, int, int]] = None      # (start, stop, times)
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Bofusun"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BofusunConfig":
        _need(d, ("vocab", "width", "norm", "layers"), "config.json")
        _need(d["norm"], ("eps",), "config.json norm")
        layers = []
        for i, l in enumerate(d["layers"]):
            _need(l, ("type", "mixer"), f"layers[{i}]")
            layers.append(BofusunLayer(str(l["type"]), dict(l["mixer"]),
                                       dict(l["mlp"]) if l.get("mlp") is not None else None))
        loop = None
        if d.get("loop") is not None:
            _need(d["loop"], ("start", "stop", "times"), "config.json loop")
            loop = (int(d["loop"]["start"]), int(d["loop"]["stop"]), int(d["loop"]["times"]))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cfg = cls(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                  layers=tuple(layers), loop=loop, eos_token_ids=eos_ids)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path) -> "BofusunConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        for i, l in enumerate(self.layers):
            m, where = l.mixer, f"layers[{i}].mixer"
            if l.type == "retention":
                _need(m, ("heads", "dim", "vdim", "decay", "rot"), where)
                _need(m["rot"], ("dims", "base"), where + ".rot")
                if len(m["decay"]) != int(m["heads"]):
                    raise ConfigError(f"{where}: {len(m['decay'])} decays for {m['heads']} heads")
                if int(m["rot"]["dims"]) % 2 or not 0 <= int(m["rot"]["dims"]) <= int(m["dim"]):
                    raise ConfigError(f"{where}: rot.dims must be even and at most dim")
            elif l.type == "parallel":
                _need(m, ("left", "right"), where)
                _need(m["left"], ("heads", "kv_heads", "dim", "vdim", "conv", "scale", "bias_max", "mask"),
                      where + ".left")
                _need(m["left"]["mask"], ("size",), where + ".left.mask")
                _need(m["right"], ("inner", "state", "dt_rank", "conv"), where + ".right")
                if int(m["left"]["heads"]) % int(m["left"]["kv_heads"]):
                    raise ConfigError(f"{where}.left: heads is no multiple of kv_heads")
                if int(m["left"]["mask"]["size"]) < 1:
                    raise ConfigError(f"{where}.left: a window of {m['left']['mask']['size']} keys is not possible")
            else:
                raise ConfigError(f"layers[{i}].type={l.type!r} is not a known mixer; known: retention, parallel")
            if l.mlp is not None:
                _need(l.mlp, ("kind", "ff"), f"layers[{i}].mlp")
                if l.mlp["kind"] != "dense":
                    raise ConfigError(f"layers[{i}].mlp.kind={l.mlp['kind']!r} is not supported; only 'dense'")
        if self.loop is not None:
            a, b, t = self.loop
            if not (0 <= a < b <= len(self.layers)) or t < 1:
                raise ConfigError(f"loop {self.loop} does not name layers of this model")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": json.loads(json.dumps(l.mixer)),
                        "mlp": json.loads(json.dumps(l.mlp)) if l.mlp is not None else None} for l in self.layers],
        }
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # --------------------------------------------------------------------- plan
    def _norm(self, name: str) -> PartSpec:
        # gains are stored around zero: the norm multiplies by 1 + w
        return PartSpec("rmsnorm", {"dim": self.width, "eps": self.norm_eps, "offset": 1.0, "suffix": ""}, name)

    def _mixer(self, l: BofusunLayer) -> PartSpec:
        m = l.mixer
        if l.type == "retention":
            rot = m["rot"]
            return PartSpec("retention", {
                "hidden_size": self.width, "num_heads": int(m["heads"]), "key_dim": int(m["dim"]),
                "value_dim": int(m["vdim"]), "decay": tuple(float(x) for x in m["decay"]),
                "key_scale": float(int(m["dim"])) ** -0.5, "norm_eps": self.norm_eps,
                "position": PartSpec("rotary", {"head_dim": int(m["dim"]), "rotary_dim": int(rot["dims"]),
                                                "theta": float(rot["base"]), "table_precision": "float64"}),
            }, "mix.")
        left, right = m["left"], m["right"]
        attention = PartSpec("window_bias_attention", {
            "hidden_size": self.width, "num_heads": int(left["heads"]), "num_kv_heads": int(left["kv_heads"]),
            "key_dim": int(left["dim"]), "value_dim": int(left["vdim"]), "conv_taps": int(left["conv"]),
            "scale": float(left["scale"]), "softcap": float(left["softcap"]) if left.get("softcap") else 0.0,
            "window": int(left["mask"]["size"]), "bias_far": float(left["bias_max"]),
        }, "left.")
        scan = PartSpec("selective_scan", {
            "hidden_size": self.width, "inner_size": int(right["inner"]), "state_size": int(right["state"]),
            "dt_rank": int(right["dt_rank"]), "conv_taps": int(right["conv"]),
        }, "right.")
        return PartSpec("normed_mean", {"hidden_size": self.width, "eps": self.norm_eps,
                                        "branches": (attention, scan)}, "mix.")

    def plan(self) -> ModelPlan:
        layers = []
        for i, l in enumerate(self.layers):
            ff = None
            norms = (self._norm("norm1"), self._norm("norm1b"))
            if l.mlp is not None:
                ff = PartSpec("dense_act", {"hidden_size": self.width, "intermediate_size": int(l.mlp["ff"]),
                                            "activation": "relu_squared", "bias": True}, "mlp.")
                norms = (*norms, self._norm("norm2"), self._norm("norm2b"))
            layers.append(LayerSpec("sandwich_norm", f"l{i}.", norms, self._mixer(l), ff))
        n = len(self.layers)
        if self.loop is None:
            order = [RunEntry(i) for i in range(n)]
        else:
            a, b, times = self.loop
            order = [RunEntry(i) for i in range(a)]
            for t in range(times):
                inject = PartSpec("pass_inject", {"dim": self.width, "passes": times, "index": t,
                                                  "add_embedding": t > 0}, "loop.")
                order += [RunEntry(i, before=inject if i == a else None) for i in range(a, b)]
            order += [RunEntry(i) for i in range(b, n)]
        plan = ModelPlan(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            embedding=PartSpec("normed_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                    "suffix": "", "norm": self._norm(".norm")}, "embed"),
            layers=tuple(layers), order=tuple(order),
            final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"hidden_size": self.width, "vocab_size": self.vocab, "tied_to": None,
                                      "suffix": ""}, "head"),
        )
        plan.validate()
        return plan

    def describe(self) -> dict:
        return self.to_dict()
