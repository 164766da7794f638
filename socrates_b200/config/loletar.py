"""Typed configuration of the Loletar decoder, read from its config.json.

The file names the design under "architecture" and gives `vocab`, `width`, `norm.eps`,
`embedding.scale` and a list `layers`; each entry has a `type` ("attention" or "delta"), the
mixer's sizes under `mixer` and its feed-forward under `mlp` (null: none; `kind` "dense" with
`ff`, or "moe" with `expert.ff` and `router`: `experts`, `top`, `identity`, `groups.count`,
`groups.keep`).  An attention mixer with `kv_from: j` has no keys and values of its own and
reads those of layer j.  Every size and every constant a checkpoint can vary comes from
there; what the design fixes is written in `plan()`:

  * the looked-up embedding rows are multiplied by `embedding.scale`;
  * a layer is x + norm(mixer(x)), then x + norm(ff(x)): RMS norms with plain gains on the
    branches' outputs only (arrangement "branch_norm");
  * attention ("gated_sink_attention"): per-head RMS norm of q and k, rotation of the first
    `rot.dims` dims in neighbouring pairs, a softmax whose denominator holds one more term of
    score 0, a sigmoid gate per head and value dim;
  * delta ("gated_delta_rule"): short convolutions with SiLU on q, k and v, unit q and k, a
    query scale of dim^-1/2;
  * feed-forwards are gated with SiLU; the routed one ("routed_experts") weighs the chosen
    experts by their plain softmax scores.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Tuple

from .bofusun import _freeze, _need
from .plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .qwen3 import ConfigError


@dataclass(frozen=True)
class LoletarLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]

    def __hash__(self):
        return hash((self.type, _freeze(self.mixer), _freeze(self.mlp)))


@dataclass(frozen=True)
class LoletarConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[LoletarLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Loletar"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LoletarConfig":
        _need(d, ("vocab", "width", "norm", "layers"), "config.json")
        _need(d["norm"], ("eps",), "config.json norm")
        layers = []
        for i, l in enumerate(d["layers"]):
            _need(l, ("type", "mixer"), f"layers[{i}]")
            layers.append(LoletarLayer(str(l["type"]), dict(l["mixer"]),
                                       dict(l["mlp"]) if l.get("mlp") is not None else None))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        scale = float((d.get("embedding") or {}).get("scale", 1.0))
        cfg = cls(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                  embedding_scale=scale, layers=tuple(layers), eos_token_ids=eos_ids)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path) -> "LoletarConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    @staticmethod
    def _router(mlp: Mapping[str, Any]) -> Dict[str, int]:
        r = mlp["router"]
        groups = r.get("groups") or {}
        return {"experts": int(r["experts"]), "top": int(r["top"]), "identity": int(r.get("identity", 0)),
                "groups": int(groups.get("count", 1)), "keep": int(groups.get("keep", groups.get("count", 1)))}

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        for i, l in enumerate(self.layers):
            m, where = l.mixer, f"layers[{i}].mixer"
            if l.type == "attention":
                _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ConfigError(f"{where}: heads is no multiple of kv_heads")
                rot = m.get("rot")
                if rot is not None:
                    _need(rot, ("dims", "base"), where + ".rot")
                    if int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= int(m["dim"]):
                        raise ConfigError(f"{where}: rot.dims must be even and at most dim")
                src = m.get("kv_from")
                if src is not None:
                    src = int(src)
                    if not 0 <= src < i or self.layers[src].type != "attention" \
                            or self.layers[src].mixer.get("kv_from") is not None:
                        raise ConfigError(f"{where}: kv_from {src} does not name an earlier attention layer "
                                          f"with keys and values of its own")
                    other = self.layers[src].mixer
                    for key in ("kv_heads", "dim", "vdim"):
                        if int(other[key]) != int(m[key]):
                            raise ConfigError(f"{where}: {key} differs from layer {src}, whose keys and values it reads")
            elif l.type == "delta":
                _need(m, ("heads", "kv_heads", "dim", "vdim", "conv"), where)
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ConfigError(f"{where}: heads is no multiple of kv_heads")
                if int(m["conv"]) < 1:
                    raise ConfigError(f"{where}: a convolution of {m['conv']} taps is not possible")
            else:
                raise ConfigError(f"layers[{i}].type={l.type!r} is not a known mixer; known: attention, delta")
            if l.mlp is not None:
                where = f"layers[{i}].mlp"
                _need(l.mlp, ("kind",), where)
                if l.mlp["kind"] == "dense":
                    _need(l.mlp, ("ff",), where)
                elif l.mlp["kind"] == "moe":
                    _need(l.mlp, ("expert", "router"), where)
                    _need(l.mlp["expert"], ("ff",), where + ".expert")
                    _need(l.mlp["router"], ("experts", "top"), where + ".router")
                    r = self._router(l.mlp)
                    total = r["experts"] + r["identity"]
                    if r["experts"] < 1 or r["identity"] < 0 or r["groups"] < 1 or total % r["groups"]:
                        raise ConfigError(f"{where}.router: {total} router outputs do not form {r['groups']} equal groups")
                    if not 1 <= r["keep"] <= r["groups"]:
                        raise ConfigError(f"{where}.router: groups.keep must be between 1 and groups.count")
                    if not 1 <= r["top"] <= r["keep"] * (total // r["groups"]):
                        raise ConfigError(f"{where}.router: top={r['top']} exceeds the experts of the kept groups")
                else:
                    raise ConfigError(f"{where}.kind={l.mlp['kind']!r} is not supported; known: dense, moe")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": l.type, "mixer": json.loads(json.dumps(l.mixer)),
                        "mlp": json.loads(json.dumps(l.mlp)) if l.mlp is not None else None} for l in self.layers],
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # --------------------------------------------------------------------- plan
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"dim": self.width, "eps": self.norm_eps, "suffix": ""}, name)

    def _mixer(self, l: LoletarLayer) -> PartSpec:
        m = l.mixer
        if l.type == "delta":
            return PartSpec("gated_delta_rule", {
                "hidden_size": self.width, "num_heads": int(m["heads"]), "num_key_heads": int(m["kv_heads"]),
                "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "conv_taps": int(m["conv"]),
                "norm_eps": self.norm_eps, "query_scale": float(int(m["dim"])) ** -0.5,
            }, "mix.")
        rot = m.get("rot")
        if rot is not None and int(rot["dims"]) > 0:
            position = PartSpec("rotary", {"head_dim": int(m["dim"]), "rotary_dim": int(rot["dims"]),
                                           "theta": float(rot["base"]), "pairing": "neighbours",
                                           "table_precision": "float64"})
        else:
            position = PartSpec("none", {})
        return PartSpec("gated_sink_attention", {
            "hidden_size": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
            "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]),
            "qk_norm_eps": self.norm_eps, "sink": 0.0, "gate": "dim", "window": None,
            "own_kv": m.get("kv_from") is None, "position": position,
        }, "mix.")

    def _feed_forward(self, l: LoletarLayer) -> Optional[PartSpec]:
        if l.mlp is None:
            return None
        if l.mlp["kind"] == "dense":
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": int(l.mlp["ff"]),
                                       "names": ("gate", "up", "down")}, "mlp.")
        r = self._router(l.mlp)
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": int(l.mlp["expert"]["ff"]),
            "num_experts": r["experts"], "num_identity": r["identity"], "top": r["top"],
            "groups": r["groups"], "keep_groups": r["keep"], "correction": True,
        }, "mlp.")

    def plan(self) -> ModelPlan:
        layers, order = [], []
        for i, l in enumerate(self.layers):
            ff = self._feed_forward(l)
            norms = (self._norm("norm1"),) if ff is None else (self._norm("norm1"), self._norm("norm2"))
            layers.append(LayerSpec("branch_norm", f"l{i}.", norms, self._mixer(l), ff))
            src = l.mixer.get("kv_from") if l.type == "attention" else None
            order.append(RunEntry(i, reads_cache_of=None if src is None else int(src)))
        plan = ModelPlan(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                             "suffix": "", "scale": self.embedding_scale}, "embed"),
            layers=tuple(layers), order=tuple(order),
            final_norm=self._norm("final.norm"),
            head=PartSpec("lm_head", {"hidden_size": self.width, "vocab_size": self.vocab, "tied_to": None,
                                      "suffix": ""}, "head"),
        )
        plan.validate()
        return plan

    def describe(self) -> dict:
        return self.to_dict()
