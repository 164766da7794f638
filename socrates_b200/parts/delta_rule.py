"""Gated delta rule: a recurrent mixer with a matrix state per head that forgets by a learned,
input-dependent decay and writes by correcting what it already holds along the new key.

    q, k, v = silu(conv(W_q x)), silu(conv(W_k x)), silu(conv(W_v x))     causal conv per channel, `conv_taps` taps
    q, k: G heads of `key_dim`, v: H heads of `value_dim`; value head h uses q/k head h // (H / G)
    q = unit(q) * key_dim^-1/2 ,  k = unit(k)                             unit(x) = x / sqrt(sum(x^2) + 1e-6)
    beta = sigmoid(W_b x) ,  g = exp(-exp(A_log) * softplus(W_a x + dt_bias))        one of each per head
    S <- g S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q      (the read sees the token's own write)
    y = o / sqrt(mean(o^2) + eps) * w * silu(W_g x) ,  out = W_o concat_h(y)

The state S [H, key_dim, value_dim] is float32 and lives in the request's state slot together with
the last `conv_taps - 1` inputs of the convolutions, so prompts may arrive in portions and requests
decode side by side.  Unit norms, beta, the decay, the recurrence and the output norm are float32 in
both engines.  All six projections are one matrix product; the convolution with its activation is
the engine's short-convolution kernel; the recurrence is one kernel and the head norm with the
gate a small second one.
Tensors: `<name>q`, `q.conv`, `k`, `k.conv`, `v`, `v.conv`, `b`, `a`, `A_log`, `dt_bias`, `norm`, `g`, `o`.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, StateSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, register_part
from .linear import Linear


class GatedDeltaRule(Part):
    out_buffer = "branch"

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p["num_key_heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        self.taps = int(p.get("conv_taps", 1))
        self.eps = float(p["norm_eps"])
        self.q_scale = float(p.get("query_scale", self.dk ** -0.5))
        if self.H % self.G:
            raise ValueError(f"{self.H} value heads are no multiple of {self.G} key heads")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"{self.taps} convolution taps; the kernel takes 1 to 16")
        if not (1 <= self.dk <= 256 and 1 <= self.dv <= 1024):
            raise ValueError(f"head sizes {self.dk} (keys, at most 256) and {self.dv} (values, at most 1024)")
        self.Cqk, self.Cv = self.G * self.dk, self.H * self.dv
        self.C = 2 * self.Cqk + self.Cv                      # channels that pass the convolution
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.conv = self.A_log = self.dt_bias = self.norm_w = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n, H = self.name, self.H
        out: Dict[str, ParamSpec] = {}
        for x, c in (("q", self.Cqk), ("k", self.Cqk), ("v", self.Cv)):
            out[n + x] = ParamSpec((c, self.hidden))
            out[n + x + ".conv"] = ParamSpec((c, self.taps), role="gain", init="uniform", bounds=(-0.5, 0.5))
        out[n + "g"] = ParamSpec((self.Cv, self.hidden))
        out[n + "b"] = ParamSpec((H, self.hidden))
        out[n + "a"] = ParamSpec((H, self.hidden))
        out[n + "A_log"] = ParamSpec((H,), role="gain", init="uniform", bounds=(-3.0, 0.5))
        out[n + "dt_bias"] = ParamSpec((H,), role="gain", init="uniform", bounds=(-2.0, 1.0))
        out[n + "norm"] = ParamSpec((self.dv,), role="gain", init="gain")
        out[n + "o"] = ParamSpec((self.hidden, self.Cv))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        self.proj = Linear(torch.cat([tensors[n + x] for x in ("q", "k", "v", "g", "b", "a")], dim=0))
        self.o = Linear(tensors[n + "o"])
        self.conv = torch.cat([tensors[n + x + ".conv"] for x in ("q", "k", "v")], dim=0).contiguous()
        self.A_log, self.dt_bias, self.norm_w = tensors[n + "A_log"], tensors[n + "dt_bias"], tensors[n + "norm"]

    def cache_needs(self) -> CacheNeeds:
        state = {"S": StateSpec((self.H, self.dk, self.dv), torch.float32)}
        if self.taps > 1:
            state["conv"] = StateSpec((self.taps - 1, self.C), torch.float32)
        return CacheNeeds(state=state)

    def streamed_weights(self):
        return [self.proj.weight, self.o.weight]

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        N, C = x.shape[0], self.C
        proj = self.proj(ctx, x, "dr_proj")
        conv = ctx.buffers.take("dr_conv", N, (C,), ctx.dtype)
        tail = cache.state("conv") if self.taps > 1 else None
        ops.short_conv(proj, None, self.conv, None, True, tail, ctx.token_rows, ctx.positions, [(0, C, conv)])
        if tail is not None:
            ops.short_conv_tail(tail, proj, None, self.taps, ctx.seq_starts, ctx.seq_rows)
        y = ctx.buffers.take("dr_y", N, (self.Cv,), ctx.dtype)
        raw = ctx.buffers.take("dr_raw", N, (self.Cv,), torch.float32)
        ops.delta_rule(y, conv, (0, self.Cqk, 2 * self.Cqk), proj, (C, C + self.Cv, C + self.Cv + self.H),
                       self.A_log, self.dt_bias, self.norm_w, cache.state("S"), ctx.seq_starts, ctx.seq_rows,
                       self.H, self.G, self.dk, self.dv, self.eps, self.q_scale, scratch=raw)
        return Branch(self.o(ctx, y, self.out_buffer, out="partial"))


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
