"""Selective scan (Mamba): a state space per channel whose step size and input and output
maps are made from the token.

    [x | z] = W_in h ;   x = silu(conv(x) + b_conv)                       (causal, per channel, K taps)
    [dt_in | B | C] = W_x x ;   dt = softplus(W_dt dt_in + b_dt) ;   A = -exp(A_log)
    S[c, n] = exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n ;   y_c = sum_n S[c, n] C_n + D_c x_c
    out = W_o (y * silu(z))

The state S [inner, states] is float32 and lives in the request's state slot, and so do the
last K-1 inputs of the convolution.  dt, its softplus, the decays exp(dt A) and the state are
float32; the product W_dt dt_in is written in float32 for that.  W_x is bound as two matrices
(rows for dt_in, rows for B and C) so that each product's output is a matrix of its own.
Tensors: `<name>in`, `conv`, `conv.b`, `x`, `dt`, `dt.b`, `A_log`, `D`, `o`.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, StateSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, register_part
from .linear import Linear


class SelectiveScan(Part):
    out_buffer = "branch"

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inner = int(p["inner_size"])
        self.states = int(p["state_size"])
        self.rank = int(p["dt_rank"])
        self.taps = int(p.get("conv_taps", 1))
        self.w_in = self.w_dtin = self.w_bc = self.w_dt = self.o = None
        self.conv = self.conv_bias = self.dt_bias = self.A_log = self.D = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n, I, S, R = self.name, self.inner, self.states, self.rank
        return {
            n + "in": ParamSpec((2 * I, self.hidden)),
            n + "conv": ParamSpec((I, self.taps), role="gain", init="around_zero"),
            n + "conv.b": ParamSpec((I,), role="gain", init="normal"),
            n + "x": ParamSpec((R + 2 * S, I)),
            n + "dt": ParamSpec((I, R)),
            n + "dt.b": ParamSpec((I,), role="gain", init="uniform", bounds=(-4.0, -1.0)),
            n + "A_log": ParamSpec((I, S), role="gain", init="uniform", bounds=(0.0, 2.5)),
            n + "D": ParamSpec((I,), role="gain", init="gain"),
            n + "o": ParamSpec((self.hidden, I)),
        }

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        self.w_in = Linear(tensors[n + "in"])
        wx = tensors[n + "x"]
        self.w_dtin, self.w_bc = Linear(wx[:self.rank]), Linear(wx[self.rank:])
        self.w_dt = Linear(tensors[n + "dt"])
        self.o = Linear(tensors[n + "o"])
        self.conv, self.conv_bias = tensors[n + "conv"], tensors[n + "conv.b"]
        self.dt_bias, self.A_log, self.D = tensors[n + "dt.b"], tensors[n + "A_log"], tensors[n + "D"]

    def cache_needs(self) -> CacheNeeds:
        state = {"ssm": StateSpec((self.inner, self.states), torch.float32)}
        if self.taps > 1:
            state["conv"] = StateSpec((self.taps - 1, self.inner), torch.float32)
        return CacheNeeds(state=state)

    def streamed_weights(self):
        return [self.w_in.weight, self.o.weight]

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        N, I = x.shape[0], self.inner
        xz = self.w_in(ctx, x, "ss_xz")
        xc = ctx.buffers.take("ss_x", N, (I,), ctx.dtype)
        tail = cache.state("conv") if self.taps > 1 else None
        ops.short_conv(xz, None, self.conv, self.conv_bias, True, tail, ctx.token_rows, ctx.positions, [(0, I, xc)])
        if tail is not None:
            ops.short_conv_tail(tail, xz, None, self.taps, ctx.seq_starts, ctx.seq_rows)
        dt_in = self.w_dtin(ctx, xc, "ss_dtin")
        bc = self.w_bc(ctx, xc, "ss_bc")
        dt_raw = self.w_dt(ctx, dt_in, "ss_dt", out="float32")
        y = ctx.buffers.take("ss_y", N, (I,), ctx.dtype)
        scratch = None
        if not ctx.all_decode and N > 128 * ctx.num_seqs:
            # few requests with long portions: scratch lets the kernel run segments of the prompt in parallel
            size = ops.selective_scan_scratch_size(N, ctx.num_seqs, I, self.states)
            if size <= (1 << 28):
                scratch = ctx.buffers.take_flat("ss_scratch", size, torch.float32)
        ops.selective_scan(y, xc, xz[:, I:], dt_raw, self.dt_bias, bc, self.A_log, self.D, cache.state("ssm"),
                           ctx.seq_starts, ctx.seq_rows, scratch=scratch)
        return Branch(self.o(ctx, y, self.out_buffer, out="partial"))


register_part("mixer", "selective_scan", SelectiveScan)
