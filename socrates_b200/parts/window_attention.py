"""Grouped-query softmax attention over a sliding window with capped scores, a learned
bias by distance, a short convolution on q, k and v, and a gate per head.  No rotation:
positions enter through the distance bias alone.

    q, k, v = conv(W_q x + b_q), conv(W_k x + b_k), conv(W_v x + b_v)    (causal, per channel, K taps)
    s_ij = (q_i . k_j) * scale ;  s_ij = cap * tanh(s_ij / cap) ;  s_ij += rel[bucket(i - j), h]
    keys 0 <= i - j < window ;  o_i = softmax_j(s_ij) v_j * sigmoid(W_g x_i)_h ;  out = W_o concat_h(o)
    bucket(n) = n                                                          for n < B/2
              = min(B - 1, B/2 + floor(log(n / (B/2)) / log(far / (B/2)) * (B - B/2)))   otherwise
with B the rows of the table `rel` [B, heads] (read from the tensor's shape) and `far` a constant.

Keys have `key_dim` dims and values `value_dim`; the convolved k and v go to the row's pages
(a windowed page group: pages behind the window are given back), the last K-1 projected values
of every sequence live in a state slot, and the bucket function is turned into a table by
distance once, on the host, in double precision.  The four projections are one matrix product.
Tensors: `<name>q`, `q.b`, `q.conv`, the same for k and v, `rel`, `g`, `o`.
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

from ..cache.manager import CacheNeeds, PagedKVSpec, StateSpec
from ..kernels import ops
from .base import Branch, ParamSpec, Part, register_part
from .linear import Linear


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of a [rows, heads] bias table for a distance n >= 0: one row per distance below rows/2,
    then rows spaced evenly in log(distance) up to `far`, the last row for everything beyond."""
    half = rows // 2
    if n < half or half == 0:
        return min(n, rows - 1)
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def bias_by_distance(rel: torch.Tensor, far: float, window: Optional[int]) -> torch.Tensor:
    """float32 [heads, L]: the bias of every distance 0..L-1; L covers the window, or reaches the
    distance from which the bucket no longer changes."""
    rows = rel.shape[0]
    L = int(math.ceil(far)) + 1
    if window:
        L = min(L, int(window))
    idx = torch.tensor([distance_bucket(n, rows, far) for n in range(L)], dtype=torch.long, device=rel.device)
    return rel.float().index_select(0, idx).t().contiguous()


class WindowBiasAttention(Part):
    out_buffer = "branch"

    def __init__(self, spec, name):
        super().__init__(spec, name)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        self.taps = int(p.get("conv_taps", 1))
        self.scale = float(p["scale"])
        self.softcap = float(p.get("softcap") or 0.0)
        self.window: Optional[int] = p.get("window")
        self.bias_far = float(p["bias_far"])
        self.bias_rows = int(p.get("bias_rows", 32))        # used for random weights only
        if self.H % self.G:
            raise ValueError(f"{self.H} query heads are no multiple of {self.G} KV heads")
        self.Cq, self.Ck, self.Cv = self.H * self.dk, self.G * self.dk, self.G * self.dv
        self.C = self.Cq + self.Ck + self.Cv
        self.qkvg: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.in_bias = self.conv = self.dist_bias = None

    def parameters(self) -> Dict[str, ParamSpec]:
        n = self.name
        out: Dict[str, ParamSpec] = {}
        for x, c in (("q", self.Cq), ("k", self.Ck), ("v", self.Cv)):
            out[n + x] = ParamSpec((c, self.hidden))
            out[n + x + ".b"] = ParamSpec((c,), role="gain", init="normal")
            out[n + x + ".conv"] = ParamSpec((c, self.taps), role="gain", init="around_zero")
        out[n + "rel"] = ParamSpec((-1, self.H), role="gain", init="around_zero",
                                   default_shape=(self.bias_rows, self.H))
        out[n + "g"] = ParamSpec((self.H, self.hidden))
        out[n + "o"] = ParamSpec((self.hidden, self.H * self.dv))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        n = self.name
        self.qkvg = Linear(torch.cat([tensors[n + x] for x in ("q", "k", "v", "g")], dim=0))
        self.o = Linear(tensors[n + "o"])
        self.in_bias = torch.cat([tensors[n + x + ".b"] for x in ("q", "k", "v")]).contiguous()
        self.conv = torch.cat([tensors[n + x + ".conv"] for x in ("q", "k", "v")], dim=0).contiguous()
        self.dist_bias = bias_by_distance(tensors[n + "rel"], self.bias_far, self.window)

    def cache_needs(self) -> CacheNeeds:
        paged = PagedKVSpec(self.G, self.dk, self.window, None if self.dv == self.dk else self.dv)
        state = {"conv": StateSpec((self.taps - 1, self.C), torch.float32)} if self.taps > 1 else None
        return CacheNeeds(paged=paged, state=state)

    def streamed_weights(self):
        return [self.qkvg.weight, self.o.weight]

    def partitions(self, ctx, N: int, max_len: int) -> int:
        """Into how many shares each token's visible keys are cut: with few tokens (a decode step) one block
        per (token, KV head) leaves the GPU idle, so the keys are shared out over about four blocks an SM, at
        least 64 keys a share, at most 16 shares.  A function of the token count and of limits alone (a
        recorded graph stays valid); it changes the order of additions, nothing else."""
        span = min(self.window or max_len, max_len)
        blocks = max(1, N * self.G)
        return max(1, min(16, (4 * ctx.num_sms) // blocks, -(-span // 64)))

    def forward(self, ctx, x: torch.Tensor, cache) -> Branch:
        N = x.shape[0]
        qkvg = self.qkvg(ctx, x, "wa_qkvg")
        q = ctx.buffers.take("wa_q", N, (self.Cq,), ctx.dtype)
        k_pool, v_pool = cache.pools()
        table = cache.block_table()
        tail = cache.state("conv") if self.taps > 1 else None
        ops.short_conv(qkvg, self.in_bias, self.conv, None, False, tail, ctx.token_rows, ctx.positions,
                       [(0, self.Cq, q), (self.Cq, self.Cq + self.Ck, k_pool), (self.Cq + self.Ck, self.C, v_pool)],
                       table)
        if tail is not None:
            ops.short_conv_tail(tail, qkvg, self.in_bias, self.taps, ctx.seq_starts, ctx.seq_rows)
        attn = ctx.buffers.take("wa_attn", N, (self.H * self.dv,), ctx.dtype)
        gate = qkvg[:, self.C:self.C + self.H]
        if (not ctx.all_decode and N >= 4 * ctx.num_seqs
                and ops.attention_bias_tile_supports(self.H, self.G, self.dk, self.dv, ctx.dtype)):
            # prompt portions: a tile of a request's consecutive tokens per block shares the keys it reads
            ops.attention_bias_tile(attn, q, k_pool, v_pool, table, ctx.seq_starts, ctx.seq_rows, ctx.seq_first_pos,
                                    self.H, self.scale, self.window or 0, self.softcap, self.dist_bias, gate=gate)
            return Branch(self.o(ctx, attn, self.out_buffer, out="partial"))
        NP, part_o, part_ml = self.partitions(ctx, N, cache.manager.max_len), None, None
        if NP > 1:
            part_o = ctx.buffers.take_flat("attn_part_o", N * self.H * NP * self.dv, torch.float32)
            part_ml = ctx.buffers.take_flat("attn_part_ml", N * self.H * NP * 2, torch.float32)
        ops.attention_bias(attn, q, k_pool, v_pool, table, ctx.token_rows, ctx.positions, self.H, self.scale,
                           self.window or 0, self.softcap, self.dist_bias, gate=gate,
                           num_partitions=NP, part_o=part_o, part_ml=part_ml)
        return Branch(self.o(ctx, attn, self.out_buffer, out="partial"))


register_part("mixer", "window_bias_attention", WindowBiasAttention)
