"""A plain, slow statement of the Loletar decoder in float64: one function per mechanism.

It shares nothing with the engine: it reads a configuration mapping and a dict of tensors by
name and walks the tokens of ONE sequence.  Recurrent layers go token by token, attention
builds the full score matrix.  The tests compare the engine with it.

    layer:      x <- x + rms(mixer(x)) * w1 ;  x <- x + rms(ff(x)) * w2       (norm on the branch only)
    attention:  q, k per head RMS-normed, the first `rot.dims` dims rotated in neighbouring pairs,
                p_j = exp(s_j) / (1 + sum_j exp(s_j)),  output times sigmoid(W_g x), then W_o
    delta:      q, k, v through a causal per-channel convolution and silu; q, k unit vectors;
                S <- g S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q
    routed ff:  softmax router, choice by score + correction inside the best groups, weights are
                the plain scores; the last `identity` router outputs stand for "the input itself"
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]; the last column multiplies the current token, zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], 0)
    out = torch.zeros_like(x)
    for j in range(K):
        out += padded[j:j + T] * taps[:, j]
    return out


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, D]: dims 2i and 2i+1 (i < dims/2) turn by position * base^(-2i/dims)."""
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=F64)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(F64)[:, None] * freq[None, :]                  # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def attention_keys_values(h, w, pre, m, eps):
    """The keys (normed, rotated) and values a layer writes: [T, G, dim], [T, G, vdim]."""
    T = h.shape[0]
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[pre + "k"].T).view(T, G, D)
    v = (h @ w[pre + "v"].T).view(T, G, Dv)
    k = rms_norm(k, w[pre + "k.norm"], eps)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    k = rotate_pairs(k, torch.arange(T), rot["dims"], rot["base"])
    return k, v


def sink_attention(q, k, v, scale, sink=True):
    """q [T, H, D], k [T, G, D], v [T, G, Dv], causal; with `sink` the denominator holds one more term of
    score 0 that has no value.  Returns [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * scale
        s = s.masked_fill(~causal, float("-inf"))
        mx = s.max(-1, keepdim=True).values
        if sink:
            mx = torch.clamp(mx, min=0.0)
        e = torch.exp(s - mx)
        denom = e.sum(-1, keepdim=True) + (torch.exp(-mx) if sink else 0.0)
        out[:, hd] = (e / denom) @ v[:, g]
    return out


def attention_mixer(h, w, pre, m, eps, kv, sink=True):
    """kv: (keys, values) of this layer or of the layer it borrows them from."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, D)
    q = rms_norm(q, w[pre + "q.norm"], eps)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_pairs(q, torch.arange(T), rot["dims"], rot["base"])
    out = sink_attention(q, kv[0], kv[1], m["scale"], sink)
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    return (out.reshape(T, H * Dv) * gate) @ w[pre + "o"].T


def delta_recurrence(q, k, v, beta, decay, S0=None):
    """q, k [T, G, D] (already unit vectors, q scaled), v [T, H, Dv], beta and decay [T, H]: per head
    S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Returns (o [T, H, Dv], S [H, D, Dv])."""
    T, H, Dv = v.shape
    G, D = q.shape[1], q.shape[2]
    out = torch.zeros(T, H, Dv, dtype=F64)
    S = torch.zeros(H, D, Dv, dtype=F64) if S0 is None else S0.clone()
    for hd in range(H):
        g = hd // (H // G)
        for t in range(T):
            S[hd] = decay[t, hd] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, g])
            S[hd] = S[hd] + torch.outer(k[t, g], u)
            out[t, hd] = S[hd].T @ q[t, g]
    return out, S


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[pre + "q"].T, w[pre + "q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ w[pre + "k"].T, w[pre + "k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ w[pre + "v"].T, w[pre + "v.conv"])).view(T, H, Dv)
    beta = torch.sigmoid(h @ w[pre + "b"].T)                                                   # [T, H]
    decay = torch.exp(-torch.exp(w[pre + "A_log"]) *
                      torch.nn.functional.softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))   # [T, H]
    out, _ = delta_recurrence(unit(q) * D ** -0.5, unit(k), v, beta, decay)
    out = rms_norm(out, w[pre + "norm"], eps)
    gate = silu(h @ w[pre + "g"].T).view(T, H, Dv)
    return (out * gate).reshape(T, H * Dv) @ w[pre + "o"].T


def gated_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(z, correction, r):
    """Router outputs z [T, E] -> chosen expert numbers [T, top] and their weights [T, top]."""
    E = r["experts"] + r.get("identity", 0)
    s = torch.softmax(z, -1)                                          # [T, E]
    choice = s + correction
    groups = r.get("groups") or {"count": 1, "keep": 1}
    n, keep = groups["count"], groups["keep"]
    per = E // n
    best = choice.view(-1, n, per).max(-1).values                     # [T, n]
    kept = best.topk(keep, -1).indices
    allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
    allowed = allowed[:, :, None].expand(-1, -1, per).reshape(-1, E)
    choice = choice.masked_fill(~allowed, float("-inf"))
    chosen = choice.topk(r["top"], -1).indices
    return chosen, s.gather(1, chosen)


def routed_ff(h, w, pre, mlp):
    r = mlp["router"]
    chosen, weight = route(h @ w[pre + "router"].T, w[pre + "correction"], r)
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, p in zip(chosen[t].tolist(), weight[t]):
            if e >= r["experts"]:                                     # an identity expert
                out[t] += p * h[t]
            else:
                x = h[t:t + 1]
                out[t] += p * gated_ff(x, w[f"{pre}e{e}.gate"], w[f"{pre}e{e}.up"], w[f"{pre}e{e}.down"])[0]
    return out


def forward(config: Mapping, weights: Mapping[str, torch.Tensor], tokens: List[int], streams: Optional[list] = None,
            sink: bool = True):
    """Logits [T, vocab] of one sequence; `streams` collects the residual after every layer.  `sink` False
    leaves the extra term out of the softmax (to show that a test would notice)."""
    w: Dict[str, torch.Tensor] = {k: v.to(F64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    kv = {}
    for i, layer in enumerate(config["layers"]):
        pre, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kv[i] = attention_keys_values(x, w, pre, m, eps)
                src = i
            y = attention_mixer(x, w, pre, m, eps, kv[src], sink)
        elif layer["type"] == "delta":
            y = delta_mixer(x, w, pre, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = gated_ff(x, w[f"l{i}.mlp.gate"], w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"])
            else:
                y = routed_ff(x, w, f"l{i}.mlp.", mlp)
            x = x + rms_norm(y, w[f"l{i}.norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
