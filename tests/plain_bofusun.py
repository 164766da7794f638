"""A plain, slow statement of the Bofusun decoder, one function per mechanism.

Whole sequences only, float64 on the CPU, token by token where the design is a
recurrence.  It shares no code with the engine: the tests compare the engine's
kernels, cache and scheduler with what these functions give.  `w` maps checkpoint
names to tensors; `cfg` is the content of config.json.

Notation: T tokens, positions 0..T-1; heads H; d_k / d_v the key and value sizes
of one head.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x over the root of (its mean square + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose stored gain is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain_gain(x, w, eps):
    return unit_rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_leading(x, positions, dims, base):
    """x [T, H, d]: the first `dims` dims of each head turn by position; dim i pairs with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * freq[None, :]                 # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def retention(h, w, p, m, eps):
    """Decayed linear attention without a denominator: per head S <- g S + k v^T, o = S^T q."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    q = rotate_leading(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_leading(k, pos, m["rot"]["dims"], m["rot"]["base"]) * dk ** -0.5
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        g = float(m["decay"][hd])
        for t in range(T):
            S = g * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = unit_rms(out, eps).reshape(T, H * dv)
    return (out * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def short_conv(u, taps_w, bias=None):
    """u [T, C], taps_w [C, K]: y_t = sum_j taps_w[:, j] u_{t-K+1+j}, zeros before the start."""
    T, C = u.shape
    K = taps_w.shape[1]
    y = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(K):
            s = t - K + 1 + j
            if s >= 0:
                y[t] += taps_w[:, j] * u[s]
    return y if bias is None else y + bias


def distance_bucket(n, rows, far):
    """Row of the distance table for a distance n >= 0: exact below rows/2, logarithmic up to `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def gated_window_attention(h, w, p, m):
    """Softmax attention over a window, scores capped by tanh, a learned bias by distance, a gate per head."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.conv"]).view(T, H, dk)
    k = short_conv(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.conv"]).view(T, G, dk)
    v = short_conv(h @ w[p + "v"].T + w[p + "v.b"], w[p + "v.conv"]).view(T, G, dv)
    rel = w[p + "rel"]
    rows = rel.shape[0]
    cap, window = m.get("softcap"), m["mask"]["size"]
    gate = torch.sigmoid(h @ w[p + "g"].T)                           # [T, H]
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        kv = hd // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, kv] @ q[i, hd]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            s = s + torch.stack([rel[distance_bucket(i - j, rows, m["bias_max"]), hd] for j in range(lo, i + 1)])
            out[i, hd] = torch.softmax(s, 0) @ v[lo:i + 1, kv]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def selective_scan(h, w, p, m):
    """Mamba: a diagonal state space per channel whose step size and in/out maps depend on the token."""
    T = h.shape[0]
    inner, n_state, rank = m["inner"], m["state"], m["dt_rank"]
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(short_conv(x, w[p + "conv"], w[p + "conv.b"]))
    proj = x @ w[p + "x"].T
    dt_in, Bm, Cm = proj[:, :rank], proj[:, rank:rank + n_state], proj[:, rank + n_state:]
    dt = torch.nn.functional.softplus(dt_in @ w[p + "dt"].T + w[p + "dt.b"])       # [T, inner]
    A = -torch.exp(w[p + "A_log"])                                                  # [inner, n_state]
    S = torch.zeros(inner, n_state, dtype=F64)
    y = torch.zeros(T, inner, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * Bm[t][None, :]
        y[t] = S @ Cm[t] + w[p + "D"] * x[t]
    return (y * silu(z)) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    left = gated_window_attention(h, w, p + "left.", m["left"])
    right = selective_scan(h, w, p + "right.", m["right"])
    return 0.5 * (norm_plain_gain(left, w[p + "left.out"], eps) + norm_plain_gain(right, w[p + "right.out"], eps))


def squared_relu_ff(h, w, p):
    u = torch.relu(h @ w[p + "up"].T + w[p + "up.b"])
    return (u * u) @ w[p + "down"].T + w[p + "down.b"]


def run_order(cfg):
    """[(layer index, pass number or None if the layer is the first of no pass)] in execution order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def layer(x, w, cfg, i):
    eps = cfg["norm"]["eps"]
    spec, p = cfg["layers"][i], f"l{i}."
    h = norm_around_zero(x, w[p + "norm1"], eps)
    if spec["type"] == "retention":
        y = retention(h, w, p + "mix.", spec["mixer"], eps)
    elif spec["type"] == "parallel":
        y = parallel_mixer(h, w, p + "mix.", spec["mixer"], eps)
    else:
        raise ValueError(spec["type"])
    x = x + norm_around_zero(y, w[p + "norm1b"], eps)
    if spec.get("mlp") is not None:
        y = squared_relu_ff(norm_around_zero(x, w[p + "norm2"], eps), w, p + "mlp.")
        x = x + norm_around_zero(y, w[p + "norm2b"], eps)
    return x


def forward(cfg, w, ids, layers_out=None):
    """Logits [T, vocab] of one sequence.  `layers_out`: a list that receives the stream after every layer run."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = norm_around_zero(w["embed"][torch.tensor(ids)], w["embed.norm"], eps)
    x0 = x
    for i, start_of_pass in run_order(cfg):
        if start_of_pass is not None:
            if start_of_pass > 0:
                x = x + x0
            x = x + w["loop.step"][start_of_pass]
        x = layer(x, w, cfg, i)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_around_zero(x, w["final.norm"], eps) @ w["head"].T
