"""Plain, slow implementation of the Mugizen design: whole sequences on the CPU in float32,
no cache, no batching, one function per mechanism. It shares no code with the package and
is the oracle the GPU tests compare the engine with.

Notation. x: residual stream [T, width]; h: a layer's normed input; p: position of a token,
from 0. A weight W stored [out, in] acts as x @ W.T. `cfg` is the model's config.json as a
dict; `w` maps tensor names to float32 tensors.

    layer:      h = dyt(x);  x <- x + (mixer(h) + ff(h))
    dyt:        tanh(alpha x) * weight + bias
    mixer:      (unit_rms(left(h)) * w_left + unit_rms(right(h)) * w_right) / 2
    left:       softmax attention without rotation: query scaled by a slowly growing
                temperature, a learned bias per (distance bucket, head), a per-head sink
                logit in the denominator
    right:      gated delta rule with one decay per (head, key channel), short causal
                convolutions on q, k, v, output gate and per-head unit-rms norm
    ff:         SiLU-gated, dense or a top-k mixture of experts
    loop:       layers start..stop-1 run `times` times; before each pass x <- W_in [x; x0]
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dyt(x, weight, bias, alpha):
    return torch.tanh(alpha * x) * weight + bias


def distance_bucket(n: int, rows: int, far: int) -> int:
    """Row of the bias table for distance n >= 0: exact below rows // 2, then logarithmic
    steps that reach the last row at distance `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def sink_attention(h, w, prefix, m):
    """The left branch over a whole sequence. m: its block of the config."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[prefix + "q"].T).view(T, H, dk)
    k = (h @ w[prefix + "k"].T).view(T, G, dk)
    v = (h @ w[prefix + "v"].T).view(T, G, dv)
    temp = torch.tensor([query_temperature(p, m["q_temp"]["coef"], m["q_temp"]["every"]) for p in range(T)])
    q = q * temp[:, None, None]
    rel, sink = w[prefix + "rel"], w[prefix + "sink"]
    by_distance = torch.stack([rel[distance_bucket(n, rel.shape[0], m["bias_max"])] for n in range(T)])   # [T, H]
    out = torch.zeros(T, H, dv)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            scores = (k[: i + 1, g] @ q[i, head]) * m["scale"]
            scores = scores + by_distance[i - torch.arange(i + 1), head]
            top = max(float(scores.max()), float(sink[head]))
            e = torch.exp(scores - top)
            denom = e.sum() + math.exp(float(sink[head]) - top)
            out[i, head] = (e / denom) @ v[: i + 1, g]
    return out.reshape(T, H * dv) @ w[prefix + "o"].T


def short_conv_silu(x, taps_w):
    """Causal convolution per channel over time, zeros before the start, then SiLU.
    x [T, C]; taps_w [C, taps], the last column multiplies the current token."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C), x], 0)
    y = torch.zeros(T, C)
    for i in range(taps):
        y = y + padded[i: i + T] * taps_w[:, i]
    return F.silu(y)


def gated_delta(h, w, prefix, m, eps, state=None):
    """The right branch over a whole sequence, token by token. Returns the output and the
    final state S [heads, dim, vdim]."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ w[prefix + "q"].T, w[prefix + "q.conv"]).view(T, G, dk)
    k = short_conv_silu(h @ w[prefix + "k"].T, w[prefix + "k.conv"]).view(T, G, dk)
    v = short_conv_silu(h @ w[prefix + "v"].T, w[prefix + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[prefix + "b"].T)                                   # [T, H]
    rate = (h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "dt_bias"]
    decay = torch.exp(-torch.exp(w[prefix + "A_log"])[None, :, None] * F.softplus(rate).view(T, H, dk))
    gate = torch.sigmoid((h @ w[prefix + "g1"].T) @ w[prefix + "g2"].T).view(T, H, dv)
    S = torch.zeros(H, dk, dv) if state is None else state.clone()
    out = torch.zeros(T, H, dv)
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            S[head] = decay[t, head][:, None] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, g])
            S[head] = S[head] + torch.outer(k[t, g], u)
            out[t, head] = S[head].T @ q[t, g]
    out = unit_rms(out, eps) * w[prefix + "norm"] * gate
    return out.reshape(T, H * dv) @ w[prefix + "o"].T, S


def parallel_mixer(h, w, prefix, m, eps):
    left = sink_attention(h, w, prefix + "left.", m["left"])
    right, _ = gated_delta(h, w, prefix + "right.", m["right"], eps)
    return 0.5 * (unit_rms(left, eps) * w[prefix + "left.out"] + unit_rms(right, eps) * w[prefix + "right.out"])


def gated_ff(h, w, prefix):
    return (F.silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def expert_mixture(h, w, prefix, m):
    """Per token: the `top` experts with the largest router logits, weighted by the softmax
    over those logits only."""
    logits = h @ w[prefix + "router"].T
    top = m["router"]["top"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        values, chosen = torch.topk(logits[t], top)
        weights = torch.softmax(values, -1)
        for weight, e in zip(weights, chosen.tolist()):
            out[t] = out[t] + weight * gated_ff(h[t: t + 1], w, f"{prefix}e{e}.")[0]
    return out


def feed_forward(h, w, prefix, m):
    if m is None:
        return torch.zeros_like(h)
    if m["kind"] == "dense":
        return gated_ff(h, w, prefix)
    if m["kind"] == "moe":
        return expert_mixture(h, w, prefix, m)
    raise ValueError(m["kind"])


def layer(x, w, index, layer_cfg, eps):
    p = f"l{index}."
    if layer_cfg["type"] != "parallel":
        raise ValueError(layer_cfg["type"])
    h = dyt(x, w[p + "norm1"], w[p + "norm1.b"], w[p + "norm1.alpha"])
    return x + (parallel_mixer(h, w, p + "mix.", layer_cfg["mixer"], eps) + feed_forward(h, w, p + "mlp.", layer_cfg["mlp"]))


def run_order(cfg):
    """(layer index, whether a pass of the loop starts here) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and the stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x, streams = x0, []
    for index, enters in run_order(cfg):
        if enters:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T
        x = layer(x, w, index, cfg["layers"][index], eps)
        streams.append(x)
    final = dyt(x, w["final.norm"], w["final.norm.b"], w["final.norm.alpha"])
    logits = final @ w["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits
