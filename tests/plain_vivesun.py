"""Plain, slow implementation of the Vivesun design: whole sequences on the CPU, no cache, no
batching, one function per mechanism, token by token where the design is a recurrence. It
shares no code with the package and is the oracle the GPU tests compare the engine with.

Notation. x: residual stream [T, width]; h: a sublayer's normed input; p: position of a token,
from 0. A weight W stored [out, in] acts as x @ W.T. `cfg` is the model's config.json as a
dict; `w` maps tensor names to tensors of the working type (float64 by default).

    embedding:  x = embed[tok] + bigram[(prev * mul_prev + tok * mul_cur) % buckets], the table's
                last row for a sequence's first token
    layer:      x <- x + mixer(norm1(x));  x <- x + ff(norm2(x));  x <- x + side(x, tok)
    norm:       x / sqrt(mean(x^2) + eps) * (1 + weight)
    side:       y = P (gelu_tanh(G x) * e_tok[layer's slice]);  y / rms(y) * weight
    'delta':    gated delta rule, scalar decay per head, short convolutions on q, k, v
    'parallel': c_left * attention + c_right * generalized delta rule
    attention:  partial rotation with scaled frequencies, keys of the query's own chunk only,
                softmax whose denominator has one added
    ff:         top-k of a softmax router over small GELU feed-forwards, renormed and scaled
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    return unit_rms(x, eps) * (1.0 + weight)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ---------------------------------------------------------------- embedding
def pair_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every token: hashed from (previous, current); a sequence's
    first token takes row `buckets`."""
    rows = [buckets]
    for i in range(1, len(tokens)):
        rows.append((tokens[i - 1] * mul_prev + tokens[i] * mul_cur) % buckets)
    return rows


def embed(tokens, w, cfg):
    b = cfg["embedding"]["bigram"]
    rows = pair_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"])
    return w["embed"][tokens] + w["bigram"][rows]


# ---------------------------------------------------------------- rotation
def rotary_frequencies(dims, base, scaling):
    """f_i = base^(-2i/dims) for i < dims/2, then rescaled by wavelength: short waves stay,
    long ones are divided by `factor`, those between are blended."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
            wave = 2.0 * math.pi / f
            if wave < original / high:
                pass
            elif wave > original / low:
                f = f / factor
            else:
                s = (original / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate(x, positions, freqs, angle_dtype=torch.float32):
    """x [T, heads, d]; the first 2 * len(freqs) elements of each head turn in pairs
    (i, i + len(freqs)) by the angle p * f_i; the angle is formed in `angle_dtype`."""
    half = len(freqs)
    f = torch.tensor(freqs, dtype=torch.float64).to(angle_dtype)
    angle = (torch.tensor(positions, dtype=angle_dtype)[:, None] * f[None, :]).to(x.dtype)
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], dim=-1)


# ---------------------------------------------------------------- attention
def chunk_attention(q, k, v, scale, chunk, start=0):
    """q [T, H, d], k [T, G, d], v [T, G, dv] at positions start .. start + T - 1. Chunk boundaries
    are the multiples of `chunk` in absolute positions; a query sees the keys j <= i that lie
    between the last boundary at or before it and itself. The weights are
    exp(s_j) / (1 + sum exp(s_j))."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for i in range(T):
        lo = ((start + i) // chunk) * chunk - start
        lo = max(lo, 0)
        for head in range(H):
            g = head // (H // G)
            s = (k[lo:i + 1, g] @ q[i, head]) * scale
            top = max(float(s.max()), 0.0)
            e = torch.exp(s - top)
            out[i, head] = (e / (e.sum() + math.exp(-top))) @ v[lo:i + 1, g]
    return out


def attention_branch(h, w, prefix, m, angle_dtype=torch.float32):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[prefix + "q"].T).view(T, H, d)
    k = (h @ w[prefix + "k"].T).view(T, G, d)
    v = (h @ w[prefix + "v"].T).view(T, G, dv)
    rot = m["rot"]
    freqs = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    positions = list(range(T))
    q, k = rotate(q, positions, freqs, angle_dtype), rotate(k, positions, freqs, angle_dtype)
    o = chunk_attention(q, k, v, m["scale"], m["mask"]["size"])
    return o.reshape(T, H * dv) @ w[prefix + "o"].T


# ---------------------------------------------------------------- recurrences
def general_delta_recurrence(r, k, v, decay, rate):
    """r, k, v, decay, rate [T, H, d]. With u = k / sqrt(|k|^2 + 1e-6):
    S <- diag(decay) S - (rate * u) (u^T S) + k v^T, both first terms from the old S; o = S^T r."""
    T, H, d = r.shape
    S = torch.zeros(H, d, d, dtype=r.dtype)
    out = torch.zeros(T, H, d, dtype=r.dtype)
    for t in range(T):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum(-1, keepdim=True) + 1e-6)
        seen = torch.einsum("hi,hij->hj", u, S)
        S = decay[t][:, :, None] * S - (rate[t] * u)[:, :, None] * seen[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hij,hi->hj", S, r[t])
    return out


def general_delta_branch(h, w, prefix, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = (h @ w[prefix + "r"].T).view(T, H, d)
    k = (h @ w[prefix + "k"].T).view(T, H, d)
    v = (h @ w[prefix + "v"].T).view(T, H, d)
    inner = torch.tanh(h @ w[prefix + "w1"].T) @ w[prefix + "w2"].T + w[prefix + "w0"]
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(inner)).view(T, H, d)
    rate = torch.sigmoid(h @ w[prefix + "a"].T + w[prefix + "a.b"]).view(T, H, d)
    o = general_delta_recurrence(r, k, v, decay, rate)
    o = unit_rms(o, eps).reshape(T, H * d) * w[prefix + "norm"] * torch.sigmoid(h @ w[prefix + "g"].T)
    return o @ w[prefix + "o"].T


def short_conv_silu(x, taps_w):
    """Causal convolution per channel over time, zeros before the start, then SiLU.
    x [T, C]; taps_w [C, taps], the last column multiplies the current token."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros(T, C, dtype=x.dtype)
    for i in range(taps):
        y = y + padded[i:i + T] * taps_w[:, i]
    return silu(y)


def gated_delta_recurrence(q, k, v, beta, g):
    """q, k [T, H, d]; v [T, H, dv]; beta, g [T, H].
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, d = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, d, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hij,hi->hj", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hij,hi->hj", S, q[t])
    return out


def gated_delta_mixer(h, w, prefix, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ w[prefix + "q"].T, w[prefix + "q.conv"]).view(T, G, d)
    k = short_conv_silu(h @ w[prefix + "k"].T, w[prefix + "k.conv"]).view(T, G, d)
    v = short_conv_silu(h @ w[prefix + "v"].T, w[prefix + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(H // G, dim=1), k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ w[prefix + "b"].T)
    g = torch.exp(-torch.exp(w[prefix + "A_log"]) * softplus(h @ w[prefix + "a"].T + w[prefix + "dt_bias"]))
    o = gated_delta_recurrence(q, k, v, beta, g)
    o = unit_rms(o, eps) * w[prefix + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ w[prefix + "g"].T)
    return o @ w[prefix + "o"].T


def parallel_mixer(h, w, prefix, m, eps, angle_dtype=torch.float32):
    left = attention_branch(h, w, prefix + "left.", m["left"], angle_dtype)
    right = general_delta_branch(h, w, prefix + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ---------------------------------------------------------------- feed-forward
def expert_mixture(h, w, prefix, m):
    experts, top, scale = m["router"]["experts"], m["router"]["top"], m["router"]["scale"]
    scores = torch.softmax(h @ w[prefix + "router"].T, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        best = torch.topk(scores[t], top)
        weights = best.values / (best.values.sum() + 1e-20) * scale
        for e, c in zip(best.indices.tolist(), weights):
            out[t] += c * (gelu_erf(h[t] @ w[f"{prefix}e{e}.up"].T) @ w[f"{prefix}e{e}.down"].T)
    return out


def token_side(x, tokens, w, prefix, layer, dim, eps):
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[prefix + "gate"].T) * e) @ w[prefix + "proj"].T
    return unit_rms(y, eps) * w[prefix + "norm"]


# ---------------------------------------------------------------- the model
def forward(cfg, w, tokens, angle_dtype=torch.float32, keep_layers=False):
    """Logits [T, vocab] of a whole sequence (and the stream after every layer if asked)."""
    eps = cfg["norm"]["eps"]
    tokens = list(tokens)
    x = embed(tokens, w, cfg)
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "delta":
            x = x + gated_delta_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            x = x + parallel_mixer(h, w, p + "mix.", layer["mixer"], eps, angle_dtype)
        else:
            raise ValueError(layer["type"])
        if layer["mlp"] is not None:
            x = x + expert_mixture(offset_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
        if cfg.get("token_side"):
            x = x + token_side(x, tokens, w, p + "side.", i, cfg["token_side"]["dim"], eps)
        streams.append(x)
    logits = offset_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(streams)) if keep_layers else logits


# ---------------------------------------------------------------- reading a model folder
def read_safetensors(path, dtype=torch.float64):
    """name -> tensor, floating tensors in `dtype`, integers as they are. Written from the
    format's description: 8 bytes of header length, a JSON header, raw little-endian data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16, "I64": torch.int64}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return out


def load_model(folder, dtype=torch.float64):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors", dtype)
