"""Small Vivesun configurations for the tests, with weights of a size that makes every mechanism
matter (unit-variance activations, biases of order one), written as a model folder.

A: odd sizes everywhere; parallel and delta layers alternating, a parallel layer first; fewer
   key/value heads than heads in both kinds; key and value widths that differ; a layer without a
   feed-forward; a rotation of the whole head in one layer and of two elements in another; one
   rotation without frequency scaling; chunks of 7 and 20 positions; a feed-forward that uses all
   its experts; multipliers whose products pass 2^31.
B: no per-layer token input; one expert; a convolution of one tap (no tail in the state); one
   head; a chunk of one position (a query sees itself only); a key width that needs two lanes per
   column in the recurrences.
D: gated-delta layers only (no paged cache at all), sizes that are no multiple of 4, one layer
   without a feed-forward, a token input of one element.
C: attention heads of 64 with equal key and value widths and pages of 16 tokens (the sizes that
   the tensor-core attention kernels take in bfloat16); two parallel layers sharing a page group.
"""
import json
from pathlib import Path

import torch

from vosti_b200.config import model_spec_from_config
from vosti_b200.config.vivesun import checkpoint_shapes
from vosti_b200.models import expected_weights
from vosti_b200.weights import write_safetensors


def _rot(base, dims, scaling=None):
    return dict(base=base, dims=dims, scaling=scaling)


def _scaling(factor, low, high, original):
    return dict(factor=factor, low=low, high=high, original=original)


def _left(heads, kv, dim, vdim, scale, chunk, rot):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, mask=dict(size=chunk), rot=rot)


def _parallel(left, right_heads, right_dim, cl, cr, mlp):
    return dict(type="parallel", mixer=dict(left=left, right=dict(heads=right_heads, dim=right_dim), left_scale=cl,
                                            right_scale=cr), mlp=mlp)


def _delta(heads, kv, dim, vdim, conv, mlp):
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv), mlp=mlp)


def _moe(experts, top, ff, scale):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=scale))


A = dict(architecture="Vivesun", vocab=211, width=72, norm=dict(eps=2e-6), token_side=dict(dim=5),
         embedding=dict(bigram=dict(buckets=97, mul_prev=20000003, mul_cur=15000007)), layers=[
    _parallel(_left(4, 2, 24, 16, 0.3, 7, _rot(100.0, 24, _scaling(4.0, 1.0, 3.0, 40))), 3, 20, 0.6, 1.2, _moe(5, 3, 24, 1.5)),
    _delta(4, 2, 8, 12, 2, None),
    _parallel(_left(2, 1, 16, 40, 0.2, 20, _rot(5000.0, 2)), 2, 40, 1.0, 0.5, _moe(4, 4, 32, 0.7)),
    _delta(3, 3, 40, 20, 4, _moe(6, 1, 16, 2.0)),
])
B = dict(architecture="Vivesun", vocab=128, width=64, norm=dict(eps=1e-5), token_side=None,
         embedding=dict(bigram=dict(buckets=31, mul_prev=1, mul_cur=1)), layers=[
    _delta(1, 1, 48, 48, 1, _moe(1, 1, 48, 1.0)),
    _parallel(_left(1, 1, 32, 32, 0.18, 1, _rot(10000.0, 8, _scaling(2.0, 0.5, 2.0, 16))), 1, 48, 0.9, 0.9, _moe(3, 2, 40, 1.0)),
])
C = dict(architecture="Vivesun", vocab=160, width=128, norm=dict(eps=1e-6), token_side=dict(dim=8),
         embedding=dict(bigram=dict(buckets=509, mul_prev=31, mul_cur=17)), layers=[
    _parallel(_left(4, 2, 64, 64, 0.125, 48, _rot(10000.0, 32, _scaling(8.0, 1.0, 4.0, 64))), 2, 32, 0.7, 1.3, _moe(4, 2, 32, 2.5)),
    _delta(4, 2, 24, 32, 3, _moe(4, 2, 32, 1.0)),
    _parallel(_left(2, 2, 64, 64, 0.125, 33, _rot(50000.0, 64)), 2, 16, 1.1, 0.4, None),
])
D = dict(architecture="Vivesun", vocab=67, width=50, norm=dict(eps=1e-5), token_side=dict(dim=1),
         embedding=dict(bigram=dict(buckets=5, mul_prev=3, mul_cur=2)), layers=[
    _delta(2, 1, 5, 3, 3, _moe(3, 2, 7, 1.0)),
    _delta(3, 3, 6, 9, 2, None),
])
ALL = {"a": (A, 3, 21), "b": (B, 2, 22), "c": (C, 8, 23), "d": (D, 1, 24)}      # config, rank of the decay pair, seed
PAGE = {"a": 8, "b": 8, "c": 16, "d": 4}


def draw(name, shape, gen):
    """One tensor by its role, float32 (the caller rounds to bfloat16)."""
    n = lambda std, mean=0.0: mean + std * torch.randn(shape, generator=gen)
    last = name.split(".")[-1]
    if name in ("embed", "bigram"):
        return n(0.7)
    if name == "side.embed":
        return n(1.0)
    if last == "conv":
        return n(0.6)
    if last == "A_log":
        return n(0.7, -0.5)
    if last in ("dt_bias", "w0"):
        return n(1.0)
    if name.endswith("a.b"):
        return n(1.0)
    if last in ("norm1", "norm2") or name == "final.norm":        # stored around zero
        return n(0.2)
    if len(shape) == 1:                      # plain weights of unit norms
        return n(0.2, 1.0)
    if last == "router":
        return n(2.0 / shape[1] ** 0.5)
    if last == "w2":
        return n(2.0 / shape[1] ** 0.5)
    return n(1.0 / shape[1] ** 0.5)


def tensors_for(config, rank, seed):
    spec = model_spec_from_config(config, checkpoint_shapes(config, decay_rank=rank))
    gen = torch.Generator().manual_seed(seed)
    return spec, {name: draw(name, tuple(w.shape), gen).to(torch.bfloat16) for name, w in expected_weights(spec).items()}


def write_model(folder, config, rank, seed):
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    _, tensors = tensors_for(config, rank, seed)
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt"})
    return str(folder)
