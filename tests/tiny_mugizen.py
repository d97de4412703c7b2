"""Small Mugizen configurations for the tests, with weights of a size that makes every mechanism
matter (unit-variance activations, biases and sinks of order one), written as a model folder.

P: odd sizes everywhere; key and value widths differ; fewer key/value heads than heads in both
   branches; a layer without a feed-forward; an expert feed-forward whose stacked width is no
   multiple of 16; a loop that starts at the second layer and runs three times; an odd number
   of bias rows; temperatures that change every 5 positions.
Q: no loop; a convolution of one tap (no tail in the state); one expert; two bias rows;
   one head; a key width that needs two lanes per column in the recurrence.
R: attention heads of 64 with equal key and value widths and pages of 16 tokens, which in
   bfloat16 run on the tensor-memory and split-key decode kernels; a loop from the first layer.
"""
import json
from pathlib import Path

import torch

from vosti_b200.config import model_spec_from_config
from vosti_b200.config.mugizen import checkpoint_shapes
from vosti_b200.models import expected_weights
from vosti_b200.weights import write_safetensors


def _left(heads, kv, dim, vdim, scale, far, coef, every):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, bias_max=far, q_temp=dict(coef=coef, every=every))


def _right(heads, kv, dim, vdim, conv):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv)


def _layer(left, right, mlp):
    return dict(type="parallel", mixer=dict(left=left, right=right), mlp=mlp)


P = dict(architecture="Mugizen", vocab=203, width=72, norm=dict(eps=2e-6), loop=dict(start=1, stop=3, times=3), layers=[
    _layer(_left(4, 2, 24, 16, 0.3, 40, 0.7, 5), _right(4, 2, 8, 12, 4),
           dict(kind="moe", expert=dict(ff=24), router=dict(experts=5, top=3))),
    _layer(_left(2, 1, 16, 40, 0.2, 40, 0.7, 5), _right(3, 3, 40, 20, 2), None),
    _layer(_left(4, 2, 24, 16, 0.3, 40, 0.7, 5), _right(4, 2, 8, 12, 4), dict(kind="dense", ff=80)),
    _layer(_left(3, 3, 8, 8, 0.5, 40, 0.7, 5), _right(2, 1, 16, 36, 3),
           dict(kind="moe", expert=dict(ff=32), router=dict(experts=4, top=1))),
])
P_SHAPES = dict(bias_rows=9, decay_rank=5, gate_rank=3)

Q = dict(architecture="Mugizen", vocab=128, width=64, norm=dict(eps=1e-5), loop=None, layers=[
    _layer(_left(2, 2, 32, 32, 0.18, 3, 0.25, 1), _right(1, 1, 48, 48, 1),
           dict(kind="moe", expert=dict(ff=48), router=dict(experts=1, top=1))),
    _layer(_left(1, 1, 64, 16, 0.12, 3, 0.25, 1), _right(2, 2, 16, 70, 5), dict(kind="dense", ff=96)),
])
Q_SHAPES = dict(bias_rows=2, decay_rank=2, gate_rank=9)

R = dict(architecture="Mugizen", vocab=160, width=128, norm=dict(eps=1e-6), loop=dict(start=0, stop=1, times=2), layers=[
    _layer(_left(4, 2, 64, 64, 0.125, 50, 0.3, 16), _right(4, 2, 24, 32, 3),
           dict(kind="moe", expert=dict(ff=32), router=dict(experts=4, top=2))),
    _layer(_left(2, 2, 64, 64, 0.125, 50, 0.3, 16), _right(2, 1, 32, 64, 4), dict(kind="dense", ff=192)),
])
R_SHAPES = dict(bias_rows=8, decay_rank=8, gate_rank=8)

ALL = {"p": (P, P_SHAPES, 11), "q": (Q, Q_SHAPES, 12), "r": (R, R_SHAPES, 13)}
PAGE = {"p": 8, "q": 8, "r": 16}


def draw(name, shape, gen):
    """One tensor by its role, float32 (the caller rounds to bfloat16)."""
    n = lambda std, mean=0.0: mean + std * torch.randn(shape, generator=gen)
    last = name.split(".")[-1]
    if name == "embed":
        return n(1.0)
    if last == "alpha":
        return n(0.1, 0.8)
    if last == "conv":
        return n(0.6)
    if last in ("rel", "sink"):
        return n(1.5)
    if last == "A_log":
        return n(0.7, -0.5)
    if last == "dt_bias":
        return n(1.0)
    if last == "b" and len(shape) == 1:
        return n(0.2)
    if len(shape) == 1:                      # plain weights of norms and branch outputs
        return n(0.2, 1.0)
    if last == "router":
        return n(2.0 / shape[1] ** 0.5)
    return n(1.0 / shape[1] ** 0.5)


def tensors_for(config, shapes_kw, seed):
    spec = model_spec_from_config(config, checkpoint_shapes(config, **shapes_kw))
    gen = torch.Generator().manual_seed(seed)
    return spec, {name: draw(name, tuple(w.shape), gen).to(torch.bfloat16) for name, w in expected_weights(spec).items()}


def write_model(folder, config, shapes_kw, seed):
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    _, tensors = tensors_for(config, shapes_kw, seed)
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt"})
    return str(folder)


def load_plain(folder):
    """config.json and float32 tensors as the plain implementation reads them."""
    from safetensors import safe_open

    config = json.loads((Path(folder) / "config.json").read_text())
    tensors = {}
    with safe_open(str(Path(folder) / "model.safetensors"), framework="pt", device="cpu") as handle:
        for name in handle.keys():
            tensors[name] = handle.get_tensor(name).float()
    return config, tensors
