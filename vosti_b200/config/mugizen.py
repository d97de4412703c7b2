"""The Mugizen design, read from its own config.json.

A decoder whose layers are parallel blocks (one Dynamic Tanh norm feeding a mixer and a
feed-forward, both added to a float32 residual stream); the mixer is two branches side by
side, softmax attention with a sink, a distance bias and a query temperature beside a gated
delta rule; the feed-forward is dense or a mixture of experts, or absent; a span of layers may
run several times in a row with the same weights (each pass with caches and states of its own),
the stream re-entering every pass through a product with the embedding output beside it.

Keys (a missing one is an error; nothing has a default):

    architecture  "Mugizen"
    vocab, width
    norm.eps                       epsilon of every root-mean-square division
    layers[i].type                 "parallel"
    layers[i].mixer.left           heads, kv_heads, dim, vdim, scale, bias_max,
                                   q_temp.coef, q_temp.every
    layers[i].mixer.right          heads, kv_heads, dim, vdim, conv
    layers[i].mlp                  null | {kind: "dense", ff} |
                                   {kind: "moe", expert.ff, router.experts, router.top}
    loop                           null | {start, stop, times}

Sizes that the config does not name (rows of the bias table, ranks of the low-rank pairs) are
read from the checkpoint's tensor shapes when a model folder is given (`shapes`).
"""
from __future__ import annotations

from typing import Any, Mapping, Optional

from .schema import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

ARCHITECTURE = "Mugizen"
MAX_POSITIONS = 1 << 30        # the design sets no limit; the cache pool does


def _need(block: Mapping[str, Any], key: str, where: str):
    if not isinstance(block, Mapping) or key not in block:
        raise ConfigError(f"Mugizen config: {where} lacks '{key}'")
    return block[key]


def _positive_int(block, key, where) -> int:
    value = _need(block, key, where)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"Mugizen config: {where}.{key} must be a positive integer, got {value!r}")
    return value


def _number(block, key, where) -> float:
    value = _need(block, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or value != value:
        raise ConfigError(f"Mugizen config: {where}.{key} must be a number, got {value!r}")
    return float(value)


def _shape(shapes, name: str, axis: int, where: str) -> int:
    if shapes is None or name not in shapes:
        raise ConfigError(f"Mugizen config: {where} is given by the shape of tensor '{name}', which is not at hand")
    return int(shapes[name][axis])


def _mixer(i: int, block: Mapping[str, Any], eps: float, shapes) -> PartSpec:
    where = f"layers[{i}].mixer"
    left, right = _need(block, "left", where), _need(block, "right", where)
    lw, rw = where + ".left", where + ".right"
    temp = _need(left, "q_temp", lw)
    attention = PartSpec.make(
        "sink_attention", num_heads=_positive_int(left, "heads", lw), num_kv_heads=_positive_int(left, "kv_heads", lw),
        head_dim=_positive_int(left, "dim", lw), v_head_dim=_positive_int(left, "vdim", lw),
        scale=_number(left, "scale", lw), window=0, sink=True,
        bias_rows=_shape(shapes, f"l{i}.mix.left.rel", 0, lw + " (rows of the distance bias)"),
        bias_far=_positive_int(left, "bias_max", lw),
        q_temp_coef=_number(temp, "coef", lw + ".q_temp"), q_temp_every=_positive_int(temp, "every", lw + ".q_temp"))
    delta = PartSpec.make(
        "gated_delta", num_heads=_positive_int(right, "heads", rw), num_kv_heads=_positive_int(right, "kv_heads", rw),
        head_dim=_positive_int(right, "dim", rw), v_head_dim=_positive_int(right, "vdim", rw),
        conv_taps=_positive_int(right, "conv", rw), eps=eps,
        decay_rank=_shape(shapes, f"l{i}.mix.right.a1", 0, rw + " (rank of the decay pair)"),
        gate_rank=_shape(shapes, f"l{i}.mix.right.g1", 0, rw + " (rank of the gate pair)"))
    return PartSpec.make("branches", eps=eps, branches=(("left", attention), ("right", delta)))


def _feed_forward(i: int, block: Optional[Mapping[str, Any]]) -> Optional[PartSpec]:
    if block is None:
        return None
    where = f"layers[{i}].mlp"
    kind = _need(block, "kind", where)
    if kind == "dense":
        return PartSpec.make("swiglu", intermediate_size=_positive_int(block, "ff", where),
                             tensor_names=("gate", "up", "down"), float32_out=True)
    if kind == "moe":
        router = _need(block, "router", where)
        return PartSpec.make("moe", experts=_positive_int(router, "experts", where + ".router"),
                             top=_positive_int(router, "top", where + ".router"),
                             intermediate_size=_positive_int(_need(block, "expert", where), "ff", where + ".expert"),
                             float32_out=True)
    raise ConfigError(f"Mugizen config: {where}.kind is {kind!r}; 'dense' and 'moe' are known")


def spec_from_config(raw: Mapping[str, Any], shapes: Optional[Mapping[str, tuple]] = None) -> ModelSpec:
    if not isinstance(raw, Mapping) or raw.get("architecture") != ARCHITECTURE:
        raise ConfigError("Mugizen config: 'architecture' must be 'Mugizen'")
    width, vocab = _positive_int(raw, "width", "config"), _positive_int(raw, "vocab", "config")
    eps = _number(_need(raw, "norm", "config"), "eps", "norm")
    norm = PartSpec.make("dyt", bias=True, bias_name="b")
    layers = _need(raw, "layers", "config")
    if not isinstance(layers, list) or not layers:
        raise ConfigError("Mugizen config: 'layers' must be a nonempty list")
    names = (("norm", "norm1"), ("mixer", "mix"), ("feed_forward", "mlp"))
    specs = []
    for i, layer in enumerate(layers):
        kind = _need(layer, "type", f"layers[{i}]")
        if kind != "parallel":
            raise ConfigError(f"Mugizen config: layers[{i}].type is {kind!r}; 'parallel' is known")
        specs.append(LayerSpec(mixer=_mixer(i, _need(layer, "mixer", f"layers[{i}]"), eps, shapes),
                               feed_forward=_feed_forward(i, _need(layer, "mlp", f"layers[{i}]")),
                               norm=norm, position=None, arrangement="parallel", names=names))
    n = len(specs)
    loop = _need(raw, "loop", "config")
    if loop is None:
        order = [RunEntry(i) for i in range(n)]
    else:
        start = _need(loop, "start", "loop")
        stop, times = _positive_int(loop, "stop", "loop"), _positive_int(loop, "times", "loop")
        if isinstance(start, bool) or not isinstance(start, int) or not 0 <= start < stop <= n:
            raise ConfigError(f"Mugizen config: loop must satisfy 0 <= start < stop <= {n} layers")
        order = [RunEntry(i) for i in range(start)]
        for run in range(times):
            order += [RunEntry(i, instance=run, reenter=(i == start)) for i in range(start, stop)]
        order += [RunEntry(i) for i in range(stop, n)]
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab, max_positions=MAX_POSITIONS,
        layers=tuple(specs), run_order=tuple(order), final_norm=norm, tie_word_embeddings=False,
        embed_name="embed", final_norm_name="final.norm", lm_head_name="head", layer_prefix="l{i}.",
        reentry=PartSpec.make("concat_linear") if loop is not None else None, reentry_name="loop.in")


def checkpoint_shapes(raw: Mapping[str, Any], *, bias_rows: int, decay_rank: int, gate_rank: int) -> dict:
    """The tensor shapes that carry the sizes a Mugizen config.json does not name, for making a
    random-weights model of `raw`: the same three numbers for every layer."""
    width = raw["width"]
    shapes = {}
    for i, layer in enumerate(raw["layers"]):
        shapes[f"l{i}.mix.left.rel"] = (bias_rows, layer["mixer"]["left"]["heads"])
        shapes[f"l{i}.mix.right.a1"] = (decay_rank, width)
        shapes[f"l{i}.mix.right.g1"] = (gate_rank, width)
    return shapes
