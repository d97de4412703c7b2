"""The Vivesun design, read from its own config.json.

A pre-norm decoder over a float32 residual stream. The embedding adds a row hashed from the
token and the one before it; every layer is mixer, mixture-of-experts feed-forward and a
per-layer token input (a gate from the stream picks from a small vector that belongs to the
token id); norms are root-mean-square norms whose weight is stored around zero; the head is the
embedding table. Two kinds of layer, in any order:

  "delta"     a gated delta rule with one decay per head, short convolutions on q, k, v and a
              SiLU output gate;
  "parallel"  two mixers side by side on the same input, added with one constant each: softmax
              attention (partial rotation with wavelength-scaled frequencies, keys of the query's
              own chunk of positions only, one added to the softmax denominator) and a generalized
              delta rule with a decay and a removal rate per (head, key channel).

Keys (a missing one is an error, except the blocks marked "optional", which may be absent or
null and then switch their mechanism off):

    architecture  "Vivesun"
    vocab, width
    norm.eps                       epsilon of every root-mean-square division
    embedding.bigram               buckets, mul_prev, mul_cur
    token_side                     optional: {dim}
    layers[i].type                 "delta" | "parallel"
    layers[i].mixer   (delta)      heads, kv_heads, dim, vdim, conv
    layers[i].mixer   (parallel)   left_scale, right_scale,
                                   left: heads, kv_heads, dim, vdim, scale, mask (optional: size),
                                         rot.base, rot.dims, rot.scaling (optional: factor, low, high, original)
                                   right: heads, dim
    layers[i].mlp                  optional: {kind: "moe", expert.ff, router.experts, router.top,
                                   router.scale (optional: 1)}

The rank of the generalized rule's decay pair is the first extent of `l<i>.mix.right.w1` in the
checkpoint (`shapes`).
"""
from __future__ import annotations

from typing import Any, Mapping, Optional

from .schema import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

ARCHITECTURE = "Vivesun"
MAX_POSITIONS = 1 << 30        # the design sets no limit (angles are formed from the position); the cache pool does


def _need(block: Mapping[str, Any], key: str, where: str):
    if not isinstance(block, Mapping) or key not in block:
        raise ConfigError(f"Vivesun config: {where} lacks '{key}'")
    return block[key]


def _positive_int(block, key, where) -> int:
    value = _need(block, key, where)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"Vivesun config: {where}.{key} must be a positive integer, got {value!r}")
    return value


def _number(block, key, where) -> float:
    value = _need(block, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or value != value:
        raise ConfigError(f"Vivesun config: {where}.{key} must be a number, got {value!r}")
    return float(value)


def _shape(shapes, name: str, axis: int, where: str) -> int:
    if shapes is None or name not in shapes:
        raise ConfigError(f"Vivesun config: {where} is given by the shape of tensor '{name}', which is not at hand")
    return int(shapes[name][axis])


def _delta(i: int, block: Mapping[str, Any], eps: float) -> PartSpec:
    where = f"layers[{i}].mixer"
    return PartSpec.make(
        "gated_delta", num_heads=_positive_int(block, "heads", where), num_kv_heads=_positive_int(block, "kv_heads", where),
        head_dim=_positive_int(block, "dim", where), v_head_dim=_positive_int(block, "vdim", where),
        conv_taps=_positive_int(block, "conv", where), eps=eps, decay="head", decay_rank=0, gate_rank=0,
        gate_activation="silu")


def _rotation(rot: Mapping[str, Any], where: str) -> PartSpec:
    scaling = rot.get("scaling")
    if scaling is not None:
        sw = where + ".scaling"
        scaling = ("wavelength", _number(scaling, "factor", sw), _number(scaling, "low", sw), _number(scaling, "high", sw),
                   _number(scaling, "original", sw))
    return PartSpec.make("rope", theta=_number(rot, "base", where), rotary_dim=_positive_int(rot, "dims", where),
                         scaling=scaling, max_positions=0)


def _parallel(i: int, block: Mapping[str, Any], eps: float, shapes) -> PartSpec:
    where = f"layers[{i}].mixer"
    left, right = _need(block, "left", where), _need(block, "right", where)
    lw, rw = where + ".left", where + ".right"
    attention = PartSpec.make(
        "sink_attention", num_heads=_positive_int(left, "heads", lw), num_kv_heads=_positive_int(left, "kv_heads", lw),
        head_dim=_positive_int(left, "dim", lw), v_head_dim=_positive_int(left, "vdim", lw),
        scale=_number(left, "scale", lw), window=0,
        chunk=0 if left.get("mask") is None else _positive_int(left["mask"], "size", lw + ".mask"),
        sink=False, sink_value=0.0, position=_rotation(_need(left, "rot", lw), lw + ".rot"))
    general = PartSpec.make(
        "general_delta", num_heads=_positive_int(right, "heads", rw), head_dim=_positive_int(right, "dim", rw), eps=eps,
        decay_rank=_shape(shapes, f"l{i}.mix.right.w1", 0, rw + " (rank of the decay pair)"))
    return PartSpec.make("branches", merge="sum", scales=(_number(block, "left_scale", where), _number(block, "right_scale", where)),
                         branches=(("left", attention), ("right", general)))


def _feed_forward(i: int, block: Optional[Mapping[str, Any]]) -> Optional[PartSpec]:
    if block is None:
        return None
    where = f"layers[{i}].mlp"
    kind = _need(block, "kind", where)
    if kind != "moe":
        raise ConfigError(f"Vivesun config: {where}.kind is {kind!r}; 'moe' is known")
    router = _need(block, "router", where)
    return PartSpec.make("moe", experts=_positive_int(router, "experts", where + ".router"),
                         top=_positive_int(router, "top", where + ".router"),
                         intermediate_size=_positive_int(_need(block, "expert", where), "ff", where + ".expert"),
                         gated=False, route="softmax_renorm",
                         scale=_number(router, "scale", where + ".router") if "scale" in router else 1.0,
                         float32_out=True)


def spec_from_config(raw: Mapping[str, Any], shapes: Optional[Mapping[str, tuple]] = None) -> ModelSpec:
    if not isinstance(raw, Mapping) or raw.get("architecture") != ARCHITECTURE:
        raise ConfigError("Vivesun config: 'architecture' must be 'Vivesun'")
    width, vocab = _positive_int(raw, "width", "config"), _positive_int(raw, "vocab", "config")
    eps = _number(_need(raw, "norm", "config"), "eps", "norm")
    norm = PartSpec.make("rms_stream", eps=eps, unit_offset=True)
    pairs = _need(_need(raw, "embedding", "config"), "bigram", "embedding")
    side = raw.get("token_side")
    side_dim = 0 if side is None else _positive_int(side, "dim", "token_side")
    layers = _need(raw, "layers", "config")
    if not isinstance(layers, list) or not layers:
        raise ConfigError("Vivesun config: 'layers' must be a nonempty list")
    names = (("input_norm", "norm1"), ("post_norm", "norm2"), ("mixer", "mix"), ("feed_forward", "mlp"), ("token_input", "side"))
    specs = []
    for i, layer in enumerate(layers):
        kind = _need(layer, "type", f"layers[{i}]")
        mixer = _need(layer, "mixer", f"layers[{i}]")
        if kind == "delta":
            mixer = _delta(i, mixer, eps)
        elif kind == "parallel":
            mixer = _parallel(i, mixer, eps, shapes)
        else:
            raise ConfigError(f"Vivesun config: layers[{i}].type is {kind!r}; 'delta' and 'parallel' are known")
        token_input = PartSpec.make("gated_table", dim=side_dim, offset=i * side_dim, eps=eps) if side_dim else None
        specs.append(LayerSpec(mixer=mixer, feed_forward=_feed_forward(i, layer.get("mlp")), norm=norm,
                               position=None, arrangement="pre_norm_stream", names=names, token_input=token_input))
    embedding = PartSpec.make(
        "pair_hash", buckets=_positive_int(pairs, "buckets", "embedding.bigram"),
        mul_prev=_positive_int(pairs, "mul_prev", "embedding.bigram"), mul_cur=_positive_int(pairs, "mul_cur", "embedding.bigram"),
        side_width=side_dim * len(specs), names=(("pairs", "bigram"), ("side", "side.embed")))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab, max_positions=MAX_POSITIONS,
        layers=tuple(specs), run_order=tuple(RunEntry(i) for i in range(len(specs))), final_norm=norm,
        tie_word_embeddings=True, embed_name="embed", final_norm_name="final.norm", lm_head_name="head",
        layer_prefix="l{i}.", embedding=embedding)


def checkpoint_shapes(raw: Mapping[str, Any], *, decay_rank: int) -> dict:
    """The tensor shapes that carry the size a Vivesun config.json does not name, for making a
    random-weights model of `raw`: the same rank for every parallel layer."""
    return {f"l{i}.mix.right.w1": (decay_rank, raw["width"]) for i, layer in enumerate(raw["layers"])
            if layer["type"] == "parallel"}
