"""The Vivesun configuration reader, tensor names and the oracle's own mechanisms (no GPU)."""
import copy
import math

import pytest
import torch

import plain_vivesun as plain
import tiny_vivesun as tiny
from vosti_b200.config import ConfigError, known_architectures, model_spec_from_config, model_spec_from_dir
from vosti_b200.config.vivesun import checkpoint_shapes
from vosti_b200.models import build_model, expected_weights


def spec_of(config, rank):
    return model_spec_from_config(config, checkpoint_shapes(config, decay_rank=rank))


def test_registered_beside_the_other_architectures():
    assert {"Vivesun", "Mugizen", "Qwen3ForCausalLM"} <= set(known_architectures())


def test_layers_parts_and_caches():
    spec = spec_of(tiny.A, 3)
    assert [layer.mixer.kind for layer in spec.layers] == ["branches", "gated_delta", "branches", "gated_delta"]
    assert all(layer.arrangement == "pre_norm_stream" for layer in spec.layers) and spec.tie_word_embeddings
    assert [layer.feed_forward is None for layer in spec.layers] == [False, True, False, False]
    assert [layer.token_input["offset"] for layer in spec.layers] == [0, 5, 10, 15]
    left = dict(spec.layers[0].mixer["branches"])["left"]
    assert left["chunk"] == 7 and left["sink_value"] == 0.0 and left["position"]["rotary_dim"] == 24
    assert left["position"]["scaling"] == ("wavelength", 4.0, 1.0, 3.0, 40.0)
    assert dict(spec.layers[2].mixer["branches"])["left"]["position"]["scaling"] is None
    assert spec.layers[2].mixer["scales"] == (1.0, 0.5) and spec.layers[2].mixer["merge"] == "sum"
    delta = spec.layers[1].mixer
    assert delta["decay"] == "head" and delta["gate_activation"] == "silu" and delta["decay_rank"] == 0
    model = build_model(spec)
    caches, states = model.cache_specs()
    assert len(caches) == len(states) == 5                       # four layers and the embedding's last token
    assert [c is not None for c in caches] == [True, False, True, False, False]
    assert states[-1].dtype == torch.int32 and states[-1].shape == (1,)
    assert states[0].shape == (3 * 20 * 20,) and states[1].shape[0] >= 4 * 8 * 12 + (2 * 2 * 8 + 4 * 12)
    without = build_model(spec_of(tiny.B, 2))
    assert all(layer.token_input is None for layer in without.spec.layers)
    assert "side.embed" not in expected_weights(without.spec)


def test_tensor_names_and_shapes():
    names = expected_weights(spec_of(tiny.A, 3))
    assert names["embed"].shape == (211, 72) and names["bigram"].shape == (98, 72) and names["side.embed"].shape == (211, 20)
    assert "head" not in names and names["final.norm"].shape == (72,)
    assert names["l0.norm1"].shape == names["l0.norm2"].shape == (72,) and "l1.norm2" not in names
    assert names["l0.mix.left.q"].shape == (96, 72) and names["l0.mix.left.k"].shape == (48, 72)
    assert names["l0.mix.left.v"].shape == (32, 72) and names["l0.mix.left.o"].shape == (72, 64)
    for key in ("r", "k", "v", "g", "a"):
        assert names[f"l0.mix.right.{key}"].shape == (60, 72)
    assert names["l0.mix.right.a.b"].shape == names["l0.mix.right.w0"].shape == names["l0.mix.right.norm"].shape == (60,)
    assert names["l0.mix.right.w1"].shape == (3, 72) and names["l0.mix.right.w2"].shape == (60, 3)
    assert names["l1.mix.q"].shape == (16, 72) and names["l1.mix.v"].shape == (48, 72) and names["l1.mix.v.conv"].shape == (48, 2)
    assert names["l1.mix.b"].shape == names["l1.mix.a"].shape == (4, 72) and names["l1.mix.dt_bias"].shape == (4,)
    assert names["l1.mix.A_log"].shape == (4,) and names["l1.mix.norm"].shape == (12,) and names["l1.mix.g"].shape == (48, 72)
    assert names["l0.mlp.router"].shape == (5, 72) and names["l0.mlp.e4.up"].shape == (24, 72) and names["l0.mlp.e4.down"].shape == (72, 24)
    assert not any(n.endswith(".gate") and ".mlp." in n for n in names)
    assert names["l3.side.gate"].shape == (5, 72) and names["l3.side.proj"].shape == (72, 5) and names["l3.side.norm"].shape == (72,)


def test_the_rank_comes_from_the_checkpoint(tmp_path):
    with pytest.raises(ConfigError, match="shape of tensor"):
        model_spec_from_config(tiny.A)
    folder = tiny.write_model(tmp_path / "m", tiny.B, 2, 3)
    spec = model_spec_from_dir(folder)
    assert dict(spec.layers[1].mixer["branches"])["right"]["decay_rank"] == 2


@pytest.mark.parametrize("damage,message", [
    (lambda c: c.pop("vocab"), "lacks 'vocab'"),
    (lambda c: c["norm"].pop("eps"), "lacks 'eps'"),
    (lambda c: c["layers"][0].update(type="window"), "'delta' and 'parallel' are known"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), "positive integer"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].pop("base"), "lacks 'base'"),
    (lambda c: c["layers"][0]["mixer"].pop("right_scale"), "lacks 'right_scale'"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "'moe' is known"),
    (lambda c: c["layers"][0]["mlp"]["router"].pop("top"), "lacks 'top'"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "lacks 'conv'"),
    (lambda c: c["embedding"]["bigram"].update(buckets=-3), "positive integer"),
    (lambda c: c["token_side"].pop("dim"), "lacks 'dim'"),
])
def test_missing_or_bad_keys_are_errors(damage, message):
    config = copy.deepcopy(tiny.A)
    damage(config)
    with pytest.raises(ConfigError, match=message):
        spec_of(config, 3)


def test_optional_blocks_may_be_absent():
    config = copy.deepcopy(tiny.A)
    config.pop("token_side")
    config["layers"][0].pop("mlp")
    config["layers"][0]["mixer"]["left"].pop("mask")
    config["layers"][0]["mixer"]["left"]["rot"].pop("scaling")
    config["layers"][2]["mlp"]["router"].pop("scale")
    spec = spec_of(config, 3)
    left = dict(spec.layers[0].mixer["branches"])["left"]
    assert left["chunk"] == 0 and left["position"]["scaling"] is None
    assert spec.layers[0].feed_forward is None and spec.layers[0].token_input is None
    assert spec.layers[2].feed_forward["scale"] == 1.0
    assert "side.embed" not in expected_weights(spec)


def test_part_parameters_are_checked():
    from vosti_b200.config import PartSpec
    from vosti_b200.parts import build_feed_forward, build_mixer, build_position
    with pytest.raises(ConfigError, match="both low-rank pairs or both plain"):
        build_mixer(PartSpec.make("gated_delta", num_heads=2, num_kv_heads=1, head_dim=8, v_head_dim=8, conv_taps=2, eps=1e-5,
                                  decay_rank=0, gate_rank=3), 32, None)
    with pytest.raises(ConfigError, match="a window or a chunk"):
        build_mixer(PartSpec.make("sink_attention", num_heads=2, num_kv_heads=1, head_dim=8, scale=1.0, window=4, chunk=4), 32, None)
    with pytest.raises(ConfigError, match="learned sink or a constant"):
        build_mixer(PartSpec.make("sink_attention", num_heads=2, num_kv_heads=1, head_dim=8, scale=1.0, sink=True, sink_value=0.0), 32, None)
    with pytest.raises(ConfigError, match="route is"):
        build_feed_forward(PartSpec.make("moe", experts=2, top=1, intermediate_size=8, route="sigmoid"), 32)
    with pytest.raises(ConfigError, match="scaling is"):
        build_position(PartSpec.make("rope", theta=10.0, rotary_dim=8, scaling=("linear", 2.0)), 32, 8)
    with pytest.raises(ConfigError, match="one constant per branch"):
        build_mixer(PartSpec.make("branches", merge="sum", scales=(1.0,), branches=(
            ("x", PartSpec.make("general_delta", num_heads=1, head_dim=8, decay_rank=1, eps=1e-5)),
            ("y", PartSpec.make("sink_attention", num_heads=2, num_kv_heads=1, head_dim=8, scale=1.0)))), 32, None)


# ---------------------------------------------------------------- the oracle checks itself
def test_oracle_recurrences_equal_their_definitions_written_out():
    gen = torch.Generator().manual_seed(0)
    T, H, d = 6, 2, 5
    r, k, v = (torch.randn(T, H, d, generator=gen, dtype=torch.float64) for _ in range(3))
    decay, rate = (torch.rand(T, H, d, generator=gen, dtype=torch.float64) for _ in range(2))
    got = plain.general_delta_recurrence(r, k, v, decay, rate)
    for h in range(H):
        S = torch.zeros(d, d, dtype=torch.float64)
        for t in range(T):
            u = k[t, h] / math.sqrt(float(k[t, h] @ k[t, h]) + 1e-6)
            S = torch.diag(decay[t, h]) @ S - torch.outer(rate[t, h] * u, u @ S) + torch.outer(k[t, h], v[t, h])
            assert torch.allclose(got[t, h], S.T @ r[t, h])
    beta, g = torch.rand(T, H, generator=gen, dtype=torch.float64), torch.rand(T, H, generator=gen, dtype=torch.float64)
    got = plain.gated_delta_recurrence(r, k, v, beta, g)
    for h in range(H):
        S = torch.zeros(d, d, dtype=torch.float64)
        for t in range(T):
            S = g[t, h] * S
            S = S + torch.outer(k[t, h], beta[t, h] * (v[t, h] - S.T @ k[t, h]))
            assert torch.allclose(got[t, h], S.T @ r[t, h])


def test_oracle_chunks_are_absolute_and_the_denominator_has_one_added():
    gen = torch.Generator().manual_seed(1)
    T, chunk = 23, 5
    q, k, v = (torch.randn(T, 1, 4, generator=gen, dtype=torch.float64) for _ in range(3))
    whole = plain.chunk_attention(q, k, v, 0.5, chunk)
    for i in range(T):
        lo = i - i % chunk
        s = (k[lo:i + 1, 0] @ q[i, 0]) * 0.5
        w = torch.exp(s) / (1.0 + torch.exp(s).sum())
        assert torch.allclose(whole[i, 0], w @ v[lo:i + 1, 0])
    # a cut sequence that starts in the middle of a chunk keeps the absolute boundaries
    tail = plain.chunk_attention(q[10:], k[10:], v[10:], 0.5, chunk, start=10)
    assert torch.allclose(tail, whole[10:])
    assert plain.pair_rows([3, 4, 4], 7, 2, 5) == [7, (3 * 2 + 4 * 5) % 7, (4 * 2 + 4 * 5) % 7]
