"""The Mugizen configuration reader, run order and tensor names (no GPU)."""
import copy

import pytest

import plain_mugizen as plain
import tiny_mugizen as tiny
from vosti_b200.config import ConfigError, known_architectures, model_spec_from_config, model_spec_from_dir
from vosti_b200.config.mugizen import checkpoint_shapes
from vosti_b200.models import build_model, expected_weights


def spec_of(config, shapes_kw):
    return model_spec_from_config(config, checkpoint_shapes(config, **shapes_kw))


def test_registered_beside_the_other_architectures():
    assert {"Mugizen", "Qwen3ForCausalLM"} <= set(known_architectures())


def test_run_order_follows_the_loop():
    spec = spec_of(tiny.P, tiny.P_SHAPES)
    runs = [(e.layer, e.instance, e.reenter) for e in spec.run_order]
    assert runs == [(0, 0, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (1, 2, True), (2, 2, False),
                    (3, 0, False)]
    assert [(i, enters) for i, _, enters in runs] == plain.run_order(tiny.P)
    model = build_model(spec)
    assert model.cache_layers == [0, 1, 2, 3, 1, 2, 1, 2]          # every pass has a cache and a state of its own
    no_loop = spec_of(tiny.Q, tiny.Q_SHAPES)
    assert [e.layer for e in no_loop.run_order] == [0, 1] and no_loop.reentry is None
    assert "loop.in" not in expected_weights(no_loop)


def test_tensor_names_and_shapes():
    names = expected_weights(spec_of(tiny.P, tiny.P_SHAPES))
    assert names["embed"].shape == (203, 72) and names["head"].shape == (203, 72) and names["loop.in"].shape == (72, 144)
    assert names["final.norm"].shape == (72,) and names["final.norm.b"].shape == (72,) and names["final.norm.alpha"].shape == ()
    assert names["l0.norm1.alpha"].shape == () and names["l0.mix.left.rel"].shape == (9, 4)
    assert names["l0.mix.left.q"].shape == (96, 72) and names["l0.mix.left.k"].shape == (48, 72)
    assert names["l0.mix.left.v"].shape == (32, 72) and names["l0.mix.left.o"].shape == (72, 64)
    assert names["l1.mix.right.q"].shape == (120, 72) and names["l1.mix.right.v.conv"].shape == (60, 2)
    assert names["l1.mix.right.a2"].shape == (120, 5) and names["l1.mix.right.g2"].shape == (60, 3)
    assert names["l1.mix.right.b"].shape == (3, 72) and names["l1.mix.right.norm"].shape == (20,)
    assert names["l0.mix.left.out"].shape == names["l0.mix.right.out"].shape == (72,)
    assert not any(n.startswith("l1.mlp") for n in names)            # a layer without a feed-forward
    assert names["l0.mlp.router"].shape == (5, 72) and names["l0.mlp.e4.down"].shape == (72, 24)
    assert names["l2.mlp.gate"].shape == (80, 72) and names["l2.mlp.down"].shape == (72, 80)


def test_sizes_that_only_tensor_shapes_give(tmp_path):
    with pytest.raises(ConfigError, match="shape of tensor"):
        model_spec_from_config(tiny.P)
    folder = tiny.write_model(tmp_path / "m", tiny.Q, tiny.Q_SHAPES, 3)
    spec = model_spec_from_dir(folder)
    left = dict(spec.layers[0].mixer["branches"])["left"]
    right = dict(spec.layers[1].mixer["branches"])["right"]
    assert left["bias_rows"] == 2 and right["decay_rank"] == 2 and right["gate_rank"] == 9 and right["conv_taps"] == 5


@pytest.mark.parametrize("damage,message", [
    (lambda c: c.pop("loop"), "lacks 'loop'"),
    (lambda c: c["loop"].update(stop=9), "start < stop"),
    (lambda c: c["layers"][0].update(type="serial"), "'parallel' is known"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "'dense' and 'moe'"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "lacks 'scale'"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(conv=0), "positive integer"),
    (lambda c: c["norm"].pop("eps"), "lacks 'eps'"),
    (lambda c: c["layers"][2]["mixer"]["left"].update(heads=3), "multiple"),
])
def test_bad_configurations_are_refused(damage, message):
    config = copy.deepcopy(tiny.P)
    damage(config)
    with pytest.raises(ConfigError, match=message):
        build_model(spec_of(config, tiny.P_SHAPES))
