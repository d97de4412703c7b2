"""The Mugizen design on the GPU against the plain implementation (tests/plain_mugizen.py).

Mechanisms alone (norm, sink attention, gated delta rule, expert feed-forward, branch merge,
re-entry), then whole models of two small configurations: whole prompts, prefill against
token-by-token decoding, portions down to two tokens, unequal requests in one batch against
each alone, pages and state slots used again, long decoding, and greedy generation through
`Engine` (scheduler, CUDA graphs, asynchronous scheduling, preemption).

Exactness is tested in float32 (differences of rounding order only). bfloat16 serving is
compared with the float32 oracle row by row with a bound on the typical error, because a
router's close call may send a token to another expert there.
"""
import math

import pytest
import torch

import plain_mugizen as plain
import tiny_mugizen as tiny
from gpu_util import Harness
from vosti_b200 import Engine, ops
from vosti_b200.config import PartSpec
from vosti_b200.engine.batch import StepEntry
from vosti_b200.engine.runner import ModelRunner
from vosti_b200.parts import build_feed_forward, build_mixer, build_norm, build_reentry

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32 = dict(atol=3e-4, rtol=3e-4)


def rounded(*shape, gen, std=1.0, mean=0.0):
    """Random values that bfloat16 holds exactly, as float32 on the CPU."""
    return (mean + std * torch.randn(tuple(shape), generator=gen)).to(torch.bfloat16).float()


def give(part, W, dtype):
    """Hand a part its tensors (keys of `weight_specs`) on the device in the serving layout."""
    assert set(W) == set(part.weight_specs()), (sorted(W), sorted(part.weight_specs()))
    store = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    part.load({k: v.to(DEV, store).contiguous() for k, v in W.items()}, dtype)
    part.setup(torch.device(DEV), dtype)


class Ctx:
    def __init__(self, dtype):
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.dtype = dtype


# ---------------------------------------------------------------- norm, merge, re-entry
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dynamic_tanh_with_deferred_sum(dtype):
    gen = torch.Generator().manual_seed(1)
    width, rows = 200, 7
    norm = build_norm(PartSpec.make("dyt", bias=True, bias_name="b"), width)
    W = {"weight": rounded(width, gen=gen, std=0.3, mean=1.0), "b": rounded(width, gen=gen, std=0.3),
         "alpha": rounded(gen=gen, std=0.1, mean=0.6)}
    give(norm, W, dtype)
    ctx = Ctx(dtype)
    stream, a, b = rounded(rows, width, gen=gen), rounded(rows, width, gen=gen), rounded(rows, width, gen=gen)
    kept = stream.clone().to(DEV)
    got, new_stream = norm.forward_add(ctx, ops.DeferredSum(a.to(DEV), b.to(DEV, dtype)), kept)
    total = stream + a + b
    assert new_stream.dtype == torch.float32 and torch.allclose(new_stream.cpu(), total, atol=1e-6)
    want = plain.dyt(total, W["weight"], W["b"], W["alpha"])
    assert got.dtype == dtype
    assert torch.allclose(got.float().cpu(), want, atol=1e-5 if dtype == torch.float32 else 2e-2)
    # the stream's first norm: nothing to add to, and the stream is created in float32
    got, created = norm.forward_add(ctx, a.to(DEV, dtype), None)
    assert created.dtype == torch.float32 and torch.equal(created.cpu(), a)
    assert torch.allclose(got.float().cpu(), plain.dyt(a, W["weight"], W["b"], W["alpha"]),
                          atol=1e-5 if dtype == torch.float32 else 2e-2)


def test_branch_merge_and_reentry():
    gen = torch.Generator().manual_seed(2)
    rows, width, eps = 5, 136, 1e-3
    xs = [rounded(rows, width, gen=gen, std=s) for s in (0.01, 3.0, 1.0)]
    ws = [rounded(width, gen=gen, std=0.2, mean=1.0) for _ in xs]
    got = ops.branch_merge([x.to(DEV) for x in xs], [w.to(DEV) for w in ws], eps)
    want = sum(plain.unit_rms(x, eps) * w for x, w in zip(xs, ws)) / 3
    assert torch.allclose(got.cpu(), want, atol=1e-5)
    for dtype in (torch.float32, torch.bfloat16):
        part = build_reentry(PartSpec.make("concat_linear"), width)
        W = {"weight": rounded(width, 2 * width, gen=gen, std=0.1)}
        give(part, W, dtype)
        first = rounded(rows, width, gen=gen)
        hidden, stream = part.forward(Ctx(dtype), ops.DeferredSum(xs[1].to(DEV), xs[2].to(DEV)), xs[0].to(DEV),
                                      first.to(DEV, dtype))
        want = torch.cat([xs[0] + xs[1] + xs[2], first], -1) @ W["weight"].T
        assert hidden is None and stream.dtype == torch.float32
        assert torch.allclose(stream.cpu(), want, atol=2e-5 if dtype == torch.float32 else 0.15)


# ---------------------------------------------------------------- sink attention alone
def attention_case(heads, kv, dk, dv, rows, far, coef, every, sink=True, scale=0.25):
    spec = PartSpec.make("sink_attention", num_heads=heads, num_kv_heads=kv, head_dim=dk, v_head_dim=dv, scale=scale,
                         window=0, sink=sink, bias_rows=rows, bias_far=far, q_temp_coef=coef, q_temp_every=every)
    block = dict(heads=heads, kv_heads=kv, dim=dk, vdim=dv, scale=scale, bias_max=far, q_temp=dict(coef=coef, every=every))
    return spec, block


def attention_weights(mixer, width, gen, spread=1.0):
    W = {}
    for key, w in mixer.weight_specs().items():
        std = 1.5 if key in ("rel", "sink") else spread / math.sqrt(w.shape[-1])
        W[key] = rounded(*w.shape, gen=gen, std=std)
    return W


def run_in_portions(mixer, harness, x, sizes, dtype, request="s"):
    outs, at = [], 0
    for size in sizes:
        ctx = harness.context([StepEntry(request, [0] * size)])
        outs.append(mixer.forward(ctx, x[at:at + size].to(DEV, dtype), harness.cache.layer_caches[0]).float().cpu())
        at += size
    assert at == x.shape[0]
    return torch.cat(outs)


@pytest.mark.parametrize("heads,kv,dk,dv", [(4, 2, 24, 40), (3, 3, 16, 8), (6, 1, 72, 136)])
def test_sink_attention_in_portions_against_plain(heads, kv, dk, dv):
    """Page borders (pages of 8), every bucket edge of the bias (distances 0..far and beyond),
    temperatures that change every 7 positions, portions down to one token."""
    gen = torch.Generator().manual_seed(heads * 100 + dk)
    width, T = 88, 75
    spec, block = attention_case(heads, kv, dk, dv, rows=10, far=33, coef=0.6, every=7)
    mixer = build_mixer(spec, width, None)
    W = attention_weights(mixer, width, gen, spread=2.0)
    give(mixer, W, torch.float32)
    harness = Harness([mixer.cache_spec()], [None], torch.float32, num_pages=16, page_size=8)
    x = rounded(T, width, gen=gen)
    got = run_in_portions(mixer, harness, x, (9, 1, 1, 30, 2, 7, 1, 24), torch.float32)
    want = plain.sink_attention(x, {"p." + k: v for k, v in W.items()}, "p.", block)
    assert torch.allclose(got, want, **F32)
    assert harness.status.item() == 0


def test_sink_attention_parts_that_can_be_left_out():
    """No sink, no bias table, no temperature: the same as a sink that weighs nothing, a table
    of zeros and a coefficient of zero."""
    gen = torch.Generator().manual_seed(5)
    width, T = 64, 40
    spec = PartSpec.make("sink_attention", num_heads=2, num_kv_heads=1, head_dim=32, v_head_dim=16, scale=0.2)
    mixer = build_mixer(spec, width, None)
    assert set(mixer.weight_specs()) == {"q", "k", "v", "o"}
    W = attention_weights(mixer, width, gen, spread=2.0)
    give(mixer, W, torch.float32)
    harness = Harness([mixer.cache_spec()], [None], torch.float32, num_pages=8, page_size=8)
    x = rounded(T, width, gen=gen)
    got = run_in_portions(mixer, harness, x, (33, 7), torch.float32)
    block = dict(heads=2, kv_heads=1, dim=32, vdim=16, scale=0.2, bias_max=5, q_temp=dict(coef=0.0, every=1))
    full = dict(W, rel=torch.zeros(4, 2), sink=torch.full((2,), -1e30))
    want = plain.sink_attention(x, {"p." + k: v for k, v in full.items()}, "p.", block)
    assert torch.allclose(got, want, **F32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk", [32, 64])
@pytest.mark.parametrize("far_key", [0, 7, 8, 15, 16, 200, 255, 256])
def test_a_far_key_that_stands_out_is_found(dtype, far_key, dk):
    """One key among hundreds matches the last query strongly: the output is that key's value.
    The key sits at the first position, at page borders (pages of 8 or 16 and multiples), far
    back. Head size 64 in bfloat16 takes the tensor-memory kernel for the prompt and the
    split-key decode kernel for the last token; everything else the CUDA-core kernel."""
    width, T, heads, dv = 2 * dk, 300, 2, dk
    gen = torch.Generator().manual_seed(far_key)
    spec, block = attention_case(heads, heads, dk, dv, rows=6, far=20, coef=0.0, every=1, scale=1.0)
    mixer = build_mixer(spec, width, None)
    eye = torch.eye(width)
    W = {"q": eye.clone(), "k": eye.clone(), "v": eye.clone(), "o": eye.clone(),
         "rel": torch.zeros(6, heads), "sink": torch.zeros(heads)}
    give(mixer, W, dtype)
    x = rounded(T, width, gen=gen, std=0.05)
    mark = torch.zeros(width)
    mark[:dk] = 1.0                                    # head 0: score dk between the marked rows
    x[far_key] += mark
    x[T - 1] += mark
    harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=40, page_size=8 if dk == 32 else 16)
    got = run_in_portions(mixer, harness, x, (T - 1, 1), dtype)
    want = plain.sink_attention(x, {"p." + k: v for k, v in W.items()}, "p.", block)
    assert torch.allclose(got, want, atol=2e-4 if dtype == torch.float32 else 3e-2)
    assert (got[T - 1, :dv] - x[far_key, :dv]).abs().max() < 0.2       # head 0 returns the marked key's value (about 1)


@pytest.mark.parametrize("heads,kv,d", [(4, 2, 64), (8, 2, 128), (2, 2, 128)])
def test_sink_attention_on_the_tensor_memory_kernel(heads, kv, d):
    """bfloat16, equal key and value widths of 64 or 128: long rows run on the tensor-memory
    kernel, requests that bring up to four tokens beside them on the split-key decode kernels. The bias
    changes within the first 90 positions back, so tiles near the diagonal look it up and tiles
    beyond add its last value; two requests of one batch, one long and one short row."""
    gen = torch.Generator().manual_seed(d + heads)
    width, T = 96, 600
    spec, block = attention_case(heads, kv, d, d, rows=12, far=90, coef=0.4, every=50, scale=d ** -0.5)
    mixer = build_mixer(spec, width, None)
    W = attention_weights(mixer, width, gen, spread=1.5)
    give(mixer, W, torch.bfloat16)
    harness = Harness([mixer.cache_spec()], [None], torch.bfloat16, num_pages=90, page_size=16)
    xa, xb = rounded(T, width, gen=gen), rounded(300, width, gen=gen)
    named = {"p." + k: v for k, v in W.items()}
    want_a, want_b = plain.sink_attention(xa, named, "p.", block), plain.sink_attention(xb, named, "p.", block)
    cache = harness.cache.layer_caches[0]
    got_a, got_b, at_a, at_b = [], [], 0, 0
    for na, nb in ((130, 1), (3, 200), (1, 1), (401, 2), (65, 96)):
        ctx = harness.context([StepEntry("a", [0] * na), StepEntry("b", [0] * nb)])
        x = torch.cat([xa[at_a:at_a + na], xb[at_b:at_b + nb]]).to(DEV, torch.bfloat16)
        out = mixer.forward(ctx, x, cache).float().cpu()
        got_a.append(out[:na])
        got_b.append(out[na:])
        at_a, at_b = at_a + na, at_b + nb
    assert at_a == T and at_b == 300
    for got, want in ((torch.cat(got_a), want_a), (torch.cat(got_b), want_b)):
        err = (got - want).abs().max(-1).values / want.abs().max()
        assert err.max() < 0.02, (float(err.max()), int(err.argmax()))
    assert harness.status.item() == 0


def test_a_sink_that_outweighs_every_key_silences_its_head():
    width, T, heads, dk = 48, 20, 3, 16
    gen = torch.Generator().manual_seed(9)
    spec, block = attention_case(heads, 1, dk, dk, rows=4, far=9, coef=0.3, every=3)
    mixer = build_mixer(spec, width, None)
    W = attention_weights(mixer, width, gen)
    W["sink"] = torch.tensor([30.0, -30.0, 0.5])
    give(mixer, W, torch.float32)
    harness = Harness([mixer.cache_spec()], [None], torch.float32, num_pages=8, page_size=4)
    x = rounded(T, width, gen=gen)
    got = run_in_portions(mixer, harness, x, (T,), torch.float32)
    want = plain.sink_attention(x, {"p." + k: v for k, v in W.items()}, "p.", block)
    assert torch.allclose(got, want, **F32)
    silenced = dict(W, sink=torch.tensor([30.0, 30.0, 30.0]))
    give(mixer, silenced, torch.float32)
    harness = Harness([mixer.cache_spec()], [None], torch.float32, num_pages=8, page_size=4)
    assert run_in_portions(mixer, harness, x, (T,), torch.float32).abs().max() < 1e-6


# ---------------------------------------------------------------- gated delta rule alone
def delta_case(heads, kv, dk, dv, taps, rank_a=4, rank_g=6, eps=1e-5):
    spec = PartSpec.make("gated_delta", num_heads=heads, num_kv_heads=kv, head_dim=dk, v_head_dim=dv, conv_taps=taps,
                         eps=eps, decay_rank=rank_a, gate_rank=rank_g)
    return spec, dict(heads=heads, kv_heads=kv, dim=dk, vdim=dv, conv=taps)


def delta_weights(mixer, gen):
    W = {}
    for key, w in mixer.weight_specs().items():
        if key.endswith("conv"):
            W[key] = rounded(*w.shape, gen=gen, std=0.6)
        elif key == "A_log":
            W[key] = rounded(*w.shape, gen=gen, std=0.7, mean=-0.5)
        elif key == "dt_bias":
            W[key] = rounded(*w.shape, gen=gen)
        elif key == "norm":
            W[key] = rounded(*w.shape, gen=gen, std=0.2, mean=1.0)
        else:
            W[key] = rounded(*w.shape, gen=gen, std=1.5 / math.sqrt(w.shape[-1]))
    return W


@pytest.mark.parametrize("heads,kv,dk,dv,taps", [(4, 2, 8, 12, 4), (2, 2, 40, 20, 2), (1, 1, 96, 70, 1), (3, 1, 136, 33, 6)])
def test_gated_delta_in_portions_and_token_by_token(heads, kv, dk, dv, taps):
    """Prefill against decoding, portions shorter than the convolution's reach, key widths that
    take 1, 2, 4 and 8 lanes per column, value widths that do not fill a block of columns."""
    gen = torch.Generator().manual_seed(dk)
    width, T = 56, 41
    spec, block = delta_case(heads, kv, dk, dv, taps)
    mixer = build_mixer(spec, width, None)
    W = delta_weights(mixer, gen)
    give(mixer, W, torch.float32)
    x = rounded(T, width, gen=gen)
    want, final = plain.gated_delta(x, {"p." + k: v for k, v in W.items()}, "p.", block, 1e-5)
    for sizes in ((T,), (1,) * T, (2, 1, 3, 2, 2, 17, 1, 1, 12)):
        harness = Harness([None], [mixer.state_spec()], torch.float32, max_requests=2)
        got = run_in_portions(mixer, harness, x, sizes, torch.float32)
        assert torch.allclose(got, want, **F32), sizes
        state = harness.cache.layer_caches[0].state[harness.cache.slot("s")].cpu()
        assert torch.allclose(state[: heads * dk * dv].view(heads, dv, dk).transpose(1, 2), final, **F32)   # kept transposed
        assert harness.status.item() == 0


def test_gated_delta_state_is_per_request_and_slots_are_cleared_for_the_next_tenant():
    gen = torch.Generator().manual_seed(3)
    width = 40
    spec, block = delta_case(2, 1, 16, 24, 3)
    mixer = build_mixer(spec, width, None)
    W = delta_weights(mixer, gen)
    give(mixer, W, torch.float32)
    named = {"p." + k: v for k, v in W.items()}
    xs = {name: rounded(n, width, gen=gen) for name, n in (("a", 9), ("b", 14), ("c", 5))}
    want = {name: plain.gated_delta(x, named, "p.", block, 1e-5)[0] for name, x in xs.items()}
    harness = Harness([None], [mixer.state_spec()], torch.float32, max_requests=2)
    cache = harness.cache.layer_caches[0]
    # a and b side by side, in unequal portions of one batch
    ctx = harness.context([StepEntry("a", [0] * 4), StepEntry("b", [0] * 13)])
    got = mixer.forward(ctx, torch.cat([xs["a"][:4], xs["b"][:13]]).to(DEV), cache).cpu()
    assert torch.allclose(got, torch.cat([want["a"][:4], want["b"][:13]]), **F32)
    ctx = harness.context([StepEntry("b", [0]), StepEntry("a", [0] * 5)])
    got = mixer.forward(ctx, torch.cat([xs["b"][13:], xs["a"][4:]]).to(DEV), cache).cpu()
    assert torch.allclose(got, torch.cat([want["b"][13:], want["a"][4:]]), **F32)
    # c takes the slot a leaves, with a's state still in it until the manager clears it
    harness.cache.finish("a")
    assert cache.state.abs().sum(-1).min() > 0
    ctx = harness.context([StepEntry("c", [0] * 5)])
    got = mixer.forward(ctx, xs["c"].to(DEV), cache).cpu()
    assert torch.allclose(got, want["c"], **F32)


# ---------------------------------------------------------------- expert feed-forward alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,ff", [(5, 3, 24), (1, 1, 48), (8, 1, 16), (6, 6, 32), (70, 4, 8)])
def test_expert_mixture_against_plain(dtype, experts, top, ff):
    gen = torch.Generator().manual_seed(experts)
    width, T = 72, 19
    part = build_feed_forward(PartSpec.make("moe", experts=experts, top=top, intermediate_size=ff, float32_out=True), width)
    W = {k: rounded(*w.shape, gen=gen, std=(3.0 if k == "router" else 1.0) / math.sqrt(w.shape[-1]))
         for k, w in part.weight_specs().items()}
    give(part, W, dtype)
    x = rounded(T, width, gen=gen)
    got = part.forward(Ctx(dtype), x.to(DEV, dtype))
    want = plain.expert_mixture(x, {"p." + k: v for k, v in W.items()}, "p.", dict(router=dict(top=top)))
    assert got.dtype == torch.float32
    assert torch.allclose(got.cpu(), want, atol=2e-5 if dtype == torch.float32 else 4e-2)
    logits = x @ W["router"].T
    chosen, weights, dense = ops.moe_route(logits.to(DEV), top)
    values, index = torch.topk(logits, top)
    assert torch.equal(chosen.cpu().long(), index)
    assert torch.allclose(weights.cpu(), torch.softmax(values, -1), atol=1e-6)
    assert torch.allclose(dense.cpu().sum(-1), torch.ones(T), atol=1e-6) and int((dense != 0).sum()) == T * top


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,ff", [(5, 3, 24), (8, 1, 16), (70, 4, 8)])
def test_expert_mixture_sorted_by_expert_for_long_portions(dtype, experts, top, ff):
    """A step of prompt portions: pairs sorted by expert, one product per expert with work (some
    of the 70 experts get none), picks added in pick order. The same result as the stacked way."""
    gen = torch.Generator().manual_seed(experts + 1)
    width, T = 72, 300
    part = build_feed_forward(PartSpec.make("moe", experts=experts, top=top, intermediate_size=ff, float32_out=True), width)
    W = {k: rounded(*w.shape, gen=gen, std=(3.0 if k == "router" else 1.0) / math.sqrt(w.shape[-1]))
         for k, w in part.weight_specs().items()}
    give(part, W, dtype)
    x = rounded(T, width, gen=gen)
    ctx = Ctx(dtype)
    ctx.all_decode = False
    assert T >= part.GROUPED_FROM
    before = ops.LAUNCHES
    got = part.forward(ctx, x.to(DEV, dtype))
    grouped_launches = ops.LAUNCHES - before
    want = plain.expert_mixture(x, {"p." + k: v for k, v in W.items()}, "p.", dict(router=dict(top=top)))
    assert torch.allclose(got.cpu(), want, atol=2e-5 if dtype == torch.float32 else 4e-2)
    ctx.all_decode = True                       # the stacked way, as a decode step takes it
    before = ops.LAUNCHES
    stacked = part.forward(ctx, x.to(DEV, dtype))
    assert ops.LAUNCHES - before < grouped_launches
    assert torch.allclose(stacked.cpu(), want, atol=2e-5 if dtype == torch.float32 else 4e-2)
    logits = (x @ W["router"].T).to(DEV)
    chosen, _, _ = ops.moe_route(logits, top)
    offsets, rows, where = ops.moe_group(chosen, experts)
    offsets, rows, where, chosen = offsets.cpu(), rows.cpu(), where.cpu(), chosen.cpu()
    assert offsets[0] == 0 and offsets[-1] == T * top and bool((offsets[1:] >= offsets[:-1]).all())
    for e in range(experts):
        run = rows[offsets[e]:offsets[e + 1]]
        assert bool((run[1:] >= run[:-1]).all())                         # inside a run: by pair index
    assert torch.equal(rows[where.long()], torch.arange(T)[:, None].expand(T, top).int())
    place_expert = torch.bucketize(where.long(), offsets[1:].long(), right=True)
    assert torch.equal(place_expert.int(), chosen)


# ---------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (config, shapes, seed) in tiny.ALL.items():
        folder = tiny.write_model(tmp_path_factory.mktemp(f"mugizen_{name}"), config, shapes, seed)
        out[name] = (folder,) + tiny.load_plain(folder)
    return out


def prompt(config, n, seed):
    return torch.randint(0, config["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def close_rows(got, want, dtype):
    """float32: every row equal up to rounding order. bfloat16: rows may differ by the rounding of
    every product, and a few by a router's close call; bound the typical and the worst row."""
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    if dtype == "float32":
        return bool(err.max() < 2e-4)
    return bool(err.median() < 0.03 and err.max() < 0.3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["p", "q", "r"])
def test_whole_prompt_portions_and_decoding_against_plain(models, name, dtype, monkeypatch):
    from vosti_b200.parts import ExpertMixture
    monkeypatch.setattr(ExpertMixture, "GROUPED_FROM", 16)      # portions of 16 tokens or more sort their pairs by expert
    folder, config, W = models[name]
    tokens = prompt(config, 61, 1)
    want = plain.forward(config, W, tokens)
    everything = list(range(len(tokens)))
    for sizes in ((61,), (29,) + (1,) * 32, (2, 5, 1, 1, 17, 2, 3, 30)):
        page = tiny.PAGE[name]
        runner = ModelRunner(folder, dtype=dtype, num_pages=96 // page, page_size=page, max_requests=2)
        runner.begin("r")
        rows, at = [], 0
        for size in sizes:
            rows.append(runner.step([StepEntry("r", tokens[at:at + size], list(range(size)))]).cpu())
            at += size
        runner.check_status()
        assert close_rows(torch.cat(rows), want[everything], dtype), sizes


def test_residual_stream_after_every_layer_run(models):
    folder, config, W = models["p"]
    tokens = prompt(config, 23, 2)
    _, want = plain.forward(config, W, tokens, return_layers=True)
    runner = ModelRunner(folder, dtype="float32", num_pages=8, page_size=8, max_requests=1)
    streams = []
    for block in runner.model.blocks:
        inner = block.forward

        def watched(ctx, hidden, residual, cache, writes_cache=True, inner=inner):
            out, stream = inner(ctx, hidden, residual, cache, writes_cache)
            streams.append(ops.stream_sum(stream, out).cpu())
            return out, stream
        block.forward = watched
    runner.begin("r")
    runner.step([StepEntry("r", tokens, [0])])
    assert len(streams) == want.shape[0] == 8          # 1 + 3 * 2 + 1 layer runs
    for got, expected in zip(streams, want):
        assert torch.allclose(got, expected, atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("name,dtype", [("p", "float32"), ("q", "float32"), ("r", "float32"), ("r", "bfloat16")])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(models, name, dtype):
    """Four requests through two state slots and a pool that holds two of them: portions of some
    beside single tokens of others; every request equals itself alone."""
    folder, config, W = models[name]
    lengths = {"a": 37, "b": 9, "c": 1, "d": 26}
    tokens = {r: prompt(config, n, 10 + i) for i, (r, n) in enumerate(lengths.items())}
    want = {r: plain.forward(config, W, t) for r, t in tokens.items()}
    page = tiny.PAGE[name]
    pool = 80 // page
    runner = ModelRunner(folder, dtype=dtype, num_pages=pool, page_size=page, max_requests=2)
    schedule = [
        [("a", 5), ("b", 2)], [("a", 1), ("b", 6)], [("b", 1), ("a", 20)], [("a", 1)],      # b ends in step 2
        [("c", 1), ("a", 2)], [("d", 3), ("a", 8)], [("d", 1)], [("d", 22)],                # c, then a end
    ]
    at = {r: 0 for r in lengths}
    got = {r: [] for r in lengths}
    for step in schedule:
        entries = []
        for r, n in step:
            if r not in runner.cache.live:
                runner.begin(r)
            entries.append(StepEntry(r, tokens[r][at[r]:at[r] + n], list(range(n))))
        logits = runner.step(entries).cpu()
        row = 0
        for r, n in step:
            got[r].append(logits[row:row + n])
            row += n
            at[r] += n
            if at[r] == lengths[r]:
                runner.finish(r)
    runner.check_status()
    runner.cache.check()
    for r in lengths:
        assert at[r] == lengths[r]
        assert close_rows(torch.cat(got[r]), want[r], dtype), r
    assert runner.cache.available_pages() == pool and len(runner.cache.free_slots) == 2


def test_long_decoding_keeps_its_state(models):
    folder, config, W = models["q"]
    tokens = prompt(config, 150, 4)
    want = plain.forward(config, W, tokens)
    runner = ModelRunner(folder, dtype="float32", num_pages=20, page_size=8, max_requests=1)
    runner.begin("r")
    rows = [runner.step([StepEntry("r", tokens[:3], [0, 1, 2])]).cpu()]
    rows += [runner.step([StepEntry("r", [t], [0])]).cpu() for t in tokens[3:]]
    assert close_rows(torch.cat(rows), want, "float32")


def plain_greedy(config, W, tokens, new_tokens):
    tokens, out = list(tokens), []
    for _ in range(new_tokens):
        out.append(int(plain.forward(config, W, tokens)[-1].argmax()))
        tokens.append(out[-1])
    return out


@pytest.mark.parametrize("cuda_graphs,async_scheduling", [(False, False), (True, False), (True, True)])
def test_greedy_generation_through_the_engine(models, cuda_graphs, async_scheduling):
    """The framework's own entry point: scheduler, portions under a token budget, CUDA graphs for
    decode steps, two slots for five requests, so few pages that a request is preempted."""
    folder, config, W = models["p"]
    prompts = [prompt(config, n, 20 + n) for n in (5, 17, 2, 11, 8)]
    want = [plain_greedy(config, W, p, 10) for p in prompts]
    engine = Engine(folder, dtype="float32", num_blocks=9, block_size=4, max_num_seqs=2, max_num_batched_tokens=16,
                    prefill_chunk_size=8, cuda_graphs=cuda_graphs, async_scheduling=async_scheduling)
    assert engine.runner.spec.architecture == "Mugizen" and engine.runner.cache.has_state
    assert (engine.graphs is not None) == cuda_graphs
    got = engine.generate(prompts, max_tokens=10, arrival_steps=[0, 0, 1, 4, 20])
    assert got == want
    assert engine.scheduler.preemptions > 0
    if cuda_graphs:
        assert engine.graphs.replays > 0
    engine.runner.cache.check()
    assert engine.runner.cache.available_pages() == 9 and len(engine.runner.cache.free_slots) == 2
