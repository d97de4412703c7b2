"""The Vivesun design on the GPU against the plain implementation (tests/plain_vivesun.py).

Mechanisms alone (pair-hash embedding and its state, the stream norm, the token input, rotated
chunked attention with one in the denominator, both recurrences, the expert feed-forward, the
branch sum), then whole models of three small configurations: whole prompts, prefill against
token-by-token decoding, portions down to two tokens, unequal requests in one batch against each
alone, pages and state slots used again, long decoding across many chunks, and greedy generation
through `Engine` (scheduler, CUDA graphs, asynchronous scheduling, preemption).

Where random inputs would hide a fault, the inputs are made so that it shows: one query and key
are scaled so that a single score stands out, at the first key of a chunk, far back inside it,
at a page border, and just outside it; scores far below zero show the one in the denominator.

Exactness is tested in float32 (differences of rounding order only). bfloat16 serving is
compared with the float32 oracle row by row with a bound on the typical error, because a
router's close call may send a token to another expert there.
"""
import math

import pytest
import torch

import plain_vivesun as plain
import tiny_vivesun as tiny
from gpu_util import Harness
from vosti_b200 import Engine, ops
from vosti_b200.config import PartSpec
from vosti_b200.engine.batch import StepEntry
from vosti_b200.engine.runner import ModelRunner
from vosti_b200.parts import (PagedCacheSpec, StateSpec, build_embedding, build_feed_forward, build_mixer, build_norm,
                              build_token_input)

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


def weights_of(part, gen, big=()):
    """Random weights for a part: matrices with unit-variance outputs, vectors of order one."""
    W = {}
    for key, w in part.weight_specs().items():
        if len(w.shape) == 2 and key.split(".")[-1] != "conv":
            W[key] = rounded(*w.shape, gen=gen, std=(2.0 if key in big else 1.0) / math.sqrt(w.shape[-1]))
        elif key.split(".")[-1] == "conv":
            W[key] = rounded(*w.shape, gen=gen, std=0.6)
        elif key == "norm":
            W[key] = rounded(*w.shape, gen=gen, std=0.2, mean=1.0)
        else:
            W[key] = rounded(*w.shape, gen=gen, std=0.8)
    return W


class Ctx:
    def __init__(self, dtype):
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.dtype = dtype
        self.extras = {}


# ---------------------------------------------------------------- embedding, norm, token input
def test_pair_hash_embedding_and_its_state_across_portions_and_slots():
    gen = torch.Generator().manual_seed(1)
    vocab, width, buckets, mp, mc = 50, 24, 13, 2000000011, 1500000001
    part = build_embedding(PartSpec.make("pair_hash", buckets=buckets, mul_prev=mp, mul_cur=mc, side_width=6,
                                         names=(("pairs", "bigram"), ("side", "side.embed"))), width, vocab)
    W = {"weight": rounded(vocab, width, gen=gen), "pairs": rounded(buckets + 1, width, gen=gen), "side": rounded(vocab, 6, gen=gen)}
    give(part, W, torch.bfloat16)
    harness = Harness([None], [part.state_spec()], torch.bfloat16, max_requests=2)
    cache = harness.cache.layer_caches[0]
    assert cache.state.dtype == torch.int32
    seqs = {"a": torch.randint(0, vocab, (11,), generator=gen).tolist(), "b": torch.randint(0, vocab, (6,), generator=gen).tolist(),
            "c": torch.randint(0, vocab, (4,), generator=gen).tolist()}
    want = {r: W["weight"][t] + W["pairs"][plain.pair_rows(t, buckets, mp, mc)] for r, t in seqs.items()}
    assert any(a * mp + b * mc >= 1 << 31 for a, b in zip(seqs["a"], seqs["a"][1:]))      # the hash needs 64 bits
    got = {r: [] for r in seqs}
    # portions of a beside b; then c takes the slot b leaves, whose last token is still in it
    for step in ([("a", 0, 2), ("b", 0, 5)], [("b", 5, 6), ("a", 2, 3)], [("a", 3, 9)], [("c", 0, 1), ("a", 9, 11)], [("c", 1, 4)]):
        entries = [StepEntry(r, seqs[r][lo:hi]) for r, lo, hi in step]
        ctx = harness.context(entries)
        rows = part.forward(ctx, ctx.tokens, cache=cache)
        assert rows.dtype == torch.float32 and torch.equal(ctx.extras["token_ids"].cpu(), ctx.tokens.cpu())
        at = 0
        for r, lo, hi in step:
            got[r].append(rows[at:at + hi - lo].cpu())
            at += hi - lo
            if hi == len(seqs[r]):
                harness.cache.finish(r)
    for r in seqs:
        assert torch.equal(torch.cat(got[r]), want[r]), r


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [200, 67])
def test_stream_norm_with_deferred_sum(dtype, width):
    gen = torch.Generator().manual_seed(2)
    rows, eps = 7, 1e-3
    norm = build_norm(PartSpec.make("rms_stream", eps=eps, unit_offset=True), width)
    W = {"weight": rounded(width, gen=gen, std=0.3)}
    give(norm, W, dtype)
    ctx = Ctx(dtype)
    stream, a, b = rounded(rows, width, gen=gen), rounded(rows, width, gen=gen), rounded(rows, width, gen=gen)
    kept = stream.clone().to(DEV)
    got, new_stream = norm.forward_add(ctx, ops.DeferredSum(a.to(DEV), b.to(DEV, dtype)), kept)
    total = stream + a + b
    assert new_stream.dtype == torch.float32 and torch.allclose(new_stream.cpu(), total, atol=1e-6)
    assert got.dtype == dtype
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(got.float().cpu(), plain.offset_norm(total, W["weight"], eps), atol=tol)
    assert torch.allclose(norm.forward(ctx, a.to(DEV)).float().cpu(), plain.offset_norm(a, W["weight"], eps), atol=tol)
    plain_weight = build_norm(PartSpec.make("rms_stream", eps=eps, out_dtype="float32"), width)
    give(plain_weight, W, dtype)
    assert torch.allclose(plain_weight.forward(ctx, a.to(DEV)).cpu(), plain.unit_rms(a, eps) * W["weight"], atol=1e-5)
    # the sum alone, stored in place and rounded to the serving type
    x = ops.rms_stream(a.to(DEV), None, 0.0, dtype, stream=kept, stream_out=kept)
    assert torch.allclose(kept.cpu(), total + a, atol=1e-6) and torch.allclose(x.float().cpu(), total + a, atol=tol * 4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_input_against_plain(dtype):
    gen = torch.Generator().manual_seed(3)
    width, vocab, dim, layers, T, eps = 72, 40, 5, 3, 9, 1e-5
    table = rounded(vocab, dim * layers, gen=gen)
    tokens = torch.randint(0, vocab, (T,), generator=gen)
    x = rounded(T, width, gen=gen)
    for layer in range(layers):
        part = build_token_input(PartSpec.make("gated_table", dim=dim, offset=layer * dim, eps=eps), width)
        W = weights_of(part, gen)
        give(part, W, dtype)
        ctx = Ctx(dtype)
        ctx.extras = {"token_ids": tokens.int().to(DEV), "token_table": table.to(DEV, dtype)}
        got = part.forward(ctx, x.to(DEV, dtype))
        w = {"side.embed": table, **{"p." + k: v for k, v in W.items()}}
        want = plain.token_side(x, tokens.tolist(), w, "p.", layer, dim, eps)
        assert got.dtype == torch.float32
        assert torch.allclose(got.cpu(), want, atol=2e-5 if dtype == torch.float32 else 6e-2), layer


def test_rotation_frequencies_follow_the_wavelength_rule():
    from vosti_b200.parts import build_position
    for dims, base, scaling in ((16, 300000.0, (6.0, 1.0, 4.0, 4096)), (24, 100.0, (4.0, 1.0, 3.0, 40)), (8, 10000.0, None),
                                (6, 50.0, (2.0, 0.5, 2.0, 16))):
        part = build_position(PartSpec.make("rope", theta=base, rotary_dim=dims, max_positions=0,
                                            scaling=None if scaling is None else ("wavelength",) + scaling), 64, 64)
        as_dict = None if scaling is None else dict(zip(("factor", "low", "high", "original"), scaling))
        want = torch.tensor(plain.rotary_frequencies(dims, base, as_dict), dtype=torch.float64)
        assert torch.allclose(part.frequencies().double(), want, rtol=2e-7, atol=0)
        if scaling is not None:      # all three branches of the rule occur
            kept = sum(abs(f - base ** (-2.0 * i / dims)) < 1e-12 for i, f in enumerate(want.tolist()))
            cut = sum(abs(f - base ** (-2.0 * i / dims) / scaling[0]) < 1e-12 for i, f in enumerate(want.tolist()))
            assert kept > 0 and cut > 0 and (dims != 16 or kept + cut < dims // 2)


# ---------------------------------------------------------------- attention alone
def attention_spec(heads, kv, dk, dv, chunk, rot_dims, base=100.0, scale=0.25):
    return PartSpec.make("sink_attention", num_heads=heads, num_kv_heads=kv, head_dim=dk, v_head_dim=dv, scale=scale,
                         window=0, chunk=chunk, sink=False, sink_value=0.0,
                         position=PartSpec.make("rope", theta=base, rotary_dim=rot_dims, scaling=None, max_positions=0))


def plain_attention(qkv, heads, kv, dk, dv, chunk, rot_dims, base, scale):
    T = qkv.shape[0]
    q, k, v = qkv.split([heads * dk, kv * dk, kv * dv], dim=-1)
    freqs = plain.rotary_frequencies(rot_dims, base, None)
    q = plain.rotate(q.view(T, heads, dk), list(range(T)), freqs)
    k = plain.rotate(k.view(T, kv, dk), list(range(T)), freqs)
    return plain.chunk_attention(q, k, v.view(T, kv, dv), scale, chunk).reshape(T, heads * dv)


def run_attention(mixer, harness, qkv, sizes, dtype, rid="r"):
    """The kernels behind the mixer's projections, fed with a hand-made q | k | v row per token."""
    cache = harness.cache.layer_caches[0]
    outs, at = [], 0
    for size in sizes:
        ctx = harness.context([StepEntry(rid, [0] * size)])
        group = ctx.group(cache.group)
        part = qkv[at:at + size].to(DEV, dtype).contiguous()
        q = ops.qkv_store(part, cache.k, cache.v, nq=mixer.nq, nkv=mixer.nkv, dk=mixer.dk, dv=mixer.dv,
                          page_size=group.page_size, positions=ctx.positions, slot_mapping=group.slot_mapping,
                          temp_coef=0.0, temp_every=1, status=ctx.status, freq=mixer.freq)
        outs.append(ops.attention_sink(ctx, q, cache.k, cache.v, group, nq=mixer.nq, nkv=mixer.nkv, dk=mixer.dk, dv=mixer.dv,
                                       scale=mixer.scale, window=0, bias=None, sink=mixer.sink, chunk=mixer.chunk).float().cpu())
        at += size
    assert int(harness.status.item()) == 0
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dk,dv,chunk,rot,page", [(4, 2, 24, 16, 7, 24, 8), (2, 1, 16, 40, 20, 2, 8), (3, 3, 8, 8, 1, 4, 4), (2, 1, 6, 10, 5, 6, 4),
                                                          (4, 2, 64, 64, 48, 32, 16), (2, 2, 128, 128, 100, 64, 16),
                                                          (6, 1, 64, 64, 33, 16, 16)])
def test_rotated_chunked_attention_against_plain(dtype, heads, kv, dk, dv, chunk, rot, page):
    gen = torch.Generator().manual_seed(heads * 100 + dk)
    T = 150
    mixer = build_mixer(attention_spec(heads, kv, dk, dv, chunk, rot), 64, None)
    mixer.setup(torch.device(DEV), dtype)
    qkv = rounded(T, heads * dk + kv * (dk + dv), gen=gen)
    want = plain_attention(qkv, heads, kv, dk, dv, chunk, rot, 100.0, 0.25)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for sizes in ((T,), (97,) + (1,) * 53, (2, 5, 1, 1, 17, 2, 3, 60, 59)):
        harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=-(-T // page) + 1, page_size=page)
        got = run_attention(mixer, harness, qkv, sizes, dtype)
        assert torch.allclose(got, want, atol=tol, rtol=tol), sizes


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dk,chunk,page", [(24, 40, 8), (64, 48, 16), (64, 120, 16)])
def test_one_key_stands_out_at_the_edges_of_a_chunk(dtype, dk, chunk, page):
    """The query of the last position and one key share a large component in a part of the head
    that does not turn. Inside the query's chunk (its first key, a key next to a page border, the
    key before the query) the output is that key's value; just outside the chunk it must not be
    seen at all. The same for a prompt portion and for a token decoded alone."""
    heads, kv, dv, rot = 2, 1, dk, 8
    gen = torch.Generator().manual_seed(dk + chunk)
    mixer = build_mixer(attention_spec(heads, kv, dk, dv, chunk, rot, scale=1.0), 64, None)
    mixer.setup(torch.device(DEV), dtype)
    T = 2 * chunk + chunk // 2 + 3                       # the last position lies in the third chunk
    first = (T - 1) // chunk * chunk
    base = rounded(T, heads * dk + kv * (dk + dv), gen=gen, std=0.1)
    base[:, heads * dk + kv * dk:] = rounded(T, kv * dv, gen=gen)            # values of order one
    inside = [first, first + 1, (first // page + 1) * page, (first // page + 1) * page - 1, T - 2]
    outside = [first - 1, first - 2, first - chunk, 0]
    for target in [j for j in inside if first <= j < T - 1] + outside:
        qkv = base.clone()
        qkv[T - 1, dk - 1] = 8.0                         # head 0's query, last element (not rotated)
        qkv[target, heads * dk + dk - 1] = 8.0           # the key at `target`
        want = plain_attention(qkv, heads, kv, dk, dv, chunk, rot, 100.0, 1.0)
        value = qkv[target, heads * dk + kv * dk:heads * dk + kv * dk + dv]
        seen = torch.allclose(want[T - 1, :dv], value, atol=1e-3)
        assert seen == (target >= first), target                            # the oracle agrees with the design
        for sizes in ((T,), (T - 1, 1), (first - 1, 3, T - first - 2)):
            harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=-(-T // page) + 1, page_size=page)
            got = run_attention(mixer, harness, qkv, sizes, dtype)
            tol = 2e-5 if dtype == torch.float32 else 3e-2
            assert torch.allclose(got[T - 1], want[T - 1], atol=tol, rtol=tol), (target, sizes)
            assert torch.allclose(got[T - 1, :dv], value, atol=2e-2) == (target >= first), (target, sizes)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_one_in_the_denominator_shows_when_scores_are_low(dtype):
    """Scores far below zero: without the added one the weights would still sum to 1."""
    heads, kv, dk, dv, chunk = 2, 2, 64, 64, 30
    gen = torch.Generator().manual_seed(9)
    mixer = build_mixer(attention_spec(heads, kv, dk, dv, chunk, 16, scale=1.0), 64, None)
    mixer.setup(torch.device(DEV), dtype)
    T = 45
    qkv = rounded(T, heads * dk + kv * (dk + dv), gen=gen, std=0.05)
    qkv[:, heads * dk + kv * dk:] = 1.0                  # every value is the vector of ones
    qkv[:, dk - 1] = 4.0                                 # head 0: q.k = -16 for every pair
    qkv[:, heads * dk + dk - 1] = -4.0
    want = plain_attention(qkv, heads, kv, dk, dv, chunk, 16, 100.0, 1.0)
    assert float(want[:, :dv].abs().max()) < 1e-4 and float(want[25:30, dv:].min()) > 0.8    # head 0 sees next to nothing
    for sizes in ((T,), (T - 5, 1, 1, 1, 1, 1)):
        harness = Harness([mixer.cache_spec()], [None], dtype, num_pages=4, page_size=16)
        got = run_attention(mixer, harness, qkv, sizes, dtype)
        assert torch.allclose(got, want, atol=2e-5 if dtype == torch.float32 else 2e-2), sizes


def test_attention_mixer_with_projections_against_plain():
    gen = torch.Generator().manual_seed(4)
    width, T = 72, 41
    block = dict(heads=4, kv_heads=2, dim=24, vdim=16, scale=0.3, mask=dict(size=7),
                 rot=dict(base=100.0, dims=24, scaling=dict(factor=4.0, low=1.0, high=3.0, original=40)))
    spec = PartSpec.make("sink_attention", num_heads=4, num_kv_heads=2, head_dim=24, v_head_dim=16, scale=0.3, window=0, chunk=7,
                         sink=False, sink_value=0.0,
                         position=PartSpec.make("rope", theta=100.0, rotary_dim=24, max_positions=0,
                                                scaling=("wavelength", 4.0, 1.0, 3.0, 40)))
    mixer = build_mixer(spec, width, None)
    W = weights_of(mixer, gen)
    give(mixer, W, torch.float32)
    x = rounded(T, width, gen=gen)
    want = plain.attention_branch(x, {"p." + k: v for k, v in W.items()}, "p.", block)
    harness = Harness([mixer.cache_spec()], [None], torch.float32, num_pages=8, page_size=8)
    outs, at = [], 0
    for size in (13, 1, 1, 2, 24):
        ctx = harness.context([StepEntry("r", [0] * size)])
        outs.append(mixer.forward(ctx, x[at:at + size].to(DEV), harness.cache.layer_caches[0]).cpu())
        at += size
    assert torch.allclose(torch.cat(outs), want, **F32)


# ---------------------------------------------------------------- the recurrences alone
def run_mixer(mixer, harness, x, sizes, dtype, rid="r"):
    outs, at = [], 0
    for size in sizes:
        ctx = harness.context([StepEntry(rid, [0] * size)])
        outs.append(mixer.forward(ctx, x[at:at + size].to(DEV, dtype), harness.cache.layer_caches[0]).float().cpu())
        at += size
    assert int(harness.status.item()) == 0
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,d,rank", [(3, 20, 3), (2, 40, 2), (1, 48, 5), (2, 64, 16), (6, 8, 1), (1, 130, 4), (2, 5, 2)])
def test_general_delta_rule_against_plain(dtype, heads, d, rank):
    gen = torch.Generator().manual_seed(heads * 10 + d)
    width, T, eps = 72, 50, 1e-5
    mixer = build_mixer(PartSpec.make("general_delta", num_heads=heads, head_dim=d, decay_rank=rank, eps=eps), width, None)
    W = weights_of(mixer, gen, big=("w2",))
    give(mixer, W, dtype)
    x = rounded(T, width, gen=gen)
    want = plain.general_delta_branch(x, {"p." + k: v for k, v in W.items()}, "p.", dict(heads=heads, dim=d), eps)
    for sizes in ((T,), (17,) + (1,) * 33, (2, 5, 1, 1, 17, 2, 3, 19)):
        harness = Harness([None], [mixer.state_spec()], dtype, max_requests=2)
        got = run_mixer(mixer, harness, x, sizes, dtype)
        if dtype == torch.float32:
            assert torch.allclose(got, want, **F32), sizes
        else:
            assert float((got - want).abs().mean() / want.abs().mean()) < 0.04, sizes


def test_general_delta_recurrence_kernel_alone_with_strong_removal():
    """The scan with hand-made inputs: decays near one, removal rates near one, so that what a key
    wrote long ago is still there and the removal term matters; against the token-by-token form."""
    gen = torch.Generator().manual_seed(5)
    heads, d, T = 2, 24, 70
    r, k, v = (torch.randn(T, heads, d, generator=gen) for _ in range(3))
    decay = 0.97 + 0.03 * torch.rand(T, heads, d, generator=gen)
    rate = 0.9 + 0.1 * torch.rand(T, heads, d, generator=gen)
    want = plain.general_delta_recurrence(r.double(), k.double(), v.double(), decay.double(), rate.double()).float()
    unit = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    flat = lambda t: t.reshape(T, heads * d).contiguous().to(DEV)
    for sizes in ((T,), (33, 1, 1, 35)):
        harness = Harness([None], [StateSpec((heads * d * d,), torch.float32)], torch.float32, max_requests=2)
        outs, at = [], 0
        for size in sizes:
            ctx = harness.context([StepEntry("r", [0] * size)])
            cut = lambda t: flat(t)[at:at + size].contiguous()
            outs.append(ops.general_delta_scan(cut(r), cut(k), cut(v), cut(decay), cut(unit), cut(rate * unit),
                                               harness.cache.layer_caches[0].state, ctx, heads=heads, d=d).cpu())
            at += size
        assert torch.allclose(torch.cat(outs).view(T, heads, d), want, atol=2e-3, rtol=2e-3), sizes


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dk,dv,taps", [(4, 2, 8, 12, 2), (3, 3, 40, 20, 4), (1, 1, 48, 48, 1), (4, 2, 64, 64, 4), (2, 1, 16, 70, 5),
                                                 (2, 1, 5, 3, 3)])
def test_gated_delta_rule_with_a_decay_per_head_against_plain(dtype, heads, kv, dk, dv, taps):
    gen = torch.Generator().manual_seed(heads * 10 + dk)
    width, T, eps = 72, 50, 1e-5
    spec = PartSpec.make("gated_delta", num_heads=heads, num_kv_heads=kv, head_dim=dk, v_head_dim=dv, conv_taps=taps, eps=eps,
                         decay="head", decay_rank=0, gate_rank=0, gate_activation="silu")
    mixer = build_mixer(spec, width, None)
    assert set(mixer.weight_specs()) == {"q", "k", "v", "q.conv", "k.conv", "v.conv", "b", "A_log", "norm", "a", "dt_bias", "g", "o"}
    assert mixer.weight_specs()["dt_bias"].shape == (heads,) and mixer.weight_specs()["a"].shape == (heads, width)
    W = weights_of(mixer, gen)
    W["A_log"] = rounded(heads, gen=gen, std=0.7, mean=-0.5)
    give(mixer, W, dtype)
    x = rounded(T, width, gen=gen)
    block = dict(heads=heads, kv_heads=kv, dim=dk, vdim=dv, conv=taps)
    want = plain.gated_delta_mixer(x, {"p." + k: v for k, v in W.items()}, "p.", block, eps)
    for sizes in ((T,), (17,) + (1,) * 33, (2, 5, 1, 1, 17, 2, 3, 19)):
        harness = Harness([None], [mixer.state_spec()], dtype, max_requests=2)
        got = run_mixer(mixer, harness, x, sizes, dtype)
        if dtype == torch.float32:
            assert torch.allclose(got, want, **F32), sizes
        else:
            assert float((got - want).abs().mean() / want.abs().mean()) < 0.04, sizes


def test_recurrent_state_of_a_slot_that_is_used_again():
    gen = torch.Generator().manual_seed(6)
    width, eps = 72, 1e-5
    mixer = build_mixer(PartSpec.make("general_delta", num_heads=2, head_dim=24, decay_rank=3, eps=eps), width, None)
    W = weights_of(mixer, gen, big=("w2",))
    give(mixer, W, torch.float32)
    xs = {r: rounded(n, width, gen=gen) for r, n in (("a", 12), ("b", 30), ("c", 5))}
    want = {r: plain.general_delta_branch(x, {"p." + k: v for k, v in W.items()}, "p.", dict(heads=2, dim=24), eps) for r, x in xs.items()}
    harness = Harness([None], [mixer.state_spec()], torch.float32, max_requests=2)
    cache = harness.cache.layer_caches[0]
    ctx = harness.context([StepEntry("a", [0] * 4), StepEntry("b", [0] * 13)])
    got = mixer.forward(ctx, torch.cat([xs["a"][:4], xs["b"][:13]]).to(DEV), cache).cpu()
    assert torch.allclose(got, torch.cat([want["a"][:4], want["b"][:13]]), **F32)
    ctx = harness.context([StepEntry("b", [0] * 17), StepEntry("a", [0] * 8)])
    got = mixer.forward(ctx, torch.cat([xs["b"][13:], xs["a"][4:]]).to(DEV), cache).cpu()
    assert torch.allclose(got, torch.cat([want["b"][13:], want["a"][4:]]), **F32)
    harness.cache.finish("a")           # c takes the slot a leaves, which the manager clears
    assert cache.state.abs().sum(-1).min() > 0
    ctx = harness.context([StepEntry("c", [0] * 5)])
    assert torch.allclose(mixer.forward(ctx, xs["c"].to(DEV), cache).cpu(), want["c"], **F32)


# ---------------------------------------------------------------- feed-forward and branch sum
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,ff,scale", [(5, 3, 24, 1.5), (1, 1, 48, 1.0), (8, 1, 16, 2.0), (6, 6, 32, 0.7), (70, 4, 8, 2.0)])
def test_gelu_expert_mixture_against_plain(dtype, experts, top, ff, scale, monkeypatch):
    from vosti_b200.parts import ExpertMixture
    gen = torch.Generator().manual_seed(experts)
    width, T = 72, 40
    part = build_feed_forward(PartSpec.make("moe", experts=experts, top=top, intermediate_size=ff, float32_out=True, gated=False,
                                            route="softmax_renorm", scale=scale), width)
    assert not any(k.endswith(".gate") for k in part.weight_specs())
    W = weights_of(part, gen)
    W["router"] = rounded(experts, width, gen=gen, std=3.0 / math.sqrt(width))
    give(part, W, dtype)
    x = rounded(T, width, gen=gen)
    block = dict(router=dict(experts=experts, top=top, scale=scale))
    want = plain.expert_mixture(x, {"p." + k: v for k, v in W.items()}, "p.", block)
    tol = 3e-5 if dtype == torch.float32 else 6e-2
    ctx = Ctx(dtype)
    ctx.all_decode = True
    got = part.forward(ctx, x.to(DEV, dtype))
    assert got.dtype == torch.float32 and torch.allclose(got.cpu(), want, atol=tol)
    monkeypatch.setattr(ExpertMixture, "GROUPED_FROM", 16)     # the way long portions take: pairs sorted by expert
    ctx.all_decode = False
    assert torch.allclose(part.forward(ctx, x.to(DEV, dtype)).cpu(), want, atol=tol)
    logits = x @ W["router"].T
    chosen, weights, dense = ops.moe_route(logits.to(DEV), top, over_all=True, scale=scale)
    values, index = torch.topk(torch.softmax(logits, -1), top)
    assert torch.equal(chosen.cpu().long(), index)
    assert torch.allclose(weights.cpu(), values / values.sum(-1, keepdim=True) * scale, atol=1e-5)
    assert torch.allclose(dense.cpu().sum(-1), torch.full((T,), scale), atol=1e-5)
    # the product and the choice in one kernel
    fused = ops.moe_router(x.to(DEV, dtype), W["router"].to(DEV), top, over_all=True, scale=scale, want_logits=True)
    assert torch.equal(fused[0].cpu().long(), index) and torch.allclose(fused[3].cpu(), logits, atol=1e-4)
    assert torch.allclose(fused[1].cpu(), weights.cpu(), atol=1e-5) and torch.allclose(fused[2].cpu(), dense.cpu(), atol=1e-5)


def test_branch_sum():
    gen = torch.Generator().manual_seed(7)
    for width in (136, 67):
        xs = [rounded(5, width, gen=gen, std=s) for s in (0.01, 3.0, 1.0)]
        got = ops.branch_sum([xs[0].to(DEV), xs[1].to(DEV, torch.bfloat16), xs[2].to(DEV)], (0.8, -0.9, 2.0))
        assert torch.allclose(got.cpu(), 0.8 * xs[0] - 0.9 * xs[1] + 2.0 * xs[2], atol=1e-5)


# ---------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (config, rank, seed) in tiny.ALL.items():
        folder = tiny.write_model(tmp_path_factory.mktemp(f"vivesun_{name}"), config, rank, seed)
        out[name] = (folder,) + plain.load_model(folder, torch.float32)
    return out


def prompt(config, n, seed):
    return torch.randint(0, config["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def close_rows(got, want, dtype):
    """float32: every row equal up to rounding order. bfloat16: rows differ by the rounding of
    every product, and a few by a router's close call (one of six experts with weight 2 makes a
    row another row); bound the typical row and the share of rows that are far off."""
    err = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    if dtype == "float32":
        return bool(err.max() < 2e-4)
    return bool(err.median() < 0.03 and (err > 0.1).float().mean() <= 0.05)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_whole_prompt_portions_and_decoding_against_plain(models, name, dtype, monkeypatch):
    from vosti_b200.parts import ExpertMixture
    monkeypatch.setattr(ExpertMixture, "GROUPED_FROM", 16)      # portions of 16 tokens or more sort their pairs by expert
    folder, config, W = models[name]
    tokens = prompt(config, 77, 1)                              # several chunks of every layer
    want = plain.forward(config, W, tokens)
    for sizes in ((77,), (45,) + (1,) * 32, (2, 5, 1, 1, 17, 2, 3, 30, 16)):
        page = tiny.PAGE[name]
        runner = ModelRunner(folder, dtype=dtype, num_pages=96 // page, page_size=page, max_requests=2)
        runner.begin("r")
        rows, at = [], 0
        for size in sizes:
            rows.append(runner.step([StepEntry("r", tokens[at:at + size], list(range(size)))]).cpu())
            at += size
        runner.check_status()
        assert close_rows(torch.cat(rows), want, dtype), sizes


def test_residual_stream_after_every_layer(models):
    folder, config, W = models["a"]
    tokens = prompt(config, 23, 2)
    _, want = plain.forward(config, W, tokens, keep_layers=True)
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
    assert len(streams) == want.shape[0] == 4
    for got, expected in zip(streams, want):
        assert torch.allclose(got, expected, atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "float32"), ("c", "bfloat16"), ("d", "float32")])
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
        if dtype == "float32":
            assert close_rows(torch.cat(got[r]), want[r], dtype), r
    if dtype != "float32":
        # A router's close call moves a row and, through the recurrent state, the rows after it, so
        # against the float32 oracle only the typical row is bounded; the batch itself is compared
        # with each request alone in the same serving type, where only rounding orders differ.
        for r in lengths:
            alone = ModelRunner(folder, dtype=dtype, num_pages=pool, page_size=page, max_requests=1)
            alone.begin(r)
            single = alone.step([StepEntry(r, tokens[r], list(range(lengths[r])))]).cpu()
            mixed = torch.cat(got[r])
            err = (mixed - single).pow(2).mean(-1).sqrt() / single.pow(2).mean().sqrt()
            assert float(err.max()) < 0.03, (r, float(err.max()))
            against = (mixed - want[r]).pow(2).mean(-1).sqrt() / want[r].pow(2).mean().sqrt()
            assert float(against.median()) < 0.03, r
    assert runner.cache.available_pages() == pool and len(runner.cache.free_slots) == 2


@pytest.mark.parametrize("name", ["b", "c"])
def test_long_decoding_keeps_its_state_across_chunks(models, name):
    folder, config, W = models[name]
    tokens = prompt(config, 150, 4)
    want = plain.forward(config, W, tokens)
    page = tiny.PAGE[name]
    runner = ModelRunner(folder, dtype="float32", num_pages=160 // page, page_size=page, max_requests=1)
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
    decode steps, two slots for five requests, so few pages that a request is preempted. The
    token before a step's first one reaches the embedding through the request's state slot, also
    when the newest token is still on the device."""
    folder, config, W = models["a"]
    prompts = [prompt(config, n, 20 + n) for n in (5, 17, 2, 11, 8)]
    want = [plain_greedy(config, W, p, 10) for p in prompts]
    engine = Engine(folder, dtype="float32", num_blocks=9, block_size=4, max_num_seqs=2, max_num_batched_tokens=16,
                    prefill_chunk_size=8, cuda_graphs=cuda_graphs, async_scheduling=async_scheduling)
    assert engine.runner.spec.architecture == "Vivesun" and engine.runner.cache.has_state
    assert (engine.graphs is not None) == cuda_graphs
    got = engine.generate(prompts, max_tokens=10, arrival_steps=[0, 0, 1, 4, 20])
    assert got == want
    assert engine.scheduler.preemptions > 0
    if cuda_graphs:
        assert engine.graphs.replays > 0
    engine.runner.cache.check()
    assert engine.runner.cache.available_pages() == 9 and len(engine.runner.cache.free_slots) == 2
