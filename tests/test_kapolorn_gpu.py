"""Kapolorn through the framework against the plain implementation (``tests/plain/kapolorn_plain.py``): each mechanism
alone, the residual after every layer run, whole prompts, token-by-token decoding through the captured steps, portions
down to two tokens, unequal requests in one batch against each alone, state slots and pages that are given back and used
again, long decoding (blocks pass while tokens are decoded), and greedy generation through the engine's own entry point
and scheduler.  Four small configurations that differ in every size (``kapolorn_configs``); weights are drawn so that
attention is peaked and states remember dozens of tokens, and the tests of the mechanisms alone first show, with the
plain implementation, that a block one position off, a sink left out or a state that forgot its past would be seen.

Tolerances are derived: the float32 engine may be off by a multiple of what float32 arithmetic costs the plain
implementation itself (float32 against float64); the bfloat16 engine by 3 times what rounding the activations to
bfloat16, where a bfloat16 run stores them, costs the plain implementation.  The models' routers are made so that no
choice of experts is a close call (``kapolorn_configs.steady_routing``), and the first token of every prompt so that no
state mixer's answer at position 0 hangs on the sign of a number near zero."""

import functools

import pytest
import torch

from clockwork_b200 import EngineConfig
from clockwork_b200.config import PartSpec
from clockwork_b200.config.registry import spec_from_raw
from clockwork_b200.engine import LLMEngine
from clockwork_b200.engine.trace import TraceSession
from clockwork_b200.parts import ResidualStream, build_part
from clockwork_b200.sampling import SamplingParams
from clockwork_b200.weights.loader import make_fetch
from tests.gpu_tools import DEV, PartHarness
from tests.kapolorn_configs import CONFIGS, draw_weights, write_model
from tests.kapolorn_configs import tokens_for as raw_tokens_for
from tests.plain import kapolorn_plain as plain
from tests.plain.qwen2_plain import read_model_dir
from tests.trace_tools import cut

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    return {name: write_model(tmp_path_factory.mktemp(f"kapolorn_{name}"), name, seed=5 + i, steady=True)
            for i, name in enumerate(sorted(CONFIGS))}


@pytest.fixture(scope="module")
def oracle(dirs):
    """(name, tokens) -> (float64 logits [T, V], what float32 costs, what bfloat16 storage costs).  The run that
    rounds uses the exact run's choices of experts, and no choice of the exact run is a close call."""
    weights = {name: read_model_dir(folder, dtype=torch.float64) for name, folder in dirs.items()}

    @functools.lru_cache(maxsize=None)
    def get(name, tokens):
        config, w = weights[name]
        log = []
        exact = plain.forward(config, w, list(tokens), dtype=torch.float64, log=log)
        assert min(float(margin.min()) for _, margin in log) > 0.2
        single = plain.forward(config, w, list(tokens), dtype=torch.float32).double()
        rounded = plain.forward(config, w, list(tokens), dtype=torch.float64, rnd=plain.to_bfloat16_and_back, routes=log)
        return exact, float((single - exact).abs().max()), float((rounded - exact).abs().max())

    return get


_first_tokens: dict = {}


def tokens_for(config, length, salt=0):
    """A prompt whose first token was chosen, once per configuration, with ``plain.steady_first_token``."""
    tokens = raw_tokens_for(config, length, salt)
    first = _first_tokens.get(config["vocab"])
    if first is not None:
        tokens[0] = first
    return tokens


@pytest.fixture(scope="module", autouse=True)
def steady_first_tokens(dirs):
    for folder in dirs.values():
        config, w = read_model_dir(folder, dtype=torch.float64)
        _first_tokens[config["vocab"]] = plain.steady_first_token(config, w)
    yield
    _first_tokens.clear()


def check(got, name, tokens, dtype, oracle, first=0):
    exact, cost32, cost16 = oracle(name, tuple(tokens))
    diff = (got.double().cpu() - exact[first : first + got.shape[0]]).abs()
    allowed = 30 * cost32 + 1e-5 if dtype == "float32" else 3 * cost16
    worst = float(diff.max())
    assert worst <= allowed, f"{name} {dtype}: off by {worst:.3g} at position {first + int(diff.max(1).values.argmax())}, allowed {allowed:.3g}"


class Replay:
    """Steps through ``TraceSession`` (what ``bin/trace_run`` runs), logits wanted everywhere."""

    def __init__(self, folder, name, dtype, max_tokens, **kw):
        self.session = TraceSession(folder, dtype, max_tokens, page_size=CONFIGS[name][1], **kw)
        self.logits: dict[str, list] = {}
        self.n = 0

    def step(self, portions: dict, end=()):
        record = {"step": self.n, "end": list(end),
                  "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))} for rid, toks in portions.items()]}
        self.n += 1
        out, _ = self.session.run_step(record)
        row = 0
        for rid, toks in portions.items():
            self.logits.setdefault(rid, []).append(torch.from_numpy(out[row : row + len(toks)].copy()))
            row += len(toks)

    def of(self, rid):
        return torch.cat(self.logits[rid])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt(name, dtype, dirs, oracle):
    tokens = tokens_for(CONFIGS[name][0], 75, salt=1)
    run = Replay(dirs[name], name, dtype, 128)
    run.step({"a": tokens}, end=["a"])
    check(run.of("a"), name, tokens, dtype, oracle)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_residual_after_every_layer_run(name, dirs):
    """float32, kernel by kernel: a looped layer counts each time it runs."""
    config, w = read_model_dir(dirs[name], dtype=torch.float64)
    tokens = tokens_for(config, 40, salt=11)
    _, want = plain.forward(config, w, tokens, dtype=torch.float64, keep_layers=True)
    _, single = plain.forward(config, w, tokens, dtype=torch.float32, keep_layers=True)
    run = Replay(dirs[name], name, "float32", 64, graphs=False)
    seen = []
    for block in run.session.model.blocks:
        def wrapped(ctx, stream, view, *args, _inner=block.forward, **kw):
            out = _inner(ctx, stream, view, *args, **kw)
            stream.flush()
            seen.append(stream.residual.clone())
            return out
        block.forward = wrapped
    run.step({"a": tokens}, end=["a"])
    assert len(seen) == want.shape[0] == len(plain.run_order(config))
    for r, got in enumerate(seen):
        allowed = 30 * float((single[r].double() - want[r]).abs().max()) + 1e-5
        assert float((got.double().cpu() - want[r]).abs().max()) <= allowed, f"layer run {r}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_then_token_by_token(name, dtype, dirs, oracle):
    """The decoded tokens run through the captured single-token steps; the first tokens of a sequence too (a prompt
    of one token).  70 tokens pass every block but the longest."""
    tokens = tokens_for(CONFIGS[name][0], 70, salt=2)
    for prompt in (9, 1):
        run = Replay(dirs[name], name, dtype, 128)
        run.step({"a": tokens[:prompt]})
        for t in tokens[prompt:]:
            run.step({"a": [t]})
        assert run.session.uses_graphs
        check(run.of("a"), name, tokens, dtype, oracle)


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_of_many_sizes(name, dtype, graphs, dirs, oracle):
    """Cuts in the middle of pages and of blocks, portions of two and three tokens, of one page, longer than a block."""
    tokens = tokens_for(CONFIGS[name][0], 90, salt=3)
    for sizes in ([2, 3, 1, 7, 2, 16, 5, 4], [37, 2, 2, 2, 30, 1, 1, 3]):
        run = Replay(dirs[name], name, dtype, 128, graphs=graphs)
        for portion in cut(tokens, sizes):
            run.step({"a": portion})
        check(run.of("a"), name, tokens, dtype, oracle)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_requests_in_one_batch_against_each_alone(name, dtype, dirs, oracle):
    config = CONFIGS[name][0]
    prompts = {"p": tokens_for(config, 61, salt=4), "q": tokens_for(config, 23, salt=5), "r": tokens_for(config, 40, salt=6),
               "s": tokens_for(config, 9, salt=7)}
    plans = {"p": [17, 2, 1, 1, 30, 1, 1, 1, 7], "q": [1, 1, 1, 5, 1, 2, 12], "r": [40], "s": [2, 1, 1, 1, 1, 1, 1, 1]}
    cuts = {rid: cut(toks, plans[rid]) for rid, toks in prompts.items()}
    together = Replay(dirs[name], name, dtype, 4 * 64)
    for i in range(max(len(c) for c in cuts.values())):
        step = {rid: c[i] for rid, c in cuts.items() if i < len(c)}
        together.step(step, end=[rid for rid, c in cuts.items() if i == len(c) - 1])
    for rid, toks in prompts.items():
        alone = Replay(dirs[name], name, dtype, 64)
        for portion in cuts[rid]:
            alone.step({rid: portion})
        if dtype == "float32":  # a row's result does not depend on the rest of the batch at all
            assert torch.equal(together.of(rid), alone.of(rid)), rid
        check(together.of(rid), name, toks, dtype, oracle)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_slots_and_pages_given_back_and_used_again(name, dtype, dirs, oracle):
    """Ten requests through four state slots and a pool of pages for 4 x 64 tokens: a request that takes a slot or a
    page that another one left starts from zero state and sees none of the other's keys."""
    config = CONFIGS[name][0]
    run = Replay(dirs[name], name, dtype, 4 * 64)
    prompts = {f"r{i}": tokens_for(config, 20 + 4 * i, salt=20 + i) for i in range(10)}
    waiting, live, at = list(prompts), [], {}
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
            at[live[-1]] = 0
        step, done = {}, []
        for k, rid in enumerate(live):
            n = min([13, 1, 2, 5][(k + at[rid]) % 4], len(prompts[rid]) - at[rid])
            step[rid] = prompts[rid][at[rid] : at[rid] + n]
            at[rid] += n
            if at[rid] == len(prompts[rid]):
                done.append(rid)
        run.step(step, end=done)
        live = [rid for rid in live if rid not in done]
    run.session.cache.check_invariants()
    assert not run.session.cache.requests and run.session.cache.state.num_free == 4
    for rid, toks in prompts.items():
        check(run.of(rid), name, toks, dtype, oracle)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_in_a_pool_that_only_passed_blocks_make_enough(dtype, dirs, oracle):
    """300 decoded tokens behind a short prompt: blocks of 21 and of 7 positions begin and end among decoded tokens,
    states are carried 300 times through every pass of the looped layer, and the pages of passed blocks go back to the
    pool while the request runs."""
    name = "A"
    tokens = tokens_for(CONFIGS[name][0], 320, salt=8)
    run = Replay(dirs[name], name, dtype, 320)
    run.step({"a": tokens[:20]})
    for t in tokens[20:]:
        run.step({"a": [t]})
    req = run.session.cache.get("a")
    assert all(sum(p >= 0 for p in table) <= 21 // 4 + 2 for table in req.tables)
    check(run.of("a"), name, tokens, dtype, oracle)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_greedy_generation_through_the_engine(name, dtype, dirs):
    """The engine's own entry point and scheduler: prompts cut under a small token budget, several requests at once."""
    config, page, _ = CONFIGS[name]
    cfg = EngineConfig.defaults(str(dirs[name]), dtype=dtype, block_size=page, num_blocks=256, max_model_len=256, max_num_seqs=4,
                                max_num_batched_tokens=24)
    engine = LLMEngine(cfg)
    prompts = [tokens_for(config, n, salt=30 + n) for n in (5, 31, 18, 1, 44)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    _, w = read_model_dir(dirs[name], dtype=torch.float64)
    for prompt, out in zip(prompts, outs):
        got = list(out.token_ids)
        log = []
        logits = plain.forward(config, w, prompt + got, dtype=torch.float64, log=log)
        single = plain.forward(config, w, prompt + got, dtype=torch.float32).double()
        rounded = plain.forward(config, w, prompt + got, dtype=torch.float64, rnd=plain.to_bfloat16_and_back, routes=log)
        # every token is within rounding of the best one, given the engine's own history
        yard = 60 * float((single - logits).abs().max()) + 2e-5 if dtype == "float32" else 6 * float((rounded - logits).abs().max())
        for i, token in enumerate(got):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[token]) <= yard
        if dtype == "float32" and all(float(r.topk(2).values.diff().abs()) > yard for r in logits[len(prompt) - 1 : -1]):
            assert got == plain.greedy_generate(config, w, prompt, 12)


# ---- every mechanism alone ----------------------------------------------------------------------------

def part_with_weights(category, spec, prefix, dtype, tensors):
    part = build_part(category, spec, prefix, dtype, DEV)
    decls = {d.name: d for d in part.tensor_decls()}
    assert set(decls) == set(tensors), (sorted(decls), sorted(tensors))
    part.load_weights(make_fetch(lambda n: tensors[n], decls, dtype, DEV))
    return part


def run_mixer(part, x, portions, page_size=4, num_pages=128):
    """The mixer's output for every row of ``x`` [T, W] (the weighted sum of the terms it hands to the norm behind
    it), fed in portions through a cache of its own."""
    harness = PartHarness({0: part.cache_need()}, part.dtype, num_pages=num_pages, page_size=page_size, slots=2)
    out, at = [], 0
    for n in portions:
        prepared = harness.prepare({"a": n})
        terms = part.mix_terms(prepared.ctx, x[at : at + n].to(DEV, part.dtype).contiguous(), prepared.ctx.views[0])
        total = sum(factor * term.float() for term, factor in terms)
        harness.commit(prepared)
        out.append(total.cpu())
        at += n
    assert at == x.shape[0]
    return torch.cat(out)


def draw(gen, shape, scale=1.0, shift=0.0):
    return (shift + scale * torch.randn(shape, generator=gen)).to(torch.bfloat16).float()


def assert_close(got, want, what, rel=3e-5):
    """float32 arithmetic against float64: a few units of float32 rounding of the largest value, per term summed."""
    worst, allowed = float((got.double() - want).abs().max()), 2e-4 + rel * float(want.abs().max())
    assert worst <= allowed, f"{what}: off by {worst:.3g}, allowed {allowed:.3g}"


def attention_tensors(gen, w, heads, kv_heads, dim, vdim):
    return {"m.q": draw(gen, (heads * dim, w), 0.5), "m.k": draw(gen, (kv_heads * dim, w), 0.5), "m.v": draw(gen, (kv_heads * vdim, w), 0.3),
            "m.o": draw(gen, (w, heads * vdim), 0.2), "m.sink": draw(gen, (heads,), 1.0, 1.0)}


def attention_spec(w, heads, kv_heads, dim, vdim, block, scale, rot, base):
    return PartSpec("window_attention", dict(hidden_size=w, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, window=block, scale=scale,
                                             mask="block", sink=True, weights="softmax", rotary={"dims": rot, "base": base}))


def attention_config(heads, kv_heads, dim, vdim, block, scale, rot, base):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, mask={"size": block}, rot={"dims": rot, "base": base})


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, block, rot, base, page", [
    (4, 2, 24, 12, 21, 8, 1000.0, 4), (3, 1, 16, 40, 7, 16, 50000.0, 8), (6, 6, 8, 8, 1, 2, 10000.0, 4), (2, 2, 12, 20, 400, 12, 100.0, 16),
    (8, 2, 32, 64, 100, 32, 10000.0, 16), (5, 5, 16, 24, 64, 4, 300.0, 16), (12, 3, 48, 80, 60, 16, 500000.0, 16), (33, 11, 8, 4, 10, 6, 20.0, 4)])
def test_blocked_attention_with_rotation_and_a_sink_alone(heads, kv_heads, dim, vdim, block, rot, base, page):
    """300 positions whole, token by token and in portions that cut pages and blocks.  First the plain implementation
    shows that the edge, the sink and the rotation count: a block one position shorter or longer, a sink far below the
    scores, or another base moves the result by far more than the test allows."""
    gen = torch.Generator().manual_seed(heads * 100 + block)
    w, scale = 48, 0.4
    t = attention_tensors(gen, w, heads, kv_heads, dim, vdim)
    wd = {k: v.double() for k, v in t.items()}
    x = draw(gen, (300, w))
    m = attention_config(heads, kv_heads, dim, vdim, block, scale, rot, base)
    want = plain.blocked_sink_attention(x.double(), wd, "m", m)
    for other in (block - 1, block + 1):
        if 1 <= other < 300:
            assert float((plain.blocked_sink_attention(x.double(), wd, "m", dict(m, mask={"size": other})) - want).abs().max()) > 0.05
    assert float((plain.blocked_sink_attention(x.double(), dict(wd, **{"m.sink": wd["m.sink"] - 60.0}), "m", m) - want).abs().max()) > 0.05
    if block > 1:
        assert float((plain.blocked_sink_attention(x.double(), wd, "m", dict(m, rot={"dims": rot, "base": base * 3})) - want).abs().max()) > 0.01
    part = part_with_weights("mixer", attention_spec(w, heads, kv_heads, dim, vdim, block, scale, rot, base), "m", torch.float32, t)
    # few enough pages that the ones of passed blocks must come back for the run to finish
    pages = (max(min(block, 300), 131) + 2 * page) // page + 4
    for portions in ([131, 169], [1] * 300, [2, 3, 1, 1, 9, 2, 5, 41, 100, 1, 1, 1, 131, 2], [page - 1, 2, page, 1, 300 - 2 * page - 2]):
        assert sum(portions) == 300
        got = run_mixer(part, x, portions, page_size=page, num_pages=pages + max(portions) // page)
        assert_close(got, want, portions)


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, block, rot, page", [
    (4, 4, 256, 256, 100, 128, 16), (8, 8, 256, 256, 64, 128, 64), (16, 1, 64, 64, 4096, 64, 16), (8, 2, 128, 128, 150, 64, 16),
    (6, 3, 96, 48, 45, 32, 8), (4, 1, 240, 200, 70, 16, 16), (2, 2, 512, 64, 90, 256, 16), (4, 4, 32, 256, 33, 32, 16)])
def test_blocked_attention_in_bfloat16_at_sizes_that_take_each_arrangement_of_the_tensor_core_kernel(heads, kv_heads, dim, vdim, block, rot, page):
    """Key/value tiles in two stages and in one (wide heads: blocks of several tiles must fetch every tile), several key/value
    heads a block and one, wide values; whole and in portions, against the plain implementation in float64; allowed is 3
    times what rounding q, k, v and the output to bfloat16 costs the plain implementation."""
    gen = torch.Generator().manual_seed(heads * 100 + block)
    w, scale = 64, dim ** -0.5
    t = attention_tensors(gen, w, heads, kv_heads, dim, vdim)
    wd = {k: v.double() for k, v in t.items()}
    x = draw(gen, (260, w))
    m = attention_config(heads, kv_heads, dim, vdim, block, scale, rot, 10000.0)
    want = plain.blocked_sink_attention(x.double(), wd, "m", m)
    rounded = plain.blocked_sink_attention(x.double(), wd, "m", m, rnd=plain.to_bfloat16_and_back)
    allowed = 3 * float((rounded - want).abs().max())
    assert allowed < 0.1 * float(want.abs().max())
    part = part_with_weights("mixer", attention_spec(w, heads, kv_heads, dim, vdim, block, scale, rot, 10000.0), "m", torch.bfloat16, t)
    for portions in ([260], [200] + [1] * 60, [3, 64, 1, 61, 2, 109] + [1] * 20):
        got = run_mixer(part, x, portions, page_size=page, num_pages=600 // page + 8)
        worst = float((got.double() - want).abs().max())
        assert worst <= allowed, f"{portions[:6]}: off by {worst:.3g}, allowed {allowed:.3g}"


def test_one_key_that_stands_out_at_either_side_of_a_block_edge():
    """A query and two keys are made so that one score towers over all others, the sink too: the key at the first
    position of the query's block takes the whole softmax, the key one further back (the last of the block before)
    must not be seen at all, in a prompt and in decoding, also where a portion ends at the edge.  The entries that
    carry the signal are not rotated."""
    heads, kv_heads, dim, vdim, block, w, rot = 2, 1, 16, 8, 37, 32, 4
    gen = torch.Generator().manual_seed(9)
    t = attention_tensors(gen, w, heads, kv_heads, dim, vdim)
    x = draw(gen, (120, w), 0.05)
    probe, inside, outside = 100, 74, 73
    assert probe // block == inside // block == outside // block + 1
    x[probe, 3] += 40.0    # every unrotated query channel reads coordinate 3, every unrotated key channel coordinate 5
    x[inside, 5] += 40.0
    x[outside, 5] += 80.0  # would win if it were visible
    t["m.q"].view(heads, dim, w)[:, rot:, 3] = 0.5
    t["m.k"].view(kv_heads, dim, w)[:, rot:, 5] = 0.5
    t["m.q"].view(heads, dim, w)[:, :rot, 3] = 0.0
    t["m.k"].view(kv_heads, dim, w)[:, :rot, 5] = 0.0
    wd = {k: v.double() for k, v in t.items()}
    m = attention_config(heads, kv_heads, dim, vdim, block, 1.0, rot, 1000.0)
    want = plain.blocked_sink_attention(x.double(), wd, "m", m)
    v_inside = (x[inside].double() @ wd["m.v"].T).repeat(heads) @ wd["m.o"].T
    assert float((want[probe] - v_inside).abs().max()) < 1e-6  # the edge key alone
    part = part_with_weights("mixer", attention_spec(w, heads, kv_heads, dim, vdim, block, 1.0, rot, 1000.0), "m", torch.float32, t)
    for portions in ([120], [probe, 1, 19], [inside, 20, 6, 1, 19], [outside, 1, 1, 25, 1, 19], [70] + [1] * 50):
        got = run_mixer(part, x, portions, page_size=8)
        assert_close(got, want, portions)


def test_a_key_far_back_in_a_long_block_and_the_sink_against_a_lone_key():
    """A block longer than the sequence: the key at position 3 stands out for a query 650 positions on, among
    hundreds, whole, decoded, and over portions.  And the first token of a sequence shares the softmax with the sink
    alone: with a sink as large as its score it gets half."""
    heads, kv_heads, dim, vdim, block, w, rot = 4, 2, 32, 16, 1000, 32, 8
    gen = torch.Generator().manual_seed(10)
    t = attention_tensors(gen, w, heads, kv_heads, dim, vdim)
    x = draw(gen, (700, w), 0.05)
    x[653, 3] += 30.0
    x[3, 5] += 30.0
    for name, col, count in (("m.q", 3, heads), ("m.k", 5, kv_heads)):
        t[name].view(count, dim, w)[:, rot:, col] = 0.5
        t[name].view(count, dim, w)[:, :rot, col] = 0.0
    t["m.sink"] = torch.zeros(heads)
    wd = {k: v.double() for k, v in t.items()}
    m = attention_config(heads, kv_heads, dim, vdim, block, 1.0, rot, 10000.0)
    want = plain.blocked_sink_attention(x.double(), wd, "m", m)
    v_far = (x[3].double() @ wd["m.v"].T).reshape(kv_heads, vdim).repeat_interleave(heads // kv_heads, 0).reshape(-1) @ wd["m.o"].T
    assert float((want[653] - v_far).abs().max()) < 1e-6
    q0 = (x[0].double() @ wd["m.q"].T).reshape(heads, dim)
    k0 = (x[0].double() @ wd["m.k"].T).reshape(kv_heads, dim).repeat_interleave(heads // kv_heads, 0)
    t["m.sink"] = (q0 * k0).sum(-1).float()  # position 0 is not rotated: the sink ties with the only key
    wd = {k: v.double() for k, v in t.items()}
    want = plain.blocked_sink_attention(x.double(), wd, "m", m)
    v_first = (x[0].double() @ wd["m.v"].T).reshape(kv_heads, vdim).repeat_interleave(heads // kv_heads, 0).reshape(-1) @ wd["m.o"].T
    assert float((want[0] - 0.5 * v_first).abs().max()) < 1e-4 * float(v_first.abs().max()) + 1e-6
    part = part_with_weights("mixer", attention_spec(w, heads, kv_heads, dim, vdim, block, 1.0, rot, 10000.0), "m", torch.float32, t)
    for portions in ([700], [640] + [1] * 60, [1, 4, 300, 345, 3, 1, 46]):
        got = run_mixer(part, x, portions, page_size=16)
        assert_close(got, want, portions)


def memory_tensors(gen, w, heads, dim, vdim, in_bias):
    return {"m.q": draw(gen, (heads * dim, w), 0.3), "m.k": draw(gen, (heads * dim, w), 0.3), "m.v": draw(gen, (heads * vdim, w), 0.3),
            "m.g": draw(gen, (heads * vdim, w), 0.2), "m.i": draw(gen, (heads, w), 0.3), "m.f": draw(gen, (heads, w), 0.3),
            "m.i.b": draw(gen, (heads,), 1.0, in_bias), "m.f.b": draw(gen, (heads,), 1.0, 3.0), "m.norm": draw(gen, (heads * vdim,), 0.2, 1.0),
            "m.o": draw(gen, (w, heads * vdim), 0.1)}


@pytest.mark.parametrize("heads, dim, vdim, cap, in_bias", [(3, 20, 12, 8.0, 0.0), (1, 24, 8, 15.0, -6.0), (4, 8, 16, 2.0, 1.0), (2, 64, 32, 10.0, 4.0),
                                                            (2, 16, 130, 20.0, -2.0), (16, 64, 128, 15.0, 0.0)])
def test_matrix_memory_alone(heads, dim, vdim, cap, in_bias):
    """Input gates far below the forget gates (the running maximum then stays where the forget gate puts it, from the
    zero it starts at, not at the first input gate), far above, and a cap that the gates reach.  First the plain
    implementation shows that the past and the cap count."""
    gen = torch.Generator().manual_seed(dim + vdim)
    w = 40
    t = memory_tensors(gen, w, heads, dim, vdim, in_bias)
    cfg = dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap)
    part = part_with_weights("mixer", PartSpec("matrix_memory", dict(cfg, hidden_size=w, eps=1e-5)), "m", torch.float32, t)
    x = draw(gen, (150, w))
    wd = {k: v.double() for k, v in t.items()}
    want = plain.matrix_memory_mixer(x.double(), wd, "m", cfg, 1e-5)
    assert float((plain.matrix_memory_mixer(x.double()[100:], wd, "m", cfg, 1e-5) - want[100:]).abs().max()) > 0.02
    assert float((plain.matrix_memory_mixer(x.double(), wd, "m", dict(cfg, gate_cap=cap / 2), 1e-5) - want).abs().max()) > 1e-3
    for portions in ([150], [1] * 150, [2, 1, 3, 2, 42, 17, 16, 1, 66]):
        got = run_mixer(part, x, portions)
        assert_close(got, want, portions)


@pytest.mark.parametrize("heads, dim, vdim, rows", [(3, 8, 8, 1500), (16, 8, 4, 700), (40, 4, 4, 260), (1, 16, 8, 2300)])
def test_matrix_memory_over_long_portions(heads, dim, vdim, rows):
    """The gates' kernel stages a fixed number of (token, head) pairs at a time: portions longer than one stage, for few and
    many heads, whole and cut where no stage ends, against the plain implementation."""
    gen = torch.Generator().manual_seed(heads + rows)
    w = 24
    t = memory_tensors(gen, w, heads, dim, vdim, 0.5)
    cfg = dict(heads=heads, dim=dim, vdim=vdim, gate_cap=12.0)
    part = part_with_weights("mixer", PartSpec("matrix_memory", dict(cfg, hidden_size=w, eps=1e-5)), "m", torch.float32, t)
    x = draw(gen, (rows, w))
    want = plain.matrix_memory_mixer(x.double(), {k: v.double() for k, v in t.items()}, "m", cfg, 1e-5)
    for portions in ([rows], [rows - 701 // heads - 5, 701 // heads, 3, 1, 1]):
        got = run_mixer(part, x, portions, page_size=16, num_pages=8)
        assert_close(got, want, portions[:2], rel=1e-4)


def delta_tensors(gen, w, heads, kv_heads, dim, vdim, taps, rank):
    conv = lambda rows: draw(gen, (rows, taps), 0.5) + (torch.arange(taps) == taps - 1).float()  # noqa: E731
    return {"m.q": draw(gen, (kv_heads * dim, w), 0.3), "m.k": draw(gen, (kv_heads * dim, w), 0.3), "m.v": draw(gen, (heads * vdim, w), 0.3),
            "m.q.conv": conv(kv_heads * dim), "m.k.conv": conv(kv_heads * dim), "m.v.conv": conv(heads * vdim),
            "m.b": draw(gen, (heads, w), 0.3), "m.A_log": draw(gen, (heads,), 0.5, -1.5), "m.dt_bias": draw(gen, (heads * dim,), 1.0, -2.0),
            "m.a1": draw(gen, (rank, w), 0.3), "m.a2": draw(gen, (heads * dim, rank), 0.5), "m.g1": draw(gen, (rank + 1, w), 0.3),
            "m.g2": draw(gen, (heads * vdim, rank + 1), 0.5), "m.norm": draw(gen, (vdim,), 0.2, 1.0), "m.o": draw(gen, (w, heads * vdim), 0.1)}


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, taps, rank", [(4, 2, 12, 20, 3, 5), (3, 3, 8, 8, 1, 8), (2, 1, 40, 8, 4, 3), (5, 5, 8, 24, 2, 7),
                                                                    (4, 2, 64, 48, 4, 24), (16, 16, 128, 128, 4, 16), (6, 1, 16, 130, 5, 4)])
def test_delta_rule_with_channel_decays_alone(heads, kv_heads, dim, vdim, taps, rank):
    gen = torch.Generator().manual_seed(dim * vdim + taps)
    w = 40
    t = delta_tensors(gen, w, heads, kv_heads, dim, vdim, taps, rank)
    cfg = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=taps)
    part = part_with_weights("mixer", PartSpec("channel_delta", dict(cfg, hidden_size=w, eps=1e-5)), "m", torch.float32, t)
    x = draw(gen, (150, w))
    wd = {k: v.double() for k, v in t.items()}
    want = plain.channel_delta_mixer(x.double(), wd, "m", cfg, 1e-5)
    assert float((plain.channel_delta_mixer(x.double()[100:], wd, "m", cfg, 1e-5) - want[100:]).abs().max()) > 0.02
    for portions in ([150], [1] * 150, [2, 1, 3, 2, 42, 17, 16, 1, 66]):
        got = run_mixer(part, x, portions)
        assert_close(got, want, portions)


def moe_tensors(gen, w, ff, experts, shared):
    t = {"f.router": draw(gen, (experts, w), 3.0 / w ** 0.5)}
    for e in range(experts):
        t.update({f"f.e{e}.gate": draw(gen, (ff, w), 0.3), f"f.e{e}.up": draw(gen, (ff, w), 0.3), f"f.e{e}.down": draw(gen, (w, ff), 0.2)})
    if shared is not None:
        t.update({"f.shared.gate": draw(gen, (shared[0], w), 0.3), "f.shared.up": draw(gen, (shared[0], w), 0.3),
                  "f.shared.down": draw(gen, (w, shared[0]), 0.2)})
    return t


@pytest.mark.parametrize("ff, limit, experts, top, groups, shared", [
    (40, 1.5, 6, 3, (3, 2), (56, 2.5)), (24, 1.0, 4, 1, (2, 1), None), (32, 2.0, 3, 3, None, None), (16, 1.0, 4, 2, (4, 2), None),
    (96, 1.0, 16, 4, (2, 1), (64, 1.5)), (28, 1.2, 8, 3, (4, 2), (36, 1.8)), (20, 0.5, 5, 2, (1, 1), (24, 3.0)), (128, 7.0, 32, 4, (4, 2), (192, 7.0))])
def test_routed_experts_in_groups_with_a_shared_expert_alone(ff, limit, experts, top, groups, shared):
    """Steps of 150, 7 and 1 rows.  Inputs are wide enough that the clamps bite; the plain implementation shows that the
    limit, the groups and the shared expert count.  Rows whose choice is closer than 1e-3 in router logits are left out
    (float32 against float64 may then differ in the choice)."""
    gen = torch.Generator().manual_seed(ff + experts)
    w = 48
    t = moe_tensors(gen, w, ff, experts, shared)
    wd = {k: v.double() for k, v in t.items()}
    m = {"expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    params = dict(hidden_size=w, expert_size=ff, limit=limit, experts=experts, top=top, scoring="all", router_bias=False)
    if groups is not None:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
        params.update(groups=groups[0], keep=groups[1])
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
        params["shared"] = {"size": shared[0], "limit": shared[1]}
    part = part_with_weights("ffn", PartSpec("moe", params), "f", torch.float32, t)
    x = draw(gen, (158, w), 2.0)
    log = []
    want = plain.mixture_of_experts(x.double(), wd, "f", m, log=log)
    sure = log[0][1] > 1e-3
    assert int(sure.sum()) > 140
    assert float((plain.mixture_of_experts(x.double(), wd, "f", dict(m, expert={"ff": ff, "limit": 3 * limit})) - want).abs().max()) > 0.05
    if groups is not None and groups[1] < groups[0] < experts and top > 1:
        free = dict(m, router={"experts": experts, "top": top})
        assert float((plain.mixture_of_experts(x.double(), wd, "f", free) - want).abs().max()) > 0.05
    if shared is not None:
        assert float((plain.mixture_of_experts(x.double(), wd, "f", {k: v for k, v in m.items() if k != "shared"}) - want).abs().max()) > 0.05
    harness = PartHarness({}, torch.float32)
    at = 0
    for n in (150, 7, 1):
        prepared = harness.prepare({"a": n})
        terms = part.output_terms(prepared.ctx, x[at : at + n].to(DEV).contiguous())
        got = sum(factor * term.float() for term, factor in terms).cpu()
        harness.commit(prepared)
        rows = sure[at : at + n]
        assert_close(got[rows], want[at : at + n][rows], (n, "rows"))
        at += n


@pytest.mark.parametrize("rows, ff, w, limit", [(1, 56, 48, 2.5), (7, 8, 72, 0.7), (150, 192, 320, 1.0), (600, 1536, 512, 7.0), (2100, 256, 1024, 1.5)])
def test_the_clamped_gated_product_on_the_tensor_cores(rows, ff, w, limit):
    """The shared expert's first two products with the clamped activation in their epilogue (the tcgen05 kernels: single
    tokens, split tiles, prompt portions) against float32 arithmetic on the same bfloat16 operands; inputs wide enough
    that all three clamps bite."""
    from clockwork_b200.ops import gemm as gemm_ops

    gen = torch.Generator().manual_seed(rows + ff)
    x = draw(gen, (rows, w), 1.5).to(torch.bfloat16).to(DEV)
    wg, wu = (draw(gen, (ff, w), 0.7 * limit / (1.5 * w ** 0.5)).to(torch.bfloat16).to(DEV) for _ in range(2))  # products of 0.7 limit
    got = gemm_ops.clamped_gated_tc(x, wg, wu, limit)
    assert got is not None and got.dtype == torch.bfloat16
    a, b = x.float() @ wg.float().T, x.float() @ wu.float().T
    assert float((a > limit).float().mean()) > 0.02 and float((b.abs() > limit).float().mean()) > 0.04
    a, b = a.clamp(max=limit), b.clamp(-limit, limit)
    want = a * torch.sigmoid(1.702 * a) * (b + 1)
    assert float((got.float() - want).abs().max()) <= 2 ** -8 * float(want.abs().max()) + 1e-3


@pytest.mark.parametrize("name, layer", [("A", 0), ("A", 2), ("B", 1), ("B", 2), ("D", 1)])
def test_the_two_mixers_side_by_side_alone(name, layer):
    """Pages for the one and a state slot for the other in the same layer; the two outputs with their factors."""
    config, page, rank = CONFIGS[name]
    assert config["layers"][layer]["type"] == "parallel"
    prefix = f"l{layer}.mix"
    t = {k: v.float() for k, v in draw_weights(config, rank, seed=2).items() if k.startswith(prefix + ".")}
    part = part_with_weights("mixer", spec_from_raw(config).layers[layer].mixer, prefix, torch.float32, t)
    gen = torch.Generator().manual_seed(6)
    x = draw(gen, (60, config["width"]))
    m, eps = config["layers"][layer]["mixer"], config["norm"]["eps"]
    wd = {k: v.double() for k, v in t.items()}
    want = plain.side_by_side(x.double(), wd, prefix, m, eps)
    assert float((plain.side_by_side(x.double(), wd, prefix, dict(m, left_scale=m["left_scale"] + 0.5), eps) - want).abs().max()) > 0.02
    assert float((plain.side_by_side(x.double(), wd, prefix, dict(m, right_scale=m["right_scale"] + 0.5), eps) - want).abs().max()) > 0.02
    for portions in ([60], [1] * 60, [7, 2, 30, 1, 20]):
        got = run_mixer(part, x, portions, page_size=page)
        assert_close(got, want, portions)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_two_mixers_on_two_streams_change_nothing(dtype, dirs):
    """The attention's kernels run on a second stream beside the matrix memory's: the same bits as one after the other,
    in prompts, portions and captured single-token steps."""
    from clockwork_b200.parts.side_by_side import SideBySide

    name = "D"
    tokens = tokens_for(CONFIGS[name][0], 120, salt=15)
    results = []
    for concurrent in (True, False):
        SideBySide.concurrent = concurrent
        try:
            run = Replay(dirs[name], name, dtype, 256)
            for portion in cut(tokens, [70, 3, 17, 1, 1, 1, 1, 1, 25]):
                run.step({"a": portion})
            results.append(run.of("a"))
        finally:
            SideBySide.concurrent = True
    assert torch.equal(results[0], results[1])


def test_capped_logits_and_the_embedding_as_the_head():
    """Logits far beyond the cap: rows of the embedding are made long, so that the products reach several times the
    cap and the bend shows in every row; the head is the embedding without its scale."""
    import copy
    import json
    import tempfile
    from pathlib import Path

    from clockwork_b200.weights import save_safetensors

    config, page, rank = copy.deepcopy(CONFIGS["B"])
    config["logit_softcap"] = 3.0
    weights = draw_weights(config, rank, seed=4)
    weights["embed"] = (weights["embed"].float() * 4.0).to(torch.bfloat16)
    tokens = raw_tokens_for(config, 30, salt=2)
    wd = {k: v.double() for k, v in weights.items()}
    want = plain.forward(config, wd, tokens, dtype=torch.float64)
    uncapped = plain.forward(dict(config, logit_softcap=None), wd, tokens, dtype=torch.float64)
    assert float(uncapped.abs().max()) > 9.0 and float(want.abs().max()) <= 3.0
    single = plain.forward(config, wd, tokens, dtype=torch.float32).double()
    with tempfile.TemporaryDirectory() as folder:
        (Path(folder) / "config.json").write_text(json.dumps(config))
        save_safetensors(Path(folder) / "model.safetensors", weights)
        session = TraceSession(folder, "float32", 64, page_size=page)
        out, _ = session.run_step({"step": 0, "end": ["a"], "entries": [{"id": "a", "tokens": tokens, "want": list(range(30))}]})
    worst = float((torch.from_numpy(out.copy()).double() - want).abs().max())
    assert worst <= 30 * float((single - want).abs().max()) + 1e-5


@pytest.mark.timeout(600)
def test_a_step_at_layer_sizes_of_a_real_model():
    """Four layers at 2,048 width (three pairs of blocked attention and matrix memory, one delta-rule layer, 32 experts):
    a prompt portion that passes a block edge and single-token steps through the captured graphs agree with the same
    steps launched kernel by kernel."""
    from clockwork_b200.cache import CacheManager
    from clockwork_b200.cli import shape_config
    from clockwork_b200.engine import ModelRunner, StepEntry, random_model

    raw = shape_config("kapolorn-2k", 4)
    model = random_model(raw, seed=3, dtype="bfloat16", device=DEV)
    prompt = raw_tokens_for({"vocab": raw["vocab"]}, 1300, salt=9)
    tail = raw_tokens_for({"vocab": raw["vocab"]}, 3, salt=10)
    results = []
    for graphs in (True, False):
        cache = CacheManager(model.cache_needs(), num_pages=128, page_size=16, dtype=model.dtype, device=DEV, num_state_slots=2)
        runner = ModelRunner(model, cache)
        if graphs:
            assert runner.enable_graphs(max_ctx=2048, max_batch=2)
        cache.open("a")
        rows = [runner.step([StepEntry("a", prompt, [len(prompt) - 1])]).float().cpu()]
        for t in tail:
            entry = [StepEntry("a", [t], [0])]
            if graphs:
                runner.decode_with_graph(entry, None)
                rows.append(runner.last_graph.logits[:1].float().cpu())
            else:
                rows.append(runner.step(entry).float().cpu())
        runner.check_status()
        assert not graphs or runner.graphs
        results.append(torch.cat(rows))
    assert torch.isfinite(results[0]).all()
    scale = float(results[1].abs().max())
    assert float((results[0] - results[1]).abs().max()) <= 0.02 * scale
