"""Nuzulorn through the framework against the plain implementation (``tests/plain/nuzulorn_plain.py``): each mechanism
alone, the residual behind every layer, whole prompts, token-by-token decoding through the captured steps, portions down
to two tokens, unequal requests in one batch against each alone, state slots and pages that are given back and used again,
long decoding (windows and blocks pass while tokens are decoded), and greedy generation through the engine's own entry
point and scheduler.  Four small configurations that differ in every size (``nuzulorn_configs``); weights are drawn so that
attention is peaked and states remember dozens of tokens, and the tests of the mechanisms alone first show, with the plain
implementation, that a window one position off, a block seen too early or too late, a sink left out or a state that forgot
its past would be seen.

Tolerances are derived: the float32 engine may be off by a multiple of what float32 arithmetic costs the plain
implementation itself (float32 against float64); the bfloat16 engine by 3 times what rounding the activations to bfloat16,
where a bfloat16 run stores them, costs the plain implementation.  The models' routers are made so that no choice of
experts is a close call (``nuzulorn_configs.steady_routing``; the margins are asserted)."""

import functools
import math

import pytest
import torch

from clockwork_b200 import EngineConfig, ops
from clockwork_b200.config import PartSpec
from clockwork_b200.engine import LLMEngine
from clockwork_b200.engine.trace import TraceSession
from clockwork_b200.parts import build_part
from clockwork_b200.sampling import SamplingParams
from clockwork_b200.weights.loader import make_fetch
from tests.gpu_tools import DEV, PartHarness
from tests.nuzulorn_configs import CONFIGS, tokens_for, write_model
from tests.plain import nuzulorn_plain as plain
from tests.trace_tools import cut

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
MARGIN = 3e-3  # between the scores of what a router takes and what it leaves, in the exact run


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    return {name: write_model(tmp_path_factory.mktemp(f"nuzulorn_{name}"), name, seed=5 + i, steady=True)
            for i, name in enumerate(sorted(CONFIGS))}


@pytest.fixture(scope="module")
def oracle(dirs):
    """(name, tokens) -> (float64 logits [T, V], what float32 costs, what bfloat16 storage costs).  The run that rounds
    uses the exact run's choices of experts, and no choice of the exact run is a close call."""
    weights = {name: plain.read_model_dir(folder, dtype=torch.float64) for name, folder in dirs.items()}

    @functools.lru_cache(maxsize=None)
    def get(name, tokens):
        config, w = weights[name]
        log = []
        exact = plain.forward(config, w, list(tokens), dtype=torch.float64, log=log)
        assert min(float(margin.min()) for _, margin in log) > MARGIN
        single = plain.forward(config, w, list(tokens), dtype=torch.float32).double()
        rounded = plain.forward(config, w, list(tokens), dtype=torch.float64, act=plain.to_bfloat16_and_back,
                                store=plain.to_bfloat16_and_back, routes=log)
        return exact, float((single - exact).abs().max()), float((rounded - exact).abs().max())

    return get


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
def test_the_residual_behind_every_layer(name, dirs):
    """float32, layer by layer: what the next layer reads (after the average over the depth), and the planes the model keeps
    (what every layer left before it)."""
    config, w = plain.read_model_dir(dirs[name], dtype=torch.float64)
    tokens = tokens_for(config, 40, salt=11)
    _, want, want_before = plain.forward(config, w, tokens, dtype=torch.float64, return_layers=True)
    _, single, _ = plain.forward(config, w, tokens, dtype=torch.float32, return_layers=True)
    run = Replay(dirs[name], name, "float32", 64, graphs=False)
    seen, planes = [], []
    for block in run.session.model.blocks:
        def wrapped(ctx, stream, view, *args, _inner=block.forward, **kw):
            out = _inner(ctx, stream, view, *args, **kw)
            seen.append(stream.residual.clone())
            planes.append(stream.layer_outputs[stream.runs_done].clone())
            return out
        block.forward = wrapped
    run.step({"a": tokens}, end=["a"])
    assert len(seen) == want.shape[0] == len(config["layers"])
    for r, (got, plane) in enumerate(zip(seen, planes)):
        allowed = 30 * float((single[r].double() - want[r]).abs().max()) + 1e-5
        assert float((got.double().cpu() - want[r]).abs().max()) <= allowed, f"behind layer {r}"
        assert float((plane.double().cpu() - want_before[r]).abs().max()) <= 3 * allowed, f"plane of layer {r}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_then_token_by_token(name, dtype, dirs, oracle):
    """The decoded tokens run through the captured single-token steps; the first tokens of a sequence too (a prompt of one
    token: the pair table's last row, then the previous token from the request's state).  70 tokens pass every window but
    the longest."""
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
    """Cuts in the middle of pages, of windows and of pooled blocks, portions of two and three tokens, of one page, longer
    than a window."""
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
    """Ten requests through four state slots and a pool of pages for 4 x 64 tokens: a request that takes a slot or a page
    that another one left starts from zero state, with no previous token, and sees none of the other's keys or blocks."""
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
def test_long_decoding_while_windows_and_blocks_pass(dtype, dirs, oracle):
    """300 decoded tokens behind a short prompt: windows of 21 and 7 positions move over decoded tokens, blocks of 5 and 9
    positions are completed by decoded tokens and come into sight later, the recurrent state is carried 300 times, and the
    pages behind the windows go back to the pool while the request runs (the rows of the blocks stay)."""
    name = "A"
    tokens = tokens_for(CONFIGS[name][0], 320, salt=8)
    run = Replay(dirs[name], name, dtype, 320)
    run.step({"a": tokens[:20]})
    for t in tokens[20:]:
        run.step({"a": [t]})
    req = run.session.cache.get("a")
    page = CONFIGS[name][1]
    groups = run.session.cache.groups
    for group, table in zip(groups, req.tables):
        held = sum(p >= 0 for p in table)
        if group.need.window is not None:
            assert held <= group.need.window // page + 2
        else:
            assert held == math.ceil(math.ceil(320 / group.every) / page)
    check(run.of("a"), name, tokens, dtype, oracle)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_greedy_generation_through_the_engine(name, dtype, dirs):
    """The engine's own entry point and scheduler: prompts cut under a small token budget, several requests at once."""
    config, page = CONFIGS[name]
    cfg = EngineConfig.defaults(str(dirs[name]), dtype=dtype, block_size=page, num_blocks=256, max_model_len=256, max_num_seqs=4,
                                max_num_batched_tokens=24)
    engine = LLMEngine(cfg)
    prompts = [tokens_for(config, n, salt=30 + n) for n in (5, 31, 18, 1, 44)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    _, w = plain.read_model_dir(dirs[name], dtype=torch.float64)
    for prompt, out in zip(prompts, outs):
        got = list(out.token_ids)
        log = []
        logits = plain.forward(config, w, prompt + got, dtype=torch.float64, log=log)
        single = plain.forward(config, w, prompt + got, dtype=torch.float32).double()
        rounded = plain.forward(config, w, prompt + got, dtype=torch.float64, act=plain.to_bfloat16_and_back,
                                store=plain.to_bfloat16_and_back, routes=log)
        # every token is within rounding of the best one, given the engine's own history
        yard = 60 * float((single - logits).abs().max()) + 2e-5 if dtype == "float32" else 6 * float((rounded - logits).abs().max())
        for i, token in enumerate(got):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[token]) <= yard
        if dtype == "float32" and all(float(r.topk(2).values.diff().abs()) > yard for r in logits[len(prompt) - 1 : -1]):
            assert got == plain.greedy(config, w, prompt, 12)


# ---- every mechanism alone ----------------------------------------------------------------------------

def part_with_weights(category, spec, prefix, dtype, tensors):
    part = build_part(category, spec, prefix, dtype, DEV)
    decls = {d.name: d for d in part.tensor_decls()}
    assert set(decls) == set(tensors), (sorted(decls), sorted(tensors))
    part.load_weights(make_fetch(lambda n: tensors[n], decls, dtype, DEV))
    return part


def run_mixer(part, x, portions, page_size=4, num_pages=128):
    """The mixer's output for every row of ``x`` [T, W], fed in portions through a cache of its own."""
    harness = PartHarness({0: part.cache_need()}, part.dtype, num_pages=num_pages, page_size=page_size, slots=2)
    out, at = [], 0
    for n in portions:
        prepared = harness.prepare({"a": n})
        got = part.mix(prepared.ctx, x[at : at + n].to(DEV, part.dtype).contiguous(), prepared.ctx.views[0])
        harness.commit(prepared)
        out.append(got.float().cpu())
        at += n
    assert at == x.shape[0]
    return torch.cat(out)


def draw(gen, shape, scale=1.0, shift=0.0):
    return (shift + scale * torch.randn(shape, generator=gen)).to(torch.bfloat16).float()


def assert_close(got, want, what, rel=3e-5):
    """float32 arithmetic against float64: a few units of float32 rounding of the largest value, per term summed."""
    worst, allowed = float((got.double() - want).abs().max()), 2e-4 + rel * float(want.abs().max())
    assert worst <= allowed, f"{what}: off by {worst:.3g}, allowed {allowed:.3g}"


def named(tensors, prefix="m"):
    return {f"{prefix}.{k}": v for k, v in tensors.items()}


def doubled(tensors):
    return {k: v.double() for k, v in tensors.items()}


def window_tensors(gen, w, heads, kv_heads, dim, vdim):
    return {"q": draw(gen, (heads * dim, w), 0.5), "q.b": draw(gen, (heads * dim,), 0.3), "k": draw(gen, (kv_heads * dim, w), 0.5),
            "k.b": draw(gen, (kv_heads * dim,), 0.3), "v": draw(gen, (kv_heads * vdim, w), 0.3), "v.b": draw(gen, (kv_heads * vdim,), 0.2),
            "g": draw(gen, (heads, w), 0.3), "o": draw(gen, (w, heads * vdim), 0.2), "o.b": draw(gen, (w,), 0.2)}


def window_spec(w, m):
    return PartSpec("window_attention", dict(hidden_size=w, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"],
                                             scale=m["scale"], weights="softmax", bias=True, out_bias=True, window=m["mask"]["size"],
                                             pool=m["mask"]["pool"], sink="zero", gate=True, rotary=dict(m["rot"])))


def window_config(heads, kv_heads, dim, vdim, size, pool, scale, rot, base):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, mask={"size": size, "pool": pool}, rot={"dims": rot, "base": base})


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, size, pool, rot, base, page", [
    (4, 2, 24, 12, 21, 5, 8, 1000.0, 4), (3, 1, 16, 40, 7, 9, 16, 50000.0, 8), (6, 6, 8, 8, 1, 1, 2, 10000.0, 4), (2, 2, 12, 20, 400, 6, 12, 100.0, 16),
    (8, 2, 32, 64, 100, 12, 32, 10000.0, 16), (5, 5, 16, 24, 64, 64, 4, 300.0, 16), (12, 3, 48, 80, 60, 7, 16, 500000.0, 16),
    (33, 11, 8, 4, 10, 3, 6, 20.0, 4)])
def test_window_with_pooled_blocks_alone(heads, kv_heads, dim, vdim, size, pool, rot, base, page):
    """300 positions whole, token by token and in portions that cut pages, windows and blocks.  First the plain
    implementation shows that the window's edge and the gate count: a window one position shorter or longer (unless every
    token is its own block: what leaves the window then comes back at once as the same key and value) or gates wide open
    move the result by far more than the test allows.  (The blocks' edges are the business of the test of keys that stand
    out: the mean of a block of random keys rarely weighs much.)"""
    gen = torch.Generator().manual_seed(heads * 100 + size)
    w, scale = 48, 0.4
    t = window_tensors(gen, w, heads, kv_heads, dim, vdim)
    wd = doubled(t)
    x = draw(gen, (300, w))
    m = window_config(heads, kv_heads, dim, vdim, size, pool, scale, rot, base)
    want = plain.window_pool_attention(x.double(), wd, m)
    for other in (size - 1, size + 1):
        if 1 <= other < 300 and pool > 1:
            assert float((plain.window_pool_attention(x.double(), wd, dict(m, mask={"size": other, "pool": pool})) - want).abs().max()) > 0.02
    assert float((plain.window_pool_attention(x.double(), dict(wd, g=wd["g"] * 0 + 5.0), m) - want).abs().max()) > 0.02
    part = part_with_weights("mixer", window_spec(w, m), "m", torch.float32, named(t))
    for portions in ([131, 169], [1] * 300, [2, 3, 1, 1, 9, 2, 5, 41, 100, 1, 1, 1, 131, 2], [page - 1, 2, page, 1, 300 - 2 * page - 2]):
        assert sum(portions) == 300
        got = run_mixer(part, x, portions, page_size=page, num_pages=300 // page + 8)
        assert_close(got, want, portions)


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, size, pool, rot, page", [
    (4, 4, 256, 256, 100, 12, 128, 16), (8, 8, 64, 64, 130, 10, 64, 64), (16, 1, 64, 64, 40, 33, 64, 16), (8, 2, 128, 128, 150, 8, 64, 16),
    (6, 3, 96, 48, 45, 4, 32, 8), (4, 1, 240, 200, 70, 5, 16, 16), (4, 4, 32, 256, 33, 1, 32, 16)])
def test_window_with_pooled_blocks_in_bfloat16_on_the_tensor_cores(heads, kv_heads, dim, vdim, size, pool, rot, page):
    """Sizes that take each arrangement of the tensor-core kernel; rows that see several tiles of pooled blocks (a block of
    one position: hundreds of them), whole and in portions, against the plain implementation in float64; allowed is 3 times
    what rounding q, k, v, the blocks' means and the output to bfloat16 costs the plain implementation."""
    gen = torch.Generator().manual_seed(heads * 100 + size)
    w, scale = 64, dim ** -0.5
    t = window_tensors(gen, w, heads, kv_heads, dim, vdim)
    wd = doubled(t)
    x = draw(gen, (260, w))
    m = window_config(heads, kv_heads, dim, vdim, size, pool, scale, rot, 10000.0)
    want = plain.window_pool_attention(x.double(), wd, m)
    rounded = plain.window_pool_attention(plain.to_bfloat16_and_back(x.double()), wd, m, store=plain.to_bfloat16_and_back)
    rounded = plain.to_bfloat16_and_back(rounded)
    allowed = 3 * float((rounded - want).abs().max()) + 0.01 * float(want.abs().max())
    assert allowed < 0.1 * float(want.abs().max())
    part = part_with_weights("mixer", window_spec(w, m), "m", torch.bfloat16, named(t))
    for portions in ([260], [200] + [1] * 60, [3, 64, 1, 61, 2, 109] + [1] * 20):
        got = run_mixer(part, x, portions, page_size=page, num_pages=600 // page + 8)
        worst = float((got.double() - want).abs().max())
        assert worst <= allowed, f"{portions[:6]}: off by {worst:.3g}, allowed {allowed:.3g}"


def _towering(t, heads, kv_heads, dim, w, rot):
    """Every unrotated query channel reads coordinate 3, every unrotated key channel coordinate 5, no bias; no key reads
    coordinate 3 and no query coordinate 5 (a towering query is no towering key of its own position)."""
    for name, col, other, count in (("q", 3, 5, heads), ("k", 5, 3, kv_heads)):
        t[name].view(count, dim, w)[:, rot:, col] = 0.5
        t[name].view(count, dim, w)[:, :rot, col] = 0.0
        t[name].view(count, dim, w)[:, :, other] = 0.0
        t[name + ".b"].zero_()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_keys_that_stand_out_at_the_edges_of_the_window_and_of_the_blocks(dtype):
    """A query and a few keys are made so that one score towers over all others, the one in the denominator too.  The key at
    the window's far edge takes the whole softmax; one position further back it is not seen at all while its block is not
    whole behind the window, and comes back as the block's mean (a fifth of its value, beside the block's other members)
    once the block is.  In a prompt and in decoding, also where a portion ends at an edge."""
    heads, kv_heads, dim, vdim, size, pool, w, rot = 2, 1, 16, 8, 37, 5, 32, 4
    gen = torch.Generator().manual_seed(9)
    t = window_tensors(gen, w, heads, kv_heads, dim, vdim)
    x = draw(gen, (120, w), 0.05)
    _towering(t, heads, kv_heads, dim, w, rot)
    probe = 100
    inside, outside = probe - size + 1, probe - size  # 64 is the window's last position; 63 is outside, and its block 60..64 not whole behind
    assert outside // pool == inside // pool
    x[probe, 3] += 40.0
    x[inside, 5] += 40.0
    x[outside, 5] += 80.0  # would win if it were visible
    wd = doubled(t)
    m = window_config(heads, kv_heads, dim, vdim, size, pool, 1.0, rot, 1000.0)
    want = plain.window_pool_attention(x.double(), wd, m)
    gate = torch.sigmoid(x[probe].double() @ wd["g"].T)
    v_inside = ((x[inside].double() @ wd["v"].T + wd["v.b"]).repeat(heads).view(heads, vdim) * gate[:, None]).reshape(-1) @ wd["o"].T + wd["o.b"]
    assert float((want[probe] - v_inside).abs().max()) < 1e-6  # the edge key alone
    # a later query whose window has left both behind sees them through their block's mean only: position 63 dominates the mean's key
    late = 103
    x[late, 3] += 40.0
    want = plain.window_pool_attention(x.double(), wd, m)
    block = outside // pool
    assert block * pool + pool - 1 <= late - size and (block + 1) * pool + pool - 1 > late - size  # the last block in sight
    rows = x[block * pool : block * pool + pool].double()
    gate = torch.sigmoid(x[late].double() @ wd["g"].T)
    v_mean = (((rows @ wd["v"].T + wd["v.b"]).mean(0)).repeat(heads).view(heads, vdim) * gate[:, None]).reshape(-1) @ wd["o"].T + wd["o.b"]
    assert float((want[late] - v_mean).abs().max()) < 1e-6
    part = part_with_weights("mixer", window_spec(w, m), "m", dtype, named(t))
    for portions in ([120], [probe, 1, 19], [inside, 20, 16, 1, 19], [outside, 1, 1, 35, 1, 19], [70] + [1] * 50, [late, 1, 16], [65, 45, 10]):
        got = run_mixer(part, x, portions, page_size=8)
        if dtype == torch.float32:
            assert_close(got, want, portions)
        else:
            assert float((got.double() - want).abs().max()) < 0.03 * float(want.abs().max()), portions


def capped_tensors(gen, w, heads, kv_heads, dim, vdim):
    return {"q": draw(gen, (heads * dim, w), 0.5), "q.b": draw(gen, (heads * dim,), 0.3), "k": draw(gen, (kv_heads * dim, w), 0.5),
            "k.b": draw(gen, (kv_heads * dim,), 0.3), "v": draw(gen, (kv_heads * vdim, w), 0.3), "v.b": draw(gen, (kv_heads * vdim,), 0.2),
            "sink": draw(gen, (heads,), 1.0, 1.0), "o": draw(gen, (w, heads * vdim), 0.2)}


def capped_spec(w, m):
    return PartSpec("window_attention", dict(hidden_size=w, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"],
                                             scale=m["scale"], weights="softmax", bias=True, out_bias=False, window=None, sink=True,
                                             softcap=m["softcap"], distance_bias={"halvings": 8.0},
                                             query_temperature=dict(m["q_temp"])))


@pytest.mark.parametrize("heads, kv_heads, dim, vdim, cap, coef, every, page, dtype", [
    (4, 2, 16, 24, 4.0, 0.4, 3, 4, torch.float32), (3, 3, 8, 8, 50.0, 1.5, 1000, 8, torch.float32), (6, 1, 8, 24, 8.0, 0.5, 16, 16, torch.float32),
    (33, 11, 8, 4, 2.0, 0.2, 7, 4, torch.float32), (8, 2, 32, 64, 20.0, 0.5, 32, 16, torch.float32),
    (8, 2, 32, 64, 20.0, 0.5, 32, 16, torch.bfloat16), (4, 2, 64, 64, 25.0, 0.3, 100, 16, torch.bfloat16), (16, 1, 128, 128, 5.0, 1.0, 10, 64, torch.bfloat16)])
def test_capped_scores_with_a_distance_bias_a_query_temperature_and_a_sink_alone(heads, kv_heads, dim, vdim, cap, coef, every, page, dtype):
    """300 positions whole, token by token and in portions.  First the plain implementation shows that each piece counts:
    no cap, no temperature, slopes of another base, a sink far below the scores."""
    gen = torch.Generator().manual_seed(heads * 100 + every)
    w, scale = 48, 0.6
    t = capped_tensors(gen, w, heads, kv_heads, dim, vdim)
    wd = doubled(t)
    x = draw(gen, (300, w))
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, softcap=cap, q_temp={"coef": coef, "every": every})
    want = plain.capped_sink_attention(x.double(), wd, m)
    if cap < 20:
        assert float((plain.capped_sink_attention(x.double(), wd, dict(m, softcap=1e6)) - want).abs().max()) > 0.01
    if every < 300:
        assert float((plain.capped_sink_attention(x.double(), wd, dict(m, q_temp={"coef": 0.0, "every": every})) - want).abs().max()) > 0.01
    assert float((plain.capped_sink_attention(x.double(), dict(wd, sink=wd["sink"] - 60.0), m) - want).abs().max()) > 0.01
    part = part_with_weights("mixer", capped_spec(w, m), "m", dtype, named(t))
    if dtype == torch.bfloat16:
        rounded = plain.to_bfloat16_and_back(plain.capped_sink_attention(plain.to_bfloat16_and_back(x.double()), wd, m, store=plain.to_bfloat16_and_back))
        allowed = 3 * float((rounded - want).abs().max()) + 0.01 * float(want.abs().max())
    for portions in ([131, 169], [1] * 300, [2, 3, 1, 1, 9, 2, 5, 41, 100, 1, 1, 1, 131, 2]):
        got = run_mixer(part, x, portions, page_size=page, num_pages=400 // page + 8)
        if dtype == torch.float32:
            assert_close(got, want, portions)
        else:
            assert float((got.double() - want).abs().max()) <= allowed, portions


def test_a_key_far_back_among_hundreds_and_the_sink_against_a_lone_key():
    """The key at position 3 stands out for a query 650 positions on, among hundreds, although the distance bias pulls it down
    (head 0's slope times 650) and the cap bends it; whole, decoded, and over portions.  And the first token of a sequence
    shares the softmax with the sink alone: with a sink as large as its (capped) score it gets half."""
    heads, kv_heads, dim, vdim, w, cap = 4, 2, 32, 16, 32, 300.0
    gen = torch.Generator().manual_seed(10)
    t = capped_tensors(gen, w, heads, kv_heads, dim, vdim)
    x = draw(gen, (700, w), 0.005)
    x[653, 3] += 60.0
    x[3, 5] += 60.0
    _towering(t, heads, kv_heads, dim, w, 0)
    t["sink"] = torch.zeros(heads)
    wd = doubled(t)
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=1.0, softcap=cap, q_temp={"coef": 0.4, "every": 100})
    want = plain.capped_sink_attention(x.double(), wd, m)
    v_far = (x[3].double() @ wd["v"].T + wd["v.b"]).reshape(kv_heads, vdim).repeat_interleave(heads // kv_heads, 0).reshape(-1) @ wd["o"].T
    assert float((want[653] - v_far).abs().max()) < 1e-6
    q0 = (x[0].double() @ wd["q"].T).reshape(heads, dim)
    k0 = (x[0].double() @ wd["k"].T).reshape(kv_heads, dim).repeat_interleave(heads // kv_heads, 0)
    t["sink"] = (cap * torch.tanh((q0 * k0).sum(-1) / cap)).float()  # position 0: temperature 1, distance 0
    wd = doubled(t)
    want = plain.capped_sink_attention(x.double(), wd, m)
    v_first = (x[0].double() @ wd["v"].T + wd["v.b"]).reshape(kv_heads, vdim).repeat_interleave(heads // kv_heads, 0).reshape(-1) @ wd["o"].T
    assert float((want[0] - 0.5 * v_first).abs().max()) < 1e-4 * float(v_first.abs().max()) + 1e-6
    part = part_with_weights("mixer", capped_spec(w, m), "m", torch.float32, named(t))
    for portions in ([700], [640] + [1] * 60, [1, 4, 300, 345, 3, 1, 46]):
        got = run_mixer(part, x, portions, page_size=16)
        assert_close(got, want, portions)


def recurrent_tensors(gen, w, heads, dim, vdim):
    return {"q": draw(gen, (heads * dim, w), 0.3), "f": draw(gen, (heads * dim, w), 0.3), "f.b": draw(gen, (heads * dim,), 1.0, 2.0),
            "lower": torch.rand((heads * dim,), generator=gen).mul(0.9).to(torch.bfloat16).float(), "v": draw(gen, (heads * vdim, w), 0.3),
            "norm": draw(gen, (vdim,), 0.2, 1.0), "o": draw(gen, (w, heads * vdim), 0.2)}


@pytest.mark.parametrize("heads, dim, vdim, dtype", [(3, 12, 20, torch.float32), (1, 16, 8, torch.float32), (5, 8, 24, torch.float32),
                                                     (4, 64, 48, torch.float32), (4, 32, 48, torch.bfloat16), (16, 128, 128, torch.bfloat16)])
def test_forget_gates_with_a_lower_bound_alone(heads, dim, vdim, dtype):
    """200 positions whole, token by token and in portions: the state is carried from portion to portion.  First the plain
    implementation shows that a state that starts from zero in the middle, or gates without their lower bound, would be seen."""
    gen = torch.Generator().manual_seed(heads * 100 + dim)
    w, eps = 48, 1e-5
    t = recurrent_tensors(gen, w, heads, dim, vdim)
    wd = doubled(t)
    x = draw(gen, (200, w))
    m = dict(heads=heads, dim=dim, vdim=vdim)
    want, _ = plain.bounded_forget_recurrence(x.double(), wd, m, eps)
    fresh, _ = plain.bounded_forget_recurrence(x[100:].double(), wd, m, eps)
    assert float((fresh - want[100:]).abs().max()) > 0.05
    unbounded, _ = plain.bounded_forget_recurrence(x.double(), dict(wd, lower=wd["lower"] * 0), m, eps)
    assert float((unbounded - want).abs().max()) > 0.05
    spec = PartSpec("hgrn2", dict(hidden_size=w, heads=heads, dim=dim, vdim=vdim, eps=eps))
    part = part_with_weights("mixer", spec, "m", dtype, named(t))
    if dtype == torch.bfloat16:
        rounded = plain.to_bfloat16_and_back(plain.bounded_forget_recurrence(plain.to_bfloat16_and_back(x.double()), wd, m, eps)[0])
        allowed = 3 * float((rounded - want).abs().max()) + 0.01 * float(want.abs().max())
    for portions in ([200], [1] * 200, [2, 3, 1, 1, 9, 2, 5, 41, 100, 1, 1, 1, 31, 2], [17, 150, 33]):
        got = run_mixer(part, x, portions)
        if dtype == torch.float32:
            assert_close(got, want, portions)
        else:
            assert float((got.double() - want).abs().max()) <= allowed, portions


@pytest.mark.parametrize("ff, experts, top, scale, groups", [(40, 6, 3, 1.5, (3, 2)), (24, 4, 1, 2.0, (2, 1)), (16, 4, 2, 0.8, (4, 2)),
                                                            (32, 3, 3, 1.0, None), (20, 5, 2, 1.2, (1, 1)), (12, 6, 6, 1.0, (3, 3)),
                                                            (96, 16, 4, 2.5, (2, 1)), (64, 8, 2, 2.5, (4, 2))])
def test_experts_ranked_by_corrected_sigmoid_scores_in_groups_alone(ff, experts, top, scale, groups):
    """Corrections as large as the scores (and some far below zero: the choice scores of whole groups are negative, so that a
    group left out must count as minus infinity, not as 0); the weights are the scores without them, times the scale, not
    renormalised.  Rows whose margins are thin are left out of the comparison."""
    gen = torch.Generator().manual_seed(experts * 10 + top)
    w = 48
    t = {"router": draw(gen, (experts, w), 0.4), "correction": draw(gen, (experts,), 0.5, -0.7)}
    for e in range(experts):
        t.update({f"e{e}.gate": draw(gen, (ff, w), 0.2), f"e{e}.up": draw(gen, (ff, w), 0.2), f"e{e}.down": draw(gen, (w, ff), 0.2)})
    x = draw(gen, (150, w))
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if groups is not None:
        f["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    log = []
    want = plain.experts(x.double(), doubled(t), f, log=log)
    steady = log[0][1] > 1e-4
    assert int(steady.sum()) > 100
    params = dict(hidden_size=w, expert_size=ff, experts=experts, top=top, scoring="sigmoid", correction=True, router_bias=False,
                  weight_scale=scale)
    if groups is not None:
        params.update(groups=groups[0], keep=groups[1], group_rank=min(2, experts // groups[0]))
    part = part_with_weights("ffn", PartSpec("moe", params), "m", torch.float32, named(t))
    harness = PartHarness({}, torch.float32)
    prepared = harness.prepare({"a": 150})
    (got, factor), = part.output_terms(prepared.ctx, x.to(DEV).contiguous())
    got = (got * factor).cpu()
    assert_close(got[steady], want[steady], "experts")


def test_the_pair_table_and_the_previous_token_of_a_request():
    """Rows of the pair table by the hash of (previous token, token); the previous token of a portion's first token comes from
    the request's state, a request's first token reads the last row, and a slot that another request used is not read."""
    gen = torch.Generator().manual_seed(3)
    buckets, mul_prev, mul_cur, w, vocab = 53, 1000003, 7919, 24, 50000
    table = draw(gen, (buckets + 1, w))
    spec = PartSpec("hashed_pair", dict(size=w, buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur, name="pairs"))
    part = part_with_weights("embedding", spec, "", torch.float32, {"pairs": table})
    harness = PartHarness({0: part.cache_need()}, torch.float32, slots=2)
    tokens = {"a": [int(v) for v in torch.randint(0, vocab, (40,), generator=gen)], "b": [int(v) for v in torch.randint(0, vocab, (25,), generator=gen)]}
    want = {rid: table[plain.pair_rows(toks, buckets, mul_prev, mul_cur)] for rid, toks in tokens.items()}
    got = {rid: [] for rid in tokens}
    at = {rid: 0 for rid in tokens}
    for step in ({"a": 3}, {"a": 1, "b": 2}, {"b": 1}, {"a": 20, "b": 1}, {"a": 1, "b": 21}, {"a": 15}):
        prepared = harness.prepare(step)
        ids = torch.tensor([t for rid, n in step.items() for t in tokens[rid][at[rid] : at[rid] + n]], dtype=torch.int32, device=DEV)
        x = torch.zeros((ids.shape[0], w), dtype=torch.float32, device=DEV)
        part.add_to_embedding(prepared.ctx, x, ids, prepared.ctx.views[0])
        harness.commit(prepared)
        row = 0
        for rid, n in step.items():
            got[rid].append(x[row : row + n].cpu())
            row += n
            at[rid] += n
    for rid in tokens:
        assert torch.equal(torch.cat(got[rid]), want[rid]), rid
    harness.cache.close("a")  # its slot goes to the next request, which starts with the table's last row
    prepared = harness.prepare({"c": 2})
    ids = torch.tensor(tokens["b"][:2], dtype=torch.int32, device=DEV)
    x = torch.zeros((2, w), dtype=torch.float32, device=DEV)
    part.add_to_embedding(prepared.ctx, x, ids, prepared.ctx.views[0])
    assert torch.equal(x.cpu(), want["b"][:2])


def test_the_scaled_sum_with_its_norm_and_the_average_over_the_depth():
    gen = torch.Generator().manual_seed(4)
    n, w, planes_n = 37, 72, 5
    x, a, b = (torch.randn((n, w), generator=gen) for _ in range(3))
    weight = 1 + 0.1 * torch.randn(w, generator=gen)
    eps = 1e-5
    into = torch.zeros((n, w), device=DEV)
    normed = ops.axpy_rmsnorm(x.to(DEV), [(a.to(DEV), 0.3), (b.to(DEV), -1.2)], weight.to(DEV), eps, torch.float32, into)
    y = x.double() + 0.3 * a.double() - 1.2 * b.double()
    assert_close(into.cpu(), y, "sum")
    assert_close(normed.cpu(), plain.unit_rms(y, eps) * weight.double(), "norm of the sum")
    history = torch.randn((planes_n, n, w), generator=gen)
    coef = torch.randn(4, generator=gen)
    h = history.to(DEV)
    out = torch.zeros((n, w), device=DEV)
    normed = ops.depth_average(h[3], [(a.to(DEV), 0.5)], h, 3, coef.to(DEV), out, weight.to(DEV), eps, torch.float32)
    plane = history[3].double() + 0.5 * a.double()
    mean = sum(c.double() * p for c, p in zip(coef[:3], history[:3].double())) + coef[3].double() * plane
    assert_close(h[3].cpu(), plane, "plane")
    assert_close(out.cpu(), mean, "average")
    assert_close(normed.cpu(), plain.unit_rms(mean, eps) * weight.double(), "norm of the average")
    assert torch.equal(h[4].cpu(), history[4]) and torch.equal(h[:3].cpu(), history[:3])


def test_a_step_at_layer_sizes_of_a_real_model():
    """Two layers of the 2,048-wide shape in bfloat16 through the engine's step function: a prompt of 300 tokens whole against
    the same prompt in portions and decoded, which must agree within rounding."""
    from clockwork_b200.config.registry import get_architecture
    from clockwork_b200.weights import write_random_model
    import tempfile

    raw = dict(get_architecture("Nuzulorn").named_shapes["nuzulorn-2k"])
    raw["layers"] = [raw["layers"][1], raw["layers"][0], raw["layers"][3]]
    raw["vocab"] = 4096
    with tempfile.TemporaryDirectory() as folder:
        write_random_model(folder, raw, seed=3)
        tokens = tokens_for(raw, 300, salt=9)
        outs = []
        for sizes in ([300], [200, 90] + [1] * 10, [64, 2, 130, 3, 101]):
            session = TraceSession(folder, "bfloat16", 512, page_size=16)
            got, n = [], 0
            for portion in cut(tokens, sizes):
                out, _ = session.run_step({"step": n, "entries": [{"id": "a", "tokens": portion, "want": [len(portion) - 1]}], "end": []})
                got.append(torch.from_numpy(out.copy()))
                n += 1
            outs.append(torch.cat(got)[-1])
        scale = float(outs[0].std())
        for other in outs[1:]:
            assert float((other - outs[0]).abs().max()) < 0.08 * scale
