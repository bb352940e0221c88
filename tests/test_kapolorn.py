"""Kapolorn without a GPU: its configuration, the description the framework makes of it, the tensors it declares,
the order its layers run in, what every run asks of the cache manager, and properties of the plain implementation that
the GPU tests lean on (it does not look ahead; a block one position longer, a sink left out, a state that starts late,
a group that is not masked are other functions by far more than the tests allow)."""

import copy

import pytest
import torch

from clockwork_b200.cache import CacheManager
from clockwork_b200.config.registry import architecture_name, shape_config, spec_from_raw
from clockwork_b200.parts import PagedKVNeed, SlotStateNeed, build_model
from clockwork_b200.parts.model import tensor_decls_for_spec
from clockwork_b200.weights.loader import WeightMismatchError, check_declarations
from tests.kapolorn_configs import CONFIGS, draw_weights, tensor_shapes, tokens_for
from tests.plain import kapolorn_plain as plain


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    config, _, rank = CONFIGS[name]
    spec = spec_from_raw(config)
    assert architecture_name(config) == "Kapolorn" and spec.architecture == "Kapolorn"
    assert spec.tie_word_embeddings and spec.embedding_scale == config["embedding"]["scale"]
    assert spec.logit_softcap == config["logit_softcap"]
    decls = tensor_decls_for_spec(spec)
    shapes = tensor_shapes(config, rank)
    check_declarations(decls, shapes, "test")  # the low-rank products' inner sizes are the checkpoint's; the head is the embedding
    assert {d.name for d in decls if not d.optional} == set(shapes)
    for layer, listed in zip(spec.layers, config["layers"]):
        assert layer.block == "sandwich_residual"
        if listed["type"] == "parallel":
            assert layer.mixer.kind == "side_by_side" and not layer.mixer["normed"]
            left, right = layer.mixer["left"], layer.mixer["right"]
            assert (left.kind, right.kind) == ("window_attention", "matrix_memory")
            assert left["mask"] == "block" and left["sink"] and left["window"] == listed["mixer"]["left"]["mask"]["size"]
            assert left["rotary"] == {"dims": listed["mixer"]["left"]["rot"]["dims"], "base": listed["mixer"]["left"]["rot"]["base"]}
            assert left["scale"] == listed["mixer"]["left"]["scale"] and right["gate_cap"] == listed["mixer"]["right"]["gate_cap"]
        else:
            assert layer.mixer.kind == "channel_delta" and layer.mixer["conv"] == listed["mixer"]["conv"]
        mlp = listed["mlp"]
        assert layer.ffn.kind == ("none" if mlp is None else "moe")
        if mlp is not None:
            groups = mlp["router"].get("groups")
            assert layer.ffn["top"] == mlp["router"]["top"] and layer.ffn["limit"] == mlp["expert"]["limit"]
            assert layer.ffn.get("groups", 1) == (groups["count"] if groups else 1)
            assert (layer.ffn.get("shared") is None) == (mlp.get("shared") is None)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_order_of_runs_and_a_cache_of_its_own_for_every_pass(name):
    config = CONFIGS[name][0]
    spec = spec_from_raw(config)
    order = plain.run_order(config)
    assert [step.layer for step in spec.schedule] == [i for i, _ in order]
    cache_layers = [step.layer if step.cache_layer is None else step.cache_layer for step in spec.schedule]
    assert len(set(cache_layers)) == len(order)  # no two runs share a cache or a state
    first_pass = [c for c, (_, p) in zip(cache_layers, order) if p == 0]
    assert first_pass == [i for i, p in order if p == 0]
    model = build_model(spec, torch.float32, "cpu")
    needs = model.cache_needs()
    assert sorted(needs) == sorted(cache_layers)
    for c, (i, _) in zip(cache_layers, order):
        assert needs[c] == needs[i]  # a further pass keeps what the first pass keeps


def test_the_named_shapes_describe_themselves():
    for name in ("kapolorn-tiny", "kapolorn-2k"):
        spec = spec_from_raw(shape_config(name))
        assert len(tensor_decls_for_spec(spec)) > 10
    assert len(spec_from_raw(shape_config("kapolorn-2k", 4)).layers) == 4
    kinds = [layer.mixer.kind for layer in spec_from_raw(shape_config("kapolorn-2k", 4)).layers]
    assert kinds.count("channel_delta") == 1 and kinds.count("side_by_side") == 3


def test_a_wrong_shape_and_a_missing_tensor_are_reported():
    config, _, rank = CONFIGS["A"]
    shapes = tensor_shapes(config, rank)
    shapes["l0.mix.left.sink"] = (5, 4)
    del shapes["l1.mix.A_log"]
    with pytest.raises(WeightMismatchError) as err:
        check_declarations(tensor_decls_for_spec(spec_from_raw(config)), shapes, "test")
    assert err.value.missing == ["l1.mix.A_log"] and [w[0] for w in err.value.wrong_shape] == ["l0.mix.left.sink"]


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="parallel_9"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown feed-forward"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("mask"), "lacks 'size'"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("rot"), "lacks 'dims'"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "must be even"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("gate_cap"), "lacks 'gate_cap'"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "lacks 'left_scale'"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "fewer than top"),
    (lambda c: c.pop("embedding"), "lacks 'scale'"),
    (lambda c: c["loop"].update(stop=9), "does not fit"),
    (lambda c: c.update(logit_softcap=-1.0), "must be positive"),
    (lambda c: c.update(layers=[]), "non-empty list"),
])
def test_a_faulty_configuration_is_refused(change, message):
    config = copy.deepcopy(CONFIGS["A"][0])
    change(config)
    with pytest.raises(ValueError, match=message):
        build_model(spec_from_raw(config), torch.float32, "cpu")


def test_a_model_without_loop_cap_groups_or_shared_expert_is_described():
    config = copy.deepcopy(CONFIGS["B"][0])
    config["logit_softcap"] = None
    spec = spec_from_raw(config)
    assert spec.logit_softcap is None and [s.layer for s in spec.schedule] == [0, 1, 2]
    assert spec.layers[0].ffn.get("shared") is None and spec.layers[0].ffn.get("groups", 1) == 1


def test_what_a_layer_keeps_and_pages_of_passed_blocks_go_back():
    """Rows of [key | value] per key/value head in a page group that keeps a request's current block only; the matrix
    memory's S with the key sum as one more column and a maximum per head; the delta rule's S and the convolution's
    last inputs."""
    config = CONFIGS["A"][0]
    needs = build_model(spec_from_raw(config), torch.float32, "cpu").cache_needs()
    left, right = config["layers"][0]["mixer"]["left"], config["layers"][0]["mixer"]["right"]
    assert needs[0] == (PagedKVNeed(left["kv_heads"], left["dim"] + left["vdim"], None, planes=1, block=left["mask"]["size"]),
                        SlotStateNeed((right["heads"] * right["dim"] * (right["vdim"] + 1) + right["heads"],)))
    d = config["layers"][1]["mixer"]
    channels = 2 * d["kv_heads"] * d["dim"] + d["heads"] * d["vdim"]
    assert needs[1] == SlotStateNeed((d["heads"] * d["dim"] * d["vdim"] + (d["conv"] - 1) * channels,))
    assert needs[3] == needs[1] and needs[4] == needs[1]  # the second and third pass of the looped layer
    cache = CacheManager(needs, num_pages=16, page_size=4, num_state_slots=2)
    blocks = sorted(g.need.block for g in cache.groups)
    assert blocks == [7, 21]
    req = cache.open("a")
    cache.reserve(req, 45)
    req.num_computed = 45
    assert cache.release_behind_window(req, 45) > 0
    held = {cache.groups[g].need.block: sum(p >= 0 for p in req.tables[g]) for g in range(len(cache.groups))}
    # position 45 lies in the block from 42 on, of either size: the pages that hold positions 42 .. 44
    assert held[7] == 2 and held[21] == 2
    cache.close("a")
    cache.check_invariants()


def test_the_plain_implementation_does_not_look_ahead_and_every_mechanism_counts():
    config, _, rank = CONFIGS["A"]
    w = draw_weights(config, rank, seed=3)
    tokens = tokens_for(config, 50, salt=1)
    whole = plain.forward(config, w, tokens, dtype=torch.float64)
    other = tokens[:23] + [(t + 1) % config["vocab"] for t in tokens[23:]]
    assert torch.allclose(plain.forward(config, w, other, dtype=torch.float64)[:23], whole[:23], atol=1e-9)

    def moved(change, weights=w):
        changed = copy.deepcopy(config)
        change(changed)
        return float((plain.forward(changed, weights, tokens, dtype=torch.float64) - whole).abs().max())

    # a block of one more or one less position, another rotation, score scale, cap, side scale, loop count: other functions
    assert moved(lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=22)) > 1e-2
    assert moved(lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=20)) > 1e-2
    assert moved(lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(base=5000.0)) > 1e-3
    assert moved(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=10)) > 1e-3
    assert moved(lambda c: c["layers"][0]["mixer"]["left"].update(scale=0.25)) > 1e-3
    assert moved(lambda c: c["layers"][0]["mixer"]["right"].update(gate_cap=1.0)) > 1e-3
    assert moved(lambda c: c["layers"][0]["mixer"].update(left_scale=1.0)) > 1e-3
    assert moved(lambda c: c["loop"].update(times=2)) > 1e-2
    assert moved(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=3)) > 1e-4
    assert moved(lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.5)) > 1e-3
    assert moved(lambda c: c.update(logit_softcap=6.0)) > 1e-2
    assert moved(lambda c: c["embedding"].update(scale=1.0)) > 1e-2
    no_sink = dict(w)
    for name in w:
        if name.endswith(".sink"):
            no_sink[name] = torch.full_like(w[name], -60.0)
    assert moved(lambda c: None, no_sink) > 1e-2


def test_states_that_start_late_are_seen():
    config, _, rank = CONFIGS["A"]
    w = {k: v.double() for k, v in draw_weights(config, rank, seed=3).items()}
    x = torch.randn(40, config["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    memory = config["layers"][0]["mixer"]["right"]
    full = plain.matrix_memory_mixer(x, w, "l0.mix.right", memory, 1e-5)
    assert float((full[25:] - plain.matrix_memory_mixer(x[25:], w, "l0.mix.right", memory, 1e-5)).abs().max()) > 1e-2
    delta = config["layers"][1]["mixer"]
    full = plain.channel_delta_mixer(x, w, "l1.mix", delta, 1e-5)
    assert float((full[25:] - plain.channel_delta_mixer(x[25:], w, "l1.mix", delta, 1e-5)).abs().max()) > 1e-2


def test_the_choice_of_experts_stays_in_the_best_groups():
    gen = torch.Generator().manual_seed(2)
    r = {"experts": 12, "top": 3, "groups": {"count": 4, "keep": 2}}
    w = {"f.router": torch.randn(12, 16, generator=gen, dtype=torch.float64)}
    h = torch.randn(200, 16, generator=gen, dtype=torch.float64)
    chosen, weights, margin = plain.route(h, w, "f", r)
    scores = torch.softmax(h @ w["f.router"].T, dim=-1)
    best = scores.reshape(200, 4, 3).max(-1).values
    for t in range(200):
        kept = set(best[t].topk(2).indices.tolist())
        assert {int(e) // 3 for e in chosen[t]} <= kept
        allowed = [e for e in range(12) if e // 3 in kept]
        assert sorted(chosen[t].tolist()) == sorted(sorted(allowed, key=lambda e: -float(scores[t, e]))[:3])
        assert torch.equal(weights[t], scores[t][chosen[t]])
    assert float(weights.sum(-1).max()) < 1.0 and bool((margin > 0).all())
    # without groups the plain top of all experts; it differs from the grouped choice for some tokens
    free, _, _ = plain.route(h, w, "f", {"experts": 12, "top": 3})
    assert torch.equal(free, scores.topk(3).indices) and not torch.equal(free.sort(-1).values, chosen.sort(-1).values)
