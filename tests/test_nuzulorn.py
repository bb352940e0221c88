"""Nuzulorn without a GPU: its configuration, the description the framework makes of it, the tensors it declares, what
every layer asks of the cache manager (a page group of one row per block of positions among them), and properties of the
plain implementation that the GPU tests lean on (it does not look ahead; a window one position longer, a block seen a
position early, a sink left out, a state that starts late, a group that is not masked are other functions by far more than
the tests allow)."""

import copy

import pytest
import torch

from clockwork_b200.cache import CacheManager
from clockwork_b200.config.registry import architecture_name, shape_config, spec_from_raw
from clockwork_b200.parts import PagedKVNeed, SlotStateNeed, build_model
from clockwork_b200.parts.model import tensor_decls_for_spec
from clockwork_b200.weights.loader import WeightMismatchError, check_declarations
from tests.nuzulorn_configs import CONFIGS, draw_weights, steady_routing, tensor_shapes, tokens_for
from tests.plain import nuzulorn_plain as plain


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    config, _ = CONFIGS[name]
    spec = spec_from_raw(config)
    assert architecture_name(config) == "Nuzulorn" and spec.architecture == "Nuzulorn"
    assert spec.tie_word_embeddings and spec.keeps_layer_outputs
    assert spec.pair_embedding.kind == "hashed_pair" and spec.pair_embedding["buckets"] == config["embedding"]["bigram"]["buckets"]
    decls = tensor_decls_for_spec(spec)
    shapes = tensor_shapes(config)
    check_declarations(decls, shapes, "test")
    assert {d.name for d in decls if not d.optional} == set(shapes)
    for i, (layer, listed) in enumerate(zip(spec.layers, config["layers"])):
        assert layer.block == "depth_averaged_residual"
        assert layer.block_params == {"residual_mult": config["residual_mult"], "run": i}
        m = listed["mixer"]
        if listed["type"] == "hgrn2":
            assert layer.mixer.kind == "hgrn2" and layer.mixer["dim"] == m["dim"]
        else:
            assert layer.mixer.kind == "window_attention" and layer.mixer["bias"] and layer.mixer["scale"] == m["scale"]
            if listed["type"] == "attention":
                assert layer.mixer["window"] == m["mask"]["size"] and layer.mixer["pool"] == m["mask"]["pool"]
                assert layer.mixer["sink"] == "zero" and layer.mixer["gate"] and layer.mixer["out_bias"]
                assert layer.mixer["rotary"] == m["rot"]
            else:
                assert layer.mixer["window"] is None and layer.mixer["sink"] is True and not layer.mixer["out_bias"]
                assert layer.mixer["softcap"] == m["softcap"] and layer.mixer["query_temperature"] == m["q_temp"]
                assert layer.mixer["distance_bias"] == {"halvings": 8.0}
        mlp = listed["mlp"]
        assert layer.ffn.kind == ("none" if mlp is None else "moe")
        if mlp is not None:
            groups = mlp["router"].get("groups")
            assert layer.ffn["top"] == mlp["router"]["top"] and layer.ffn["weight_scale"] == mlp["router"]["scale"]
            assert layer.ffn["scoring"] == "sigmoid" and layer.ffn["correction"]
            assert layer.ffn.get("groups", 1) == (groups["count"] if groups else 1)
            if groups:
                assert layer.ffn["group_rank"] == min(2, mlp["router"]["experts"] // groups["count"])


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_what_every_layer_asks_of_the_cache_manager(name):
    config, page = CONFIGS[name]
    model = build_model(spec_from_raw(config), torch.float32, "cpu")
    needs = model.cache_needs()
    assert sorted(needs) == list(range(len(config["layers"]) + 1))  # every layer, and the previous token above them
    assert needs[len(config["layers"])] == SlotStateNeed((1,), torch.int32)
    for i, listed in enumerate(config["layers"]):
        m = listed["mixer"]
        if listed["type"] == "hgrn2":
            assert needs[i] == SlotStateNeed((m["heads"] * m["dim"] * m["vdim"],))
        elif listed["type"] == "attention_2":
            assert needs[i] == PagedKVNeed(m["kv_heads"], m["dim"] + m["vdim"], None, planes=1)
        else:
            size, pool = m["mask"]["size"], m["mask"]["pool"]
            assert needs[i] == (PagedKVNeed(m["kv_heads"], m["dim"] + m["vdim"], max(size, pool), planes=1),
                                PagedKVNeed(m["kv_heads"], m["dim"] + m["vdim"], None, planes=1, every=pool))
    cache = CacheManager(needs, num_pages=64, page_size=page, num_state_slots=4)
    req = cache.open("a")
    cache.reserve(req, 100)
    for group, table in zip(cache.groups, req.tables):
        rows = -(-100 // group.every)
        assert len(table) == -(-rows // page)
    cache.check_invariants()
    cache.close("a")
    assert all(g.allocator.num_free == g.allocator.num_pages for g in cache.groups)


def test_a_page_group_of_one_row_per_block_of_positions():
    """Tables, slots and pools of a group that keeps one row per 5 positions beside one that keeps a window of rows."""
    tokens_need = PagedKVNeed(2, 8, 12, planes=1)
    blocks_need = PagedKVNeed(2, 8, None, planes=1, every=5)
    cache = CacheManager({0: (tokens_need, blocks_need)}, num_pages=16, page_size=4, num_state_slots=3)
    g_tokens, g_blocks = cache.group_of_need[tokens_need], cache.group_of_need[blocks_need]
    assert cache.groups[g_blocks].allocator.num_pages == -(-16 // 5) + 3  # a fifth of the rows, a part-filled page a request
    req = cache.open("a")
    cache.reserve(req, 23)
    assert len(req.tables[g_tokens]) == 6 and len(req.tables[g_blocks]) == 2  # 23 positions touch 5 blocks: 2 pages of 4 rows
    slots = cache.slots(req, g_blocks, 0, 23)
    table = req.tables[g_blocks]
    assert slots == [table[(p // 5) // 4] * 4 + (p // 5) % 4 for p in range(23)]
    assert slots[4] == slots[0] and slots[5] != slots[4]  # a block's positions share its row
    req.num_computed = 23
    cache.release_behind_window(req, 23)
    assert sum(p >= 0 for p in req.tables[g_tokens]) == 3 and all(p >= 0 for p in req.tables[g_blocks])  # the blocks' rows stay
    cache.reserve(req, 41)
    assert len(req.tables[g_blocks]) == 3  # position 40 opens block 8: a third page
    assert cache.view_order[0] == (tokens_need, blocks_need)  # the mixer's views come in the order of its needs
    other = cache.open("b")
    cache.reserve(other, 24)
    assert not cache.can_open(64 * 4)
    cache.check_invariants()
    cache.close("a")
    cache.close("b")
    assert all(g.allocator.num_free == g.allocator.num_pages for g in cache.groups)
    with pytest.raises(ValueError):
        CacheManager({0: PagedKVNeed(2, 8, 12, planes=1, every=3)}, num_pages=4, page_size=4)


def test_the_named_shapes_describe_themselves():
    for name in ("nuzulorn-tiny", "nuzulorn-2k"):
        spec = spec_from_raw(shape_config(name))
        assert len(tensor_decls_for_spec(spec)) > 10
    kinds = [layer.mixer.kind for layer in spec_from_raw(shape_config("nuzulorn-2k")).layers]
    assert kinds.count("hgrn2") == 2 and kinds.count("window_attention") == 6


def test_a_wrong_shape_and_a_missing_tensor_are_reported():
    config, _ = CONFIGS["A"]
    shapes = tensor_shapes(config)
    shapes["l2.mix.sink"] = (5, 4)
    del shapes["l1.mix.lower"]
    shapes["l0.dwa"] = (3,)
    with pytest.raises(WeightMismatchError) as e:
        check_declarations(tensor_decls_for_spec(spec_from_raw(config)), shapes, "test")
    text = str(e.value)
    assert "l2.mix.sink" in text and "l1.mix.lower" in text and "l0.dwa" in text


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "attention_3", "layer type"), (("layers", 0, "mixer", "mask"), {"size": 4}, "pool"),
    (("layers", 2, "mixer", "q_temp"), {"coef": 0.1}, "every"), (("layers", 1, "mixer", "vdim"), None, "vdim"),
    (("layers", 0, "mlp", "router", "scale"), None, "scale"), (("residual_mult",), None, "residual_mult"),
    (("embedding",), {"bigram": {"buckets": 5, "mul_prev": 1}}, "mul_cur"), (("layers", 0, "mlp", "kind"), "dense", "feed-forward")])
def test_configuration_errors_name_the_place(path, value, word):
    config = copy.deepcopy(CONFIGS["A"][0])
    at = config
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ValueError) as e:
        spec_from_raw(config)
    assert word in str(e.value)


def _model(name, seed=3):
    config = CONFIGS[name][0]
    return config, {k: v.double() for k, v in steady_routing(config, draw_weights(config, seed), seed).items()}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plain_implementation_does_not_look_ahead(name):
    config, w = _model(name)
    tokens = tokens_for(config, 50, salt=1)
    whole = plain.forward(config, w, tokens)
    for cut_at in (1, 7, 33):
        assert torch.allclose(plain.forward(config, w, tokens[:cut_at]), whole[:cut_at], atol=1e-9, rtol=0)
    other = list(tokens)
    other[20] = (other[20] + 1) % config["vocab"]
    changed = plain.forward(config, w, other)
    assert torch.equal(changed[:20], whole[:20])
    assert float((changed[21] - whole[21]).abs().max()) > 1e-3  # position 21 reads token 20 twice: through the layers and the pair table


def test_what_the_plain_implementation_is_sensitive_to():
    config = CONFIGS["A"][0]
    w = {k: v.double() for k, v in draw_weights(config, 3).items()}  # (routers as drawn: the groups' masks matter)
    tokens = tokens_for(config, 60, salt=2)
    want = plain.forward(config, w, tokens)

    def moved(change):
        other = copy.deepcopy(config)
        change(other)
        return float((plain.forward(other, w, tokens) - want).abs().max())

    assert moved(lambda c: c["layers"][0]["mixer"]["mask"].update(size=22)) > 0.01
    assert moved(lambda c: c["layers"][0]["mixer"]["mask"].update(pool=4)) > 0.01
    assert moved(lambda c: c["layers"][3]["mixer"]["mask"].update(size=6)) > 0.01
    assert moved(lambda c: c["layers"][2]["mixer"].update(softcap=400.0)) > 0.01
    assert moved(lambda c: c["layers"][2]["mixer"]["q_temp"].update(every=4)) > 0.01
    assert moved(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=3)) > 0.01
    assert moved(lambda c: c["layers"][1]["mlp"]["router"].update(scale=1.0)) > 0.01
    assert moved(lambda c: c.update(residual_mult=0.5)) > 0.01
    assert moved(lambda c: c["embedding"]["bigram"].update(mul_prev=30)) > 0.01
    # the first token reads the pair table's last row, the sink is in every softmax, the average reads every plane
    for name, change in (("bigram", lambda t: t[-1].add_(1.0)), ("l2.mix.sink", lambda t: t.sub_(30.0)), ("l3.dwa", lambda t: t[0].add_(0.5)),
                         ("l1.mix.lower", lambda t: t.mul_(0.0)), ("l0.mlp.correction", lambda t: t[0].add_(2.0))):
        t = w[name].clone()
        change(t)
        assert float((plain.forward(config, dict(w, **{name: t}), tokens) - want).abs().max()) > 0.01, name


def test_the_visible_blocks_of_a_position():
    # size 4, blocks of 3: position 6 sees positions 3..6 and block 0 (positions 0..2, which ends at 2 <= 6 - 4); block 1 ends at 5
    assert [plain.visible_blocks(t, 4, 3) for t in range(12)] == [0, 0, 0, 0, 0, 0, 1, 1, 1, 2, 2, 2]
    assert [plain.visible_blocks(t, 1, 1) for t in range(4)] == [0, 1, 2, 3]
    assert plain.visible_blocks(50, 200, 6) == 0
