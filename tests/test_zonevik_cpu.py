"""What needs no GPU of the Zonevik architecture: its configuration file, its plan (the order of a looped range, tensor
names), the cache entries its parts ask for (a window that keeps the first positions' pages), and the plain
implementation's own consistency."""
import copy
from importlib import import_module

import pytest
import torch

import plain_zonevik as plain

CFG = {"architecture": "Zonevik", "vocab": 83, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
       "loop": {"start": 1, "stop": 3, "times": 2},
       "layers": [
           {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3},
            "mlp": {"kind": "moe", "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}, "expert": {"ff": 16}}},
           {"type": "parallel",
            "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3, "mask": {"size": 9, "keep_first": 2}},
                      "right": {"heads": 4, "vdim": 6, "state": 10, "groups": 2, "conv": 3, "norm_groups": 2}},
            "mlp": None},
           {"type": "attention",
            "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.25,
                      "rot": {"base": 1000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}},
            "mlp": {"kind": "moe", "router": {"experts": 3, "top": 1}, "expert": {"ff": 24}}},
           {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 16, "vdim": 8, "conv": 2}, "mlp": None}]}


def test_config_reads_every_layer_by_itself_and_writes_it_back(pe):
    cfg = pe.ZonevikConfig.from_dict(CFG)
    left, right = cfg.layers[1].mixer.left, cfg.layers[1].mixer.right
    assert (left.window, left.keep_first, left.vdim, right.conv, right.state, right.norm_groups) == (9, 2, 20, 3, 10, 2)
    assert cfg.layers[0].mlp.groups == 3 and cfg.layers[0].mlp.keep_groups == 2 and cfg.layers[2].mlp.groups == 1
    assert cfg.layers[2].mixer.rot_scaling.factor == 4.0 and cfg.layers[1].mlp is None
    assert cfg.loop.times == 2 and cfg.embedding_scale == 1.5
    assert pe.ZonevikConfig.from_dict(cfg.to_dict()) == cfg
    assert pe.config.architecture_of(CFG).name == "Zonevik"
    for path, value, word in [(("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "left", "kv_heads"), 3, "multiple"),
                              (("layers", 2, "mixer", "rot", "dims"), 18, "dims"), (("layers", 0, "mlp", "kind"), "dense", "kind"),
                              (("layers", 0, "mlp", "router", "top"), 5, "top"), (("norm",), None, "norm"),
                              (("layers", 1, "mixer", "right", "groups"), 3, "multiple"), (("loop", "stop"), 5, "loop"),
                              (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),
                              (("layers", 1, "mixer", "right", "norm_groups"), 5, "norm_groups")]:
        bad = copy.deepcopy(CFG)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(pe.ConfigError, match=word):
            pe.ZonevikConfig.from_dict(bad)
    # a model without a loop, a scale, a mask or rotation is one too
    plainer = copy.deepcopy(CFG)
    del plainer["loop"], plainer["embedding"], plainer["layers"][1]["mixer"]["left"]["mask"], plainer["layers"][2]["mixer"]["rot"]
    cfg2 = pe.ZonevikConfig.from_dict(plainer)
    assert cfg2.loop is None and cfg2.embedding_scale == 1.0 and cfg2.layers[1].mixer.left.window is None
    plan = pe.config.architecture("Zonevik").plan(cfg2)
    assert not plan.keep_embedding_output and not plan.positions and [r.block for r in plan.order] == [0, 1, 2, 3]


def test_plan_runs_the_looped_layers_again_with_cache_entries_of_their_own(pe):
    loader = import_module("pytorch-engine_b200.weights.loader")
    cfg = pe.ZonevikConfig.from_dict(CFG)
    plan = pe.config.architecture("Zonevik").plan(cfg)
    assert [r.block for r in plan.order] == [r for r, _ in plain.run_order(CFG)] == [0, 1, 2, 1, 2, 3]
    assert len({r.cache_entry for r in plan.order}) == 6 and plan.keep_embedding_output
    assert "inject" in plan.blocks[1].parts and all("inject" not in plan.blocks[i].parts for i in (0, 2, 3))
    want = loader.expected_tensors(plan)
    have = plain.random_weights(CFG, 0)
    assert set(want) == set(have)
    for name, decl in want.items():
        assert decl.fits(have[name].shape), name
    assert [b.arrangement for b in plan.blocks] == ["sandwich"] * 4
    assert plan.blocks[1].mixer_names() == ("left", "right") and plan.blocks[0].mixer_names() == ("mixer",)
    assert "ffn" not in plan.blocks[1].parts and plan.blocks[0].part("ffn").params["choice"] == "sigmoid_groups"
    assert plan.head.weights["weight"] == plan.embedding.weights["weight"] == "embed" and len(plan.positions) == 1
    assert plan.blocks[0].part("mixer").params["decay"] == "head" and plan.blocks[0].part("mixer_norm").kind == "dynamic_tanh"


def test_cache_entries_of_the_parts_and_the_pages_a_window_keeps(pe):
    parts = pe.parts
    cfg = pe.ZonevikConfig.from_dict(CFG)
    plan = pe.config.architecture("Zonevik").plan(cfg)
    reqs = {}
    for run in plan.order:
        b = plan.blocks[run.block]
        for name in b.mixer_names():
            spec = b.part(name)
            key = run.cache_entry if len(b.mixer_names()) == 1 else (run.cache_entry, name)
            reqs[key] = parts.lookup("mixer", spec.kind).cache_request(spec.params)
    assert len(reqs) == 8                              # two runs of the two-mixer block, four runs of one-mixer blocks
    left = reqs[(1, "left")]
    assert left.window == 9 and left.keep_first == 2 and left.value_dim == 20
    assert dict((n, s) for n, s, _ in reqs[(1, "right")].state_shapes) == {"S": (4, 10, 6), "conv": (2, 4 * 6 + 2 * 2 * 10)}
    assert dict((n, s) for n, s, _ in reqs[0].state_shapes) == {"S": (4, 8, 12), "conv": (2, 2 * 2 * 8 + 4 * 12)}
    spec = copy.deepcopy(dict(plan.blocks[1].part("left").params))
    spec["window"], spec["keep_first"] = 100, 70
    wide = parts.lookup("mixer", "attention").cache_request(spec)
    cache = pe.cache.PagedCache({0: wide, 1: reqs[0]}, max_tokens=1024, max_slots=3, max_seq_len=640, dtype=torch.float32, device="cpu")
    s = cache.alloc_slot()
    cache.view(1).state("S")[s].fill_(3.0)
    for n in (390, 400, 500):
        cache.reserve(s, n)
        cache.commit(s, n)
    held = [i for i, p in enumerate(cache.groups[0].pages_of_slot[s]) if p >= 0]
    assert held == [0, 1, 6, 7], held                  # positions 0..69 stay; the next query at 500 sees keys from 401 on
    cache.check()
    cache.free_slot(s)
    assert cache.alloc_slot() == s and float(cache.view(1).state("S")[s].abs().max()) == 0.0
    cache.check()


def test_plain_implementation_is_causal_and_its_masks_and_loop_matter():
    w = plain.random_weights(CFG, 5)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, CFG["vocab"], (40,), generator=g).tolist()
    whole = plain.forward(CFG, w, toks)
    assert (whole[:25] - plain.forward(CFG, w, toks[:25])).abs().max() < 1e-9
    # the window matters from the first position beyond it on, unless the kept positions cover the difference
    wider = copy.deepcopy(CFG)
    wider["layers"][1]["mixer"]["left"]["mask"]["size"] = 10
    other = plain.forward(wider, w, toks)
    assert (whole[:11] - other[:11]).abs().max() < 1e-12 and (whole[11] - other[11]).abs().max() > 1e-7
    kept = copy.deepcopy(CFG)
    kept["layers"][1]["mixer"]["left"]["mask"]["keep_first"] = 3
    other = plain.forward(kept, w, toks)
    assert (whole[:11] - other[:11]).abs().max() < 1e-12 and (whole[11] - other[11]).abs().max() > 1e-7
    once = copy.deepcopy(CFG)
    once["loop"]["times"] = 1
    assert (whole - plain.forward(once, w, toks)).abs().max() > 1e-4
    # rounding the products to bfloat16 moves the logits a little, not much
    with plain.stored(torch.bfloat16):
        rounded = plain.forward(CFG, w, toks)
    assert 1e-5 < (whole - rounded).abs().max() < 0.2 * whole.abs().max()


def test_router_of_the_plain_implementation():
    s = torch.tensor([[0.9, 0.1, 0.1, 0.5, 0.6, 0.2, 0.7, 0.45, 0.0]], dtype=torch.float64)
    chosen, weight = plain.router_choice(s, {"top": 3, "groups": {"count": 3, "keep": 2}})
    assert sorted(chosen[0].tolist()) == [3, 4, 6] and torch.allclose(weight, s[0][chosen[0]][None])   # 0.9 sits in the weakest group
    chosen, _ = plain.router_choice(s, {"top": 3})
    assert sorted(chosen[0].tolist()) == [0, 4, 6]
