"""What needs no GPU of the Vemepel architecture: its configuration file, its plan and tensor names, the cache entries
its parts ask for (with the pages that a chunk mask lets go), and the plain implementation's own consistency."""
import copy
from importlib import import_module

import pytest
import torch

import plain_vemepel as plain

CFG = {"architecture": "Vemepel", "vocab": 83, "width": 40, "logit_scale": 0.8, "norm": {"eps": 1e-5},
       "layers": [
           {"type": "attention",
            "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.3, "diff": 0.55, "mask": {"size": 9}},
            "mlp": {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 16}}},
           {"type": "latent_attention_2",
            "mixer": {"heads": 2, "dim": 8, "rot_dim": 6, "vdim": 10, "kv_rank": 14, "scale": 0.25, "rot": {"base": 700.0, "dims": 4}},
            "mlp": {"kind": "dense", "ff": 32}},
           {"type": "attention",
            "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.2, "diff": 0.3, "mask": {"size": 9}, "kv_from": 0},
            "mlp": None},
           {"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "vdim": 4, "kv_rank": 10, "scale": 0.4},
            "mlp": {"kind": "dense", "ff": 24}},
           {"type": "attention",
            "mixer": {"heads": 2, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.2, "diff": 0.3, "mask": {"size": 13}, "kv_from": 0},
            "mlp": None}]}


def _without_last(cfg):
    c = copy.deepcopy(cfg)
    c["layers"] = c["layers"][:-1]
    return c


def test_config_reads_every_layer_by_itself_and_writes_it_back(pe):
    cfg = pe.VemepelConfig.from_dict(CFG)
    a, l2, l1 = cfg.layers[0].mixer, cfg.layers[1].mixer, cfg.layers[3].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.chunk, a.kv_from, a.diff) == (4, 2, 12, 20, 9, None, 0.55)
    assert (l2.rot_dim, l2.rot_dims, l2.rot_base, l2.kv_rank) == (6, 4, 700.0, 14) and (l1.rot_dim, l1.vdim) == (0, 4)
    assert cfg.layers[2].mixer.kv_from == 0 and cfg.layers[2].mlp is None and cfg.layers[0].mlp.top == 2
    assert cfg.logit_scale == 0.8 and cfg.to_dict()["layers"] == CFG["layers"]
    assert pe.VemepelConfig.from_dict(cfg.to_dict()) == cfg
    assert pe.config.architecture_of(CFG).name == "Vemepel"
    for path, value, word in [(("layers", 0, "type"), "conv", "type"), (("layers", 0, "mixer", "kv_heads"), 3, "multiple"),
                              (("layers", 1, "mixer", "rot", "dims"), 8, "dims"), (("layers", 0, "mlp", "kind"), "sparse", "kind"),
                              (("layers", 0, "mlp", "router", "top"), 8, "top"), (("norm",), None, "norm"),
                              (("layers", 2, "mixer", "kv_from"), 3, "kv_from"), (("layers", 2, "mixer", "kv_from"), 1, "kv_from"),
                              (("layers", 2, "mixer", "vdim"), 12, "kv_from|equal"), (("layers", 3, "mixer", "kv_rank"), 0, "kv_rank")]:
        bad = copy.deepcopy(CFG)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(pe.ConfigError, match=word):
            pe.VemepelConfig.from_dict(bad)


def test_plan_names_the_tensors_of_the_plain_implementation(pe):
    loader = import_module("pytorch-engine_b200.weights.loader")
    cfg = pe.VemepelConfig.from_dict(CFG)
    plan = pe.config.architecture("Vemepel").plan(cfg)
    want = loader.expected_tensors(plan)
    have = plain.tensor_shapes(CFG)
    assert set(want) == set(have)
    for name, decl in want.items():
        assert decl.fits(have[name]), name
    assert [b.arrangement for b in plan.blocks] == ["sandwich_depth"] * 5
    assert plan.blocks[0].keeper_names() == ("shift", "mixer", "average") and plan.blocks[0].mixer_names() == ("mixer",)
    assert "ffn" not in plan.blocks[2].parts and plan.blocks[0].part("ffn").params["choice"] == "top_logits"
    assert plan.blocks[3].part("average").params["terms"] == 5 and plan.blocks[1].part("mixer").params["gate"] == "feature"
    assert plan.ignored == ("l2.norm2", "l2.norm2b", "l4.norm2", "l4.norm2b")
    # a layer that reads another layer's keys names that entry for its mixer alone, and writes nothing there
    run = plan.order[2]
    assert (run.cache_entry, run.writes_cache, run.shared) == (0, False, ("mixer",))
    assert run.entry_of("mixer") == 0 and run.entry_of("shift") == 2 and run.writes("shift") and not run.writes("mixer")
    assert plan.order[0].entry_of("mixer") == 0 and plan.order[0].writes("mixer")
    # readers with chunks of 9, 9 and 13: the cache keeps everything; with one chunk for all it may let pages go
    assert plan.blocks[0].part("mixer").params["cache_chunk"] is None
    same = pe.config.architecture("Vemepel").plan(pe.VemepelConfig.from_dict(_without_last(CFG)))
    assert same.blocks[0].part("mixer").params["cache_chunk"] == 9
    assert len(plan.positions) == 1 and next(iter(plan.positions.values())).params["style"] == "interleaved"


def test_cache_entries_of_the_parts(pe):
    """A latent layer keeps one row per position that is key and value at once; a differential layer twice as many key
    heads as value heads; every layer a float32 row for its token shift, zero when a slot is taken again."""
    parts = pe.parts
    cfg = pe.VemepelConfig.from_dict(_without_last(CFG))
    plan = pe.config.architecture("Vemepel").plan(cfg)
    reqs = {}
    for run in plan.order:
        b = plan.blocks[run.block]
        for name in b.keeper_names():
            if run.writes(name):
                role, spec = b.parts[name]
                cls = parts.lookup(role, spec.kind)
                if hasattr(cls, "cache_request"):
                    reqs[(run.entry_of(name), name)] = cls.cache_request(spec.params)
    assert sorted(k for k in reqs if k[1] == "mixer") == [(0, "mixer"), (1, "mixer"), (3, "mixer")]
    assert sorted(k[0] for k in reqs if k[1] == "shift") == [0, 1, 2, 3]
    d, lat = reqs[(0, "mixer")], reqs[(1, "mixer")]
    assert (d.kv_heads, d.n_value_heads, d.head_dim, d.value_dim, d.chunk) == (4, 2, 12, 20, 9)
    assert (lat.kv_heads, lat.head_dim, lat.value_dim, lat.values_in_keys) == (1, 20, 14, True)
    assert reqs[(3, "mixer")].head_dim == 10 and reqs[(2, "shift")].state_shapes == (("prev", (40,), "float32"),)
    cache = pe.cache.PagedCache(reqs, max_tokens=64 * 6, max_slots=3, max_seq_len=64 * 8, dtype=torch.float32, device="cpu")
    v = cache.view((0, "mixer"))
    assert tuple(v.k_pages.shape) == (6, 4, 64, 12) and tuple(v.v_pages.shape) == (6, 2, 64, 20)
    v = cache.view((1, "mixer"))
    assert tuple(v.k_pages.shape) == (6, 1, 64, 20) and v.v_pages.data_ptr() == v.k_pages.data_ptr()
    s = cache.alloc_slot()
    cache.view((2, "shift")).state("prev")[s].fill_(3.0)
    cache.reserve(s, 300)
    cache.commit(s, 300)
    # the chunked group lets go of the pages before the block of 9 positions that position 300 falls into (297 // 64 = 4
    # pages); the latent groups keep all five
    free = {g.request.head_dim: g.pool.free_count for g in cache.groups if g.request.kind == "kv"}
    assert free == {12: 5, 20: 1, 10: 1}
    cache.reserve(s, 330)
    cache.commit(s, 330)
    cache.free_slot(s)
    assert cache.alloc_slot() == s
    assert float(cache.view((2, "shift")).state("prev")[s].abs().max()) == 0.0
    cache.check()


def test_plain_implementation_whole_token_by_token_and_in_portions():
    w = plain.random_weights(CFG, 5)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, CFG["vocab"], (40,), generator=g).tolist()
    whole = plain.forward(CFG, w, toks)
    one = plain.forward(CFG, w, toks, portions=[1] * 40)
    assert (whole - one).abs().max() < 1e-9
    parts = plain.forward(CFG, w, toks, portions=[7, 2, 31])
    assert (whole - parts).abs().max() < 1e-9
    # the chunk matters: a larger one gives other logits from the first position on at which it shows a key more ...
    wider = copy.deepcopy(CFG)
    wider["layers"][0]["mixer"]["mask"]["size"] = 10
    other = plain.forward(wider, w, toks)
    assert (whole[:9] - other[:9]).abs().max() < 1e-12 and (whole[9] - other[9]).abs().max() > 1e-6
    # ... the reader's own mask is its own: another chunk there changes nothing before position 9 either
    reader = copy.deepcopy(CFG)
    reader["layers"][2]["mixer"]["mask"]["size"] = 11
    other = plain.forward(reader, w, toks)
    assert (whole[:9] - other[:9]).abs().max() < 1e-12 and (whole[9] - other[9]).abs().max() > 1e-6
    # ... the token shift reaches one token back: another first token moves the second token's logits
    moved = plain.forward(CFG, w, [toks[0] + 1] + toks[1:])
    assert (moved[1] - whole[1]).abs().max() > 1e-6


def test_mechanisms_of_the_plain_implementation():
    f = torch.float64
    # the router: the largest of logits + bias, ties to the lower index, softmax over the chosen alone
    router = torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.5, 0.5], [1.0, 0.0]], dtype=f)
    bias = torch.tensor([0.0, 0.0, 1.5, 0.0], dtype=f)
    which, weight = plain.choose_experts(torch.tensor([[2.0, 0.0]], dtype=f), router, bias, 3)
    assert which.tolist() == [[2, 0, 3]]
    assert torch.allclose(weight, torch.softmax(torch.tensor([2.5, 2.0, 2.0], dtype=f), 0)[None])
    # the turn of adjacent pairs: a quarter turn of (1, 0) at position 1 with angle pi / 2
    x = torch.tensor([[[1.0, 0.0, 5.0, 7.0]]], dtype=f)
    base = (2.0 / torch.pi) ** 2          # dims = 2: f_0 = 1, so use position pi/2 through the base of a second pair
    out = plain.rotate_pairs(x, torch.tensor([1]), base, 2)
    assert torch.allclose(out[0, 0], torch.tensor([torch.cos(torch.tensor(1.0, dtype=f)), torch.sin(torch.tensor(1.0, dtype=f)), 5.0, 7.0], dtype=f))
    # the token shift keeps the unmoved last row
    h = torch.arange(6, dtype=f).view(3, 2)
    moved, kept = plain.token_shift(h, torch.zeros(2, dtype=f), torch.tensor([0.5, 1.0], dtype=f))
    assert moved.tolist() == [[0.0, 0.0], [1.0, 1.0], [3.0, 3.0]] and kept.tolist() == [4.0, 5.0]
    # PolyNorm of a constant row: every power has root mean square |z|^p
    z = torch.full((1, 8), 2.0, dtype=f)
    assert torch.allclose(plain.polynorm(z, torch.tensor([1.0, 2.0, 3.0, 0.5]), 0.0), torch.full((1, 8), 6.5, dtype=f))
