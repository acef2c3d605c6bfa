"""Zonevik configurations drawn at random (sizes, head counts, layer order, windows, looped ranges, routers, constants), each
with random weights, in float32 against the plain implementation: a whole prompt, most of it in one step and the rest token by
token, and two unequal requests in one batch that decode together."""
import random

import pytest
import torch

import plain_zonevik as plain
from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _divisor(rng, n):
    return rng.choice([d for d in range(1, n + 1) if n % d == 0])


def _moe(rng):
    if rng.random() < 0.25:
        return None
    experts = rng.choice([2, 3, 4, 6, 8, 12])
    router = {"experts": experts}
    allowed = experts
    if rng.random() < 0.7:
        count = _divisor(rng, experts)
        keep = rng.randint(1, count)
        router["groups"] = {"count": count, "keep": keep}
        allowed = keep * (experts // count)
    router["top"] = rng.randint(1, allowed)
    return {"kind": "moe", "router": router, "expert": {"ff": rng.choice([6, 8, 20, 32])}}


def _heads(rng):
    heads = rng.choice([1, 2, 3, 4, 6])
    return heads, _divisor(rng, heads)


def draw_config(seed):
    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["attention", "delta", "parallel"])
        if kind == "attention":
            heads, kv = _heads(rng)
            dim = rng.choice([8, 12, 16, 24, 64])
            m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": rng.choice([dim, 8, 20]), "scale": rng.uniform(0.1, 0.5)}
            dims = rng.choice([0, 2, dim // 2 // 2 * 2, dim])
            if dims:
                m["rot"] = {"base": rng.choice([100.0, 5000.0, 1e6]), "dims": dims}
                if rng.random() < 0.6:
                    m["rot"]["scaling"] = {"factor": rng.choice([2.0, 8.0, 40.0]), "original": rng.choice([16, 64, 2048]),
                                           "fast": rng.choice([4.0, 32.0]), "slow": rng.choice([1.0, 2.0])}
        elif kind == "delta":
            heads, kv = _heads(rng)
            m = {"heads": heads, "kv_heads": kv, "dim": rng.choice([4, 8, 16, 32]), "vdim": rng.choice([4, 8, 24]), "conv": rng.randint(1, 5)}
        else:
            heads, kv = _heads(rng)
            dim = rng.choice([8, 16, 24])
            left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": rng.choice([dim, 12]), "scale": rng.uniform(0.1, 0.5)}
            if rng.random() < 0.8:
                left["mask"] = {"size": rng.choice([1, 3, 17, 40, 64, 90]), "keep_first": rng.choice([0, 1, 5, 64, 70])}
            rh = rng.choice([1, 2, 4, 6])
            vdim = rng.choice([4, 8, 12])
            right = {"heads": rh, "vdim": vdim, "state": rng.choice([4, 8, 16, 40, 64]), "groups": _divisor(rng, rh),
                     "conv": rng.randint(1, 5), "norm_groups": _divisor(rng, rh * vdim)}
            m = {"left": left, "right": right}
        layers.append({"type": kind, "mixer": m, "mlp": _moe(rng)})
    cfg = {"architecture": "Zonevik", "vocab": rng.randint(40, 300), "width": rng.choice([24, 40, 52, 64, 96]),
           "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-4])}, "layers": layers}
    if rng.random() < 0.7:
        cfg["embedding"] = {"scale": rng.uniform(0.5, 12.0)}
    if rng.random() < 0.75:
        start = rng.randrange(len(layers))
        cfg["loop"] = {"start": start, "stop": rng.randint(start + 1, len(layers)), "times": rng.randint(1, 3)}
    return cfg


@pytest.mark.parametrize("seed", range(24))
def test_a_configuration_drawn_at_random(pe, seed):
    cfg = draw_config(1000 + seed)
    w = plain.random_weights(cfg, 2000 + seed)
    eng = pe.Engine(None, config=pe.ZonevikConfig.from_dict(cfg), weights={k: v.to(DEV) for k, v in w.items()}, dtype="float32",
                    max_context_len=512, max_cache_tokens=64 * 24, max_batch=4)
    g = torch.Generator().manual_seed(seed)
    long = torch.randint(0, cfg["vocab"], (150,), generator=g).tolist()
    short = torch.randint(0, cfg["vocab"], (37,), generator=g).tolist()
    ref_long, ref_short = plain.forward(cfg, w, long).float(), plain.forward(cfg, w, short).float()
    tol = 3e-5
    s = eng.alloc_slot()
    whole = eng.step([pe.StepEntry(s, long, tuple(range(150)))]).clone()
    eng.free_slot(s)
    assert rel_err(whole.cpu(), ref_long) < tol, (seed, "whole", cfg)
    s = eng.alloc_slot()
    rows = [eng.step([pe.StepEntry(s, long[:110], (109,))]).clone()]
    for t in long[110:]:
        rows.append(eng.step([pe.StepEntry(s, [t], (0,))]).clone())
    eng.free_slot(s)
    assert rel_err(torch.cat(rows).cpu(), ref_long[109:]) < tol, (seed, "decoded", cfg)
    # two unequal requests start together, decode together, the shorter one ends earlier
    a, b = eng.alloc_slot(), eng.alloc_slot()
    out = eng.step([pe.StepEntry(a, long[:120], (119,)), pe.StepEntry(b, short[:30], (29,))]).clone()
    got_a, got_b = [out[0:1]], [out[1:2]]
    for i in range(12):
        entries = [pe.StepEntry(a, [long[120 + i]], (0,))]
        if 30 + i < len(short):
            entries.append(pe.StepEntry(b, [short[30 + i]], (0,)))
        out = eng.step(entries).clone()
        got_a.append(out[0:1])
        if len(entries) == 2:
            got_b.append(out[1:2])
            if 30 + i == len(short) - 1:
                eng.free_slot(b)
    eng.free_slot(a)
    assert rel_err(torch.cat(got_a).cpu(), ref_long[119:132]) < tol, (seed, "together, long", cfg)
    assert rel_err(torch.cat(got_b).cpu(), ref_short[29:37]) < tol, (seed, "together, short", cfg)
    assert not eng.cache.live_slots
    eng.cache.check()
