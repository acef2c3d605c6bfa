"""The Zonevik architecture on the engine against the plain implementation in ``plain_zonevik.py``: mechanisms at kernel level
with inputs made so that a fault shows, every mechanism alone as a one-layer model, then whole models: prompts, token-by-token
decoding, prompts in portions, unequal batches, slots and pages used again, long decoding, generation through the entry point."""
import copy

import pytest
import torch

import plain_zonevik as plain
from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"float32": 3e-5, "bfloat16": 2e-2}
# a gap between two experts' (or two groups') scores, in units of the router's logits, below which a bfloat16 rounding may
# choose otherwise
CLOSE_CALL = 0.01
# positions behind one whose nearly tied choice fell the other way that are left out with it (the convolutions' taps, the
# recurrent state and the window carry the other expert's output on)
AFTER_A_CLOSE_CALL = 3


def _att(heads, kv, dim, vdim, scale, dims=0, base=10000.0, scaling=None):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if dims:
        d["rot"] = {"base": base, "dims": dims}
        if scaling:
            d["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return d


def _left(heads, kv, dim, vdim, scale, window=None, keep=0):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        d["mask"] = {"size": window, "keep_first": keep}
    return d


def _right(heads, vdim, state, groups, conv, parts):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": parts}


def _moe(experts, top, ff, groups=None):
    r = {"experts": experts, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": r, "expert": {"ff": ff}}


# The tests' own models.  A has sizes that are no multiple of 8 or 32 anywhere, a looped range in the middle that runs three
# times, a window that is no multiple of a page with a few kept positions, partial rotation with scaled frequencies and whole
# rotation without, convolutions of 3 and 2 taps, one chosen expert without groups and all experts of the kept groups chosen,
# a layer without feed-forward.  B has the sizes that the tensor-core attention kernels take, no loop, a scale of one, kept
# positions that fill more than a page, a state of 128 rows, one group, one norm part, convolutions of 4 taps and of 1.
# C loops over all its layers once, has a window of exactly a page without kept positions and one where more positions are
# kept than the window is long, a state-space head with more rows than a thread keeps in registers, a single head.
CONFIGS = {
    "A": {"architecture": "Zonevik", "vocab": 131, "width": 72, "norm": {"eps": 2e-6}, "embedding": {"scale": 3.0},
          "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [
              {"type": "attention", "mixer": _att(4, 2, 24, 16, 0.3, 16, 1000.0, (8.0, 64, 16.0, 2.0)), "mlp": _moe(6, 2, 40, (3, 2))},
              {"type": "parallel", "mixer": {"left": _left(6, 2, 16, 24, 0.3, 37, 3), "right": _right(4, 20, 24, 2, 3, 4)},
               "mlp": _moe(5, 1, 24)},
              {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 20, "conv": 3}, "mlp": None},
              {"type": "attention", "mixer": _att(3, 3, 8, 8, 0.4, 8, 300.0), "mlp": _moe(4, 4, 16, (2, 2))}]},
    "B": {"architecture": "Zonevik", "vocab": 256, "width": 128, "norm": {"eps": 1e-6},
          "layers": [
              {"type": "delta", "mixer": {"heads": 4, "kv_heads": 4, "dim": 64, "vdim": 64, "conv": 1}, "mlp": _moe(8, 2, 64, (2, 1))},
              {"type": "attention", "mixer": _att(4, 2, 64, 64, 0.125, 64, 30000.0, (2.0, 128, 8.0, 1.0)), "mlp": _moe(8, 3, 64, (8, 5))},
              {"type": "parallel", "mixer": {"left": _left(4, 2, 64, 64, 0.125, 100, 70), "right": _right(4, 64, 128, 1, 4, 1)},
               "mlp": _moe(4, 2, 128)}]},
    "C": {"architecture": "Zonevik", "vocab": 90, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
          "loop": {"start": 0, "stop": 2, "times": 1},
          "layers": [
              {"type": "parallel", "mixer": {"left": _left(2, 1, 8, 12, 0.5, 64, 0), "right": _right(2, 12, 136, 2, 2, 2)}, "mlp": None},
              {"type": "parallel", "mixer": {"left": _left(1, 1, 40, 8, 0.2, 20, 33), "right": _right(1, 100, 8, 1, 4, 5)},
               "mlp": _moe(3, 2, 20, (3, 2))}]},
    # D: nothing is a multiple of 4: no kernel may take its 16-byte paths; five taps; the last layer alone runs twice
    "D": {"architecture": "Zonevik", "vocab": 77, "width": 54, "norm": {"eps": 3e-6}, "embedding": {"scale": 2.5},
          "loop": {"start": 2, "stop": 3, "times": 2},
          "layers": [
              {"type": "attention", "mixer": _att(3, 1, 10, 6, 0.3, 6, 100.0, (3.0, 16, 4.0, 1.0)), "mlp": _moe(3, 2, 10)},
              {"type": "parallel", "mixer": {"left": _left(2, 2, 6, 10, 0.4, 5, 2), "right": _right(3, 6, 5, 3, 5, 9)}, "mlp": None},
              {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 6, "vdim": 10, "conv": 5}, "mlp": _moe(6, 3, 14, (2, 1))}]},
}
SEEDS = {"A": 31, "B": 32, "C": 33, "D": 34}


def _tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class Models:
    def __init__(self, pe):
        self.pe = pe
        self.configs = dict(CONFIGS)
        self.weights = {}
        self.engines = {}
        self.refs = {}

    def add(self, key, cfg, seed):
        self.configs[key] = cfg
        SEEDS[key] = seed

    def w(self, key):
        if key not in self.weights:
            self.weights[key] = plain.random_weights(self.configs[key], SEEDS[key])
        return self.weights[key]

    def engine(self, key, dtype, **kw):
        ident = (key, dtype, tuple(sorted(kw.items())))
        if ident not in self.engines:
            cfg = self.pe.ZonevikConfig.from_dict(self.configs[key])
            args = dict(dtype=dtype, max_context_len=1024, max_cache_tokens=64 * 40, max_batch=8)
            args.update(kw)
            self.engines[ident] = self.pe.Engine(None, config=cfg, weights={k: v.to(DEV) for k, v in self.w(key).items()}, **args)
        return self.engines[ident]

    def ref(self, key, toks):
        ident = (key, tuple(toks))
        if ident not in self.refs:
            margins = []
            self.refs[ident] = plain.forward(self.configs[key], self.w(key), toks, margins=margins).float()
            self.refs[ident + ("decided",)] = (torch.stack(margins).min(0).values if margins
                                               else torch.full((len(toks),), float("inf"), dtype=torch.float64))
        return self.refs[ident]

    def decided(self, key, toks):
        """Per position: the smallest gap by which any router of the model chose its experts there."""
        self.ref(key, toks)
        return self.refs[(key, tuple(toks), "decided")]

    def noise(self, key, toks):
        """How far rounding to bfloat16 alone moves each position's logits (root mean square over the vocabulary)."""
        ident = (key, tuple(toks), "noise")
        if ident not in self.refs:
            with plain.stored(torch.bfloat16):
                rounded = plain.forward(self.configs[key], self.w(key), toks)
            self.refs[ident] = (rounded - self.ref(key, toks).double()).pow(2).mean(dim=1).sqrt()
        return self.refs[ident]

    def check(self, key, dtype, toks, got, positions, what):
        """float32: every logit within 3e-5 of the largest.  bfloat16: the error is held against what rounding alone does
        in the plain implementation: on average no more than twice that, and at no more than one position in fifty (or
        one) above three times the larger of that position's own figure and the average.  Positions where a router's choice
        hung on a gap of less than CLOSE_CALL (in the router's logits) between two scores are left out: there a rounding may
        pick another expert, which moves that position by ten times what rounding does elsewhere; where it did, the
        AFTER_A_CLOSE_CALL positions behind it are left out too.  The average also leaves the worst position out."""
        positions = list(positions)
        ref = self.ref(key, toks)[positions]
        got = got.float().cpu()
        assert got.shape == ref.shape, what
        if dtype == "float32":
            err = float((got.double() - ref.double()).abs().max() / ref.double().abs().max())
            assert err < TOL[dtype], f"{what}: error {err:.3e} (limit {TOL[dtype]:.0e})"
            return
        noise = self.noise(key, toks)
        floor = float(noise.mean())
        tied = self.decided(key, toks) < CLOSE_CALL
        all_err = (got.double() - ref.double()).pow(2).mean(dim=1).sqrt()
        left_out = set()
        for p, e in zip(positions, all_err.tolist()):
            if bool(tied[p]):
                left_out.add(p)
                if e > 3.0 * max(float(noise[p]), floor):          # it fell the other way: the next few positions feel it
                    left_out.update(range(p + 1, p + 1 + AFTER_A_CLOSE_CALL))
        keep = [i for i, p in enumerate(positions) if p not in left_out]
        assert len(keep) >= max(1, len(positions) // 4), f"{what}: too many positions with nearly tied experts"
        positions, got, ref = [positions[i] for i in keep], got[keep], ref[keep]
        noise = self.noise(key, toks)
        err = (got.double() - ref.double()).pow(2).mean(dim=1).sqrt()
        floor = float(noise.mean())
        mean = float(err.mean()) if len(positions) < 5 else float((err.sum() - err.max()) / (len(positions) - 1))
        assert mean <= 2.0 * max(float(noise[positions].mean()), floor), \
            f"{what}: mean error {mean:.3e}, rounding alone {float(noise[positions].mean()):.3e}"
        over = int((err > 3.0 * torch.clamp(noise[positions], min=floor)).sum())
        assert over <= max(1, len(positions) // 50), f"{what}: {over} of {len(positions)} positions beyond three times rounding"


@pytest.fixture(scope="module")
def models(pe):
    return Models(pe)


def _entry(pe, slot, toks, want):
    return pe.StepEntry(slot, toks, tuple(want))


def _batch(q_lens, slots):
    """(token_seq, seq_slot, seq_qstart) of a step, int32 on the device."""
    seq = torch.tensor([b for b, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    qstart = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    return seq, torch.tensor(slots, dtype=torch.int32, device=DEV), qstart


# ---- mechanisms at kernel level -----------------------------------------------------------------------------------
@pytest.mark.parametrize("dim", [50, 72])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_tanh_norm_alone_with_its_add_and_the_next_norm(pe, dtype, dim):
    ops = pe.kernels.ops
    g = torch.Generator().manual_seed(1)
    n = 37
    x = torch.randn(n, dim, generator=g) * 3
    d = (torch.randn(n, dim, generator=g) * 2).to(dtype)
    w = {f"n{i}{s}": torch.randn(dim, generator=g) for i in (1, 2) for s in ("", ".b")}
    w["n1.alpha"], w["n2.alpha"] = torch.tensor(0.7), torch.tensor(1.9)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    rows = torch.tensor([5, 0, 36], dtype=torch.int32, device=DEV)
    out = torch.empty(3, dim, dtype=dtype, device=DEV)
    ops.dyt(x.to(DEV), w["n1"].to(DEV), w["n1.b"].to(DEV), 0.7, out, rows)
    assert (out.float().cpu() - plain.tanh_norm(x[[5, 0, 36]].double(), w, "n1")).abs().max() < tol
    stream = x.clone().to(DEV)
    nxt = torch.empty(n, dim, dtype=dtype, device=DEV)
    ops.dyt_add(stream, d.to(DEV), w["n1"].to(DEV), w["n1.b"].to(DEV), 0.7, (w["n2"].to(DEV), w["n2.b"].to(DEV), 1.9), nxt)
    want = x.double() + plain.tanh_norm(d.double(), w, "n1")
    assert (stream.cpu() - want).abs().max() < 1e-5
    assert (nxt.float().cpu() - plain.tanh_norm(want, w, "n2")).abs().max() < tol
    # two outputs side by side: each over its own root mean square, weighted, half their sum; alone, and with the norm on
    # it, the add and the next norm in the same kernel
    e = (torch.randn(n, dim, generator=g) * 0.3).to(dtype)
    wa, wb = torch.randn(dim, generator=g), torch.randn(dim, generator=g)
    mix = 0.5 * (plain.unit(d.double(), 1e-5) * wa + plain.unit(e.double(), 1e-5) * wb)
    out = torch.empty(n, dim, dtype=dtype, device=DEV)
    ops.rmsnorm_pair_mix(d.to(DEV), e.to(DEV), wa.to(DEV), wb.to(DEV), 1e-5, 0.5, 0.5, out)
    assert (out.float().cpu() - mix).abs().max() < tol
    for with_next in (False, True):
        stream = x.clone().to(DEV)
        nxt.fill_(float("nan"))
        ops.rmsnorm_pair_mix_dyt_add(d.to(DEV), e.to(DEV), wa.to(DEV), wb.to(DEV), 1e-5, 0.5, 0.5, stream,
                                     (w["n1"].to(DEV), w["n1.b"].to(DEV), 0.7),
                                     (w["n2"].to(DEV), w["n2.b"].to(DEV), 1.9) if with_next else None, nxt if with_next else None)
        want = x.double() + plain.tanh_norm(mix, w, "n1")
        assert (stream.cpu() - want).abs().max() < 1e-5
        if with_next:
            assert (nxt.float().cpu() - plain.tanh_norm(want, w, "n2")).abs().max() < tol


def test_router_groups_two_best_scores_kept_groups_and_plain_scores_as_weights(pe):
    """A group with the single best expert loses against groups whose two best are better together; the weights are the
    sigmoid scores themselves; equal scores go to the lower index; groups of one; no groups at all."""
    ops = pe.kernels.ops
    z = torch.tensor([[4.0, -9.0, -9.0, 1.0, 1.5, 0.5, 2.0, 0.9, -1.0],       # group 0 has the best expert and loses
                      [0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0],
                      [-2.0, -1.0, -3.0, 5.0, 5.1, 5.2, -4.0, 6.0, -8.0]], device=DEV)
    for groups, keep, top in ((3, 2, 3), (3, 1, 2), (9, 4, 4), (1, 1, 3), (3, 3, 9)):
        chosen = torch.empty(3, top, dtype=torch.int32, device=DEV)
        weight = torch.empty(3, top, device=DEV)
        ops.moe_route_sigmoid_groups(z, top, groups, keep, chosen, weight)
        r = {"top": top}
        if groups > 1:
            r["groups"] = {"count": groups, "keep": keep}
        want_c, want_w = plain.router_choice(torch.sigmoid(z.double().cpu()), r)
        for t in (0, 2):
            assert sorted(chosen[t].tolist()) == sorted(want_c[t].tolist()), (groups, keep, top, t)
        assert (weight.cpu().double() - torch.sigmoid(z.double().cpu()).gather(1, chosen.cpu().long())).abs().max() < 1e-6
        if (groups, keep, top) == (3, 2, 3):
            assert 0 not in chosen[0].tolist() and chosen[1].tolist() == [0, 1, 2]


class Pages:
    """A hand-made paged cache for kernel tests: sequence b's logical page i is physical page ``table[b][i]``."""

    def __init__(self, lens, kvh, d, dv, seed=0):
        g = torch.Generator().manual_seed(seed)
        n_pages = sum(-(-n // 64) for n in lens) + 3
        order = torch.randperm(n_pages, generator=g).tolist()
        self.table = torch.full((len(lens), max(-(-n // 64) for n in lens) + 1), -1, dtype=torch.int32)
        for b, n in enumerate(lens):
            for i in range(-(-n // 64)):
                self.table[b, i] = order.pop()
        self.k = torch.zeros(n_pages, kvh, 64, d)
        self.v = torch.zeros(n_pages, kvh, 64, dv)
        self.n_pages = n_pages

    def put(self, b, pos, k, v):
        page = int(self.table[b, pos // 64])
        self.k[page, :, pos % 64] = k
        self.v[page, :, pos % 64] = v


@pytest.mark.parametrize("kernel", ["float32 arithmetic", "tensor cores"])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window,keep", [(37, 3), (64, 64), (20, 70), (130, 1), (50, 0), (100, 129)])
def test_keys_at_the_edges_of_the_window_and_of_the_kept_positions(pe, decode, window, keep, kernel):
    """One key matches the query far better than all others.  At the window's oldest position, or at the last kept position,
    the output is its value; one position further back (or one behind the kept ones and in front of the window) it must not
    be seen, and the output is the average of the values that are (all of score zero).  The query sits so that the edges fall
    before, on and behind page borders; a prompt's rows are checked as a whole step of several queries."""
    ops = pe.kernels.ops
    nh, nkv, d, dv = (6, 2, 16, 24) if kernel == "float32 arithmetic" else (8, 2, 64, 64)
    dt = torch.float32 if kernel == "float32 arithmetic" else torch.bfloat16
    g = torch.Generator().manual_seed(window)
    for n in (window + 1, 128, 129, 300, 700):
        i = n - 1                                   # the last query's position
        lo = max(0, i - window + 1)
        spots = {lo: True, lo - 1: lo - 1 < keep, keep - 1: True, keep: keep >= lo, 0: keep > 0 or lo == 0}
        for target, seen in spots.items():
            if target < 0 or target > i:
                continue
            pages = Pages([n], nkv, d, dv, seed=n + target)
            vals = torch.randn(n, nkv, dv, generator=g)
            for pos in range(n):
                k = torch.zeros(nkv, d)
                k[:, 0] = 1.0 if pos == target else 0.0
                pages.put(0, pos, k, vals[pos])
            nq = 1 if decode else min(5, n)         # the step's queries: the last positions of the sequence
            q = torch.zeros(nq, nh * d)
            q.view(nq, nh, d)[:, :, 0] = 40.0
            qstart = torch.tensor([0, nq], dtype=torch.int32, device=DEV)
            past = torch.tensor([n - nq], dtype=torch.int32, device=DEV)
            slots = torch.zeros(1, dtype=torch.int32, device=DEV)
            out = torch.full((nq, nh * dv), float("nan"), dtype=dt, device=DEV)
            status = torch.zeros(4, dtype=torch.int32, device=DEV)
            max_splits = -(-n // 64) if decode else 0
            scratch = torch.full((ops.attention_generic_scratch_floats(1, nh, dv, max(max_splits, 3)),), float("nan"), device=DEV) if decode else None
            where = (qstart, past, slots, pages.table.to(DEV), pages.n_pages, pages.k.to(DEV, dt), pages.v.to(DEV, dt))
            if kernel == "float32 arithmetic":
                ops.attention_generic_masked(decode, q.to(DEV), out, 1, nq, nh, nkv, d, dv, 1.0, *where, scratch, 64, max_splits,
                                             status, window=window, keep_first=keep)
            else:
                for split_keys, splits in ((64, max_splits), (0, 3)):       # ranges of a page; three even ranges
                    out.fill_(float("nan"))
                    ops.attention_mma_masked(decode, q.to(DEV, dt), out, 1, nq, nh, nkv, d, 1.0, *where, scratch, split_keys, splits,
                                             status, window=window, keep_first=keep)
                    if not decode:
                        break
                    if split_keys:
                        first = out.clone()
                if decode:
                    assert (out.float() - first.float()).abs().max() < 2e-2
            assert status.tolist()[0] == 0
            visible = [j for j in range(i + 1) if i - j < window or j < keep]
            assert (target in visible) == seen
            want = vals[target] if seen else vals[visible].mean(0)
            want = want.repeat_interleave(nh // nkv, dim=0).view(1, nh * dv)
            assert (out[-1:].float().cpu() - want).abs().max() < (1e-3 if dt == torch.float32 else 3e-2), (decode, window, keep, n, target, seen)


@pytest.mark.parametrize("n_state,dv", [(8, 8), (24, 20), (64, 48), (128, 64), (136, 12), (40, 100), (300, 8), (100, 260), (16, 600)])
def test_state_space_recurrence_whole_chunked_in_steps_and_on_kept_state(pe, n_state, dv):
    """Whole sequences (short: one go; long: chunks side by side) against the same sequences cut into steps of 1, 3 and many
    tokens, two sequences of unequal length on slots whose neighbours hold other state, against the plain recurrence."""
    ops = pe.kernels.ops
    heads, groups = 4, 2
    g = torch.Generator().manual_seed(n_state + dv)
    lens = [300, 41]
    ch = heads * dv + 2 * groups * n_state
    xbc = [torch.randn(n, ch, generator=g) * 0.5 for n in lens]
    dt = [torch.randn(n, heads + 3, generator=g) for n in lens]                 # the step sizes are columns 3.. of wider rows
    dt_bias, A_log, D = (torch.randn(heads, generator=g) * 0.5 for _ in range(3))
    want = []
    for x, t in zip(xbc, dt):
        step = torch.nn.functional.softplus(t[:, 3:].double() + dt_bias.double())
        y = torch.zeros(len(x), heads, dv, dtype=torch.float64)
        for h in range(heads):
            gi = h // (heads // groups)
            S = torch.zeros(n_state, dv, dtype=torch.float64)
            B = x[:, heads * dv + gi * n_state:heads * dv + (gi + 1) * n_state].double()
            C = x[:, heads * dv + (groups + gi) * n_state:heads * dv + (groups + gi + 1) * n_state].double()
            for i in range(len(x)):
                xv = x[i, h * dv:(h + 1) * dv].double()
                S = torch.exp(-torch.exp(A_log[h].double()) * step[i, h]) * S + step[i, h] * torch.outer(B[i], xv)
                y[i, h] = S.T @ C[i] + D[h].double() * xv
        want.append(y.reshape(len(x), heads * dv))
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for cuts in ([300], [1, 3, 1, 200, 95]):
        S = torch.randn(5, heads, n_state, dv, device=DEV)                      # slots 0, 2, 4 keep what they hold
        before = S.clone()
        S[3].zero_()
        S[1].zero_()
        got, at = [[], []], [0, 0]
        for step in cuts:
            live = [b for b in range(2) if at[b] < lens[b]]
            q = [min(step, lens[b] - at[b]) for b in live]
            seq, slot, qstart = _batch(q, [3 - 2 * b for b in live])
            x = torch.cat([xbc[b][at[b]:at[b] + n] for b, n in zip(live, q)]).to(DEV)
            t = torch.cat([dt[b][at[b]:at[b] + n] for b, n in zip(live, q)]).to(DEV)
            y = torch.full((sum(q), heads * dv), float("nan"), device=DEV)
            chunk, max_chunks, scratch = 0, 1, None
            if max(q) > 128:
                chunk, max_chunks = 64, -(-max(q) // 64)
                scratch = torch.full((ops.ssd_scratch_floats(len(live), heads, n_state, dv, max_chunks),), float("nan"), device=DEV)
            ops.ssd_recurrence(x, t[:, 3:], dt_bias.to(DEV), A_log.to(DEV), D.to(DEV), y, S, slot, qstart, len(live), max(q), heads,
                               groups, n_state, dv, status, chunk, max_chunks, scratch)
            for b, n, lo in zip(live, q, qstart.tolist()):
                got[b].append(y[lo:lo + n].cpu())
                at[b] += n
        for b in range(2):
            err = (torch.cat(got[b]).double() - want[b]).abs().max() / want[b].abs().max()
            assert err < 2e-5, (n_state, dv, cuts, b, float(err))
        assert torch.equal(S[[0, 2, 4]], before[[0, 2, 4]])
    assert status.tolist()[0] == 0


@pytest.mark.parametrize("taps", [1, 3])
def test_short_convolution_with_a_bias_continues_from_the_kept_inputs(pe, taps):
    ops = pe.kernels.ops
    C, lens = 24, [9, 14]
    g = torch.Generator().manual_seed(taps)
    xs = [torch.randn(n, C + 3, generator=g) for n in lens]             # the channels are columns 3.. of wider rows
    w, bias = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    want = [plain.short_conv(x[:, 3:].double(), w.double(), bias.double()) for x in xs]
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    for cuts in ([9, 14], [1, 2, 1, 5, 20]):
        tail = torch.zeros(4, max(taps - 1, 1), C, device=DEV)
        got, at = [[], []], [0, 0]
        for step in cuts:
            live = [b for b in range(2) if at[b] < lens[b]]
            q = [min(step, lens[b] - at[b]) for b in live]
            seq, slot, qstart = _batch(q, [3 - b for b in live])
            x = torch.cat([xs[b][at[b]:at[b] + n] for b, n in zip(live, q)]).to(DEV)
            out = torch.empty(sum(q), C, device=DEV)
            ops.short_conv_silu(x, 3, w.to(DEV), tail, seq, slot, qstart, out, len(live), status, bias=bias.to(DEV))
            for b, n, lo in zip(live, q, qstart.tolist()):
                got[b].append(out[lo:lo + n].cpu())
                at[b] += n
        for b in range(2):
            assert (torch.cat(got[b]).double() - want[b]).abs().max() < 1e-5, (taps, cuts, b)
    assert status.tolist()[0] == 0


def test_a_far_key_among_hundreds_through_the_rotation(pe, models):
    """A one-layer attention model whose query and key projections are made so that position 3 stands out for the last query
    of a 500-token prompt: the rotation is switched off for the features that carry the match (they lie behind ``rot.dims``),
    so the softmax must put nearly all weight on one far key, in a prompt and when the last token is decoded alone."""
    key = "far key"
    cfg = {"architecture": "Zonevik", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
           "layers": [{"type": "attention", "mixer": _att(2, 1, 16, 16, 1.0, 8, 100.0), "mlp": None}]}
    models.add(key, cfg, 77)
    w = models.w(key)
    # token 7 appears at position 3 only and token 5 as the last token only; the key projection copies feature 0 (large for
    # token 7) and the query projection feature 1 (large for token 5) into an unrotated head feature with a large factor
    w["embed"][:] = w["embed"] * 0.05
    w["embed"][7, 0] = w["embed"][5, 1] = 4.0
    for n in ("q", "k"):
        w[f"l0.mix.{n}"].zero_()
    w["l0.norm1"].fill_(1.0)
    w["l0.norm1.b"].zero_()
    w["l0.mix.q"][12, 1] = w["l0.mix.q"][28, 1] = 8.0
    w["l0.mix.k"][12, 0] = 8.0
    toks = [t if t not in (5, 7) else 8 for t in _tokens(64, 500, 5)]
    toks[3], toks[-1] = 7, 5
    for dtype in ("float32", "bfloat16"):
        eng = models.engine(key, dtype)
        s = eng.alloc_slot()
        whole = eng.step([_entry(pe, s, toks, [499])]).clone()
        eng.free_slot(s)
        s = eng.alloc_slot()
        eng.step([_entry(pe, s, toks[:499], [])])
        alone = eng.step([_entry(pe, s, toks[499:], [0])]).clone()
        eng.free_slot(s)
        models.check(key, dtype, toks, whole, [499], "far key in a prompt")
        models.check(key, dtype, toks, alone, [499], "far key decoded")
    # the case the test is for: without position 3 the logits differ
    other = list(toks)
    other[3] = 9
    assert rel_err(plain.forward(cfg, w, other)[499:].float(), models.ref(key, toks)[499:]) > 1e-2


# ---- every mechanism alone, as a model of one layer ---------------------------------------------------------------
_TINY_LEFT = _left(1, 1, 8, 8, 0.5)
_TINY_RIGHT = _right(1, 8, 8, 1, 2, 1)
ALONE = {
    "attention gated": {"type": "attention", "mixer": _att(4, 1, 24, 16, 0.5, 12, 500.0, (4.0, 32, 8.0, 1.0)), "mlp": None},
    "attention no rotation": {"type": "attention", "mixer": _att(2, 2, 16, 40, 0.25), "mlp": None},
    "attention tensor cores": {"type": "attention", "mixer": _att(8, 2, 128, 128, 0.09, 64, 10000.0, (16.0, 100, 32.0, 1.0)), "mlp": None},
    "delta": {"type": "delta", "mixer": {"heads": 6, "kv_heads": 2, "dim": 20, "vdim": 12, "conv": 4}, "mlp": None},
    "delta wide": {"type": "delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 80, "vdim": 96, "conv": 2}, "mlp": None},
    "delta widest": {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 136, "vdim": 24, "conv": 1}, "mlp": None},
    "window and state space": {"type": "parallel", "mlp": None,
                               "mixer": {"left": _left(4, 1, 24, 16, 0.5, 50, 5), "right": _right(6, 12, 20, 3, 4, 3)}},
    "no window": {"type": "parallel", "mlp": None, "mixer": {"left": _left(3, 3, 16, 16, 0.3), "right": _TINY_RIGHT}},
    "state space wide": {"type": "parallel", "mlp": None, "mixer": {"left": _TINY_LEFT, "right": _right(2, 64, 128, 2, 4, 1)}},
    "state space widest": {"type": "parallel", "mlp": None, "mixer": {"left": _TINY_LEFT, "right": _right(3, 24, 200, 1, 1, 8)}},
    "experts": {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 2}, "mlp": _moe(12, 3, 36, (4, 2))},
    "experts one group": {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 2}, "mlp": _moe(7, 2, 20, (1, 1))},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_one_mechanism_alone_whole_and_token_by_token(pe, models, name, dtype):
    key = "alone " + name
    cfg = {"architecture": "Zonevik", "vocab": 90, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "layers": [copy.deepcopy(ALONE[name])]}
    models.add(key, cfg, 40 + sorted(ALONE).index(name))
    eng = models.engine(key, dtype, max_cache_tokens=64 * 12)
    toks = _tokens(90, 150, 9)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(150))]).clone()
    eng.free_slot(s)
    models.check(key, dtype, toks, got, range(150), f"{name} whole")
    s = eng.alloc_slot()
    rows = [eng.step([_entry(pe, s, toks[:3], [2])]).clone()]
    for t in toks[3:150]:
        rows.append(eng.step([_entry(pe, s, [t], [0])]).clone())
    eng.free_slot(s)
    models.check(key, dtype, toks, torch.cat(rows), range(2, 150), f"{name} token by token")


# ---- whole models -----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C", "D"])
def test_whole_prompt_and_its_first_tokens(pe, models, key, dtype):
    eng = models.engine(key, dtype)
    toks = _tokens(CONFIGS[key]["vocab"], 300, 1)
    ref = models.ref(key, toks)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(300))]).clone()
    eng.free_slot(s)
    models.check(key, dtype, toks, got, range(300), f"{key} whole prompt")
    s = eng.alloc_slot()                               # a prompt of one token, on the slot that was just freed
    one = eng.step([_entry(pe, s, toks[:1], [0])]).clone()
    eng.free_slot(s)
    err = rel_err(one.cpu(), ref[:1])
    assert err < TOL[dtype], f"{key} one token on a used slot: {err:.3e}"
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C", "D"])
def test_long_token_by_token_decoding_equals_the_prompt(pe, models, key, dtype):
    """A short prompt, then 240 tokens one by one (past every window, over three page borders, through CUDA graphs),
    against the plain implementation of the whole sequence."""
    eng = models.engine(key, dtype)
    toks = _tokens(CONFIGS[key]["vocab"], 255, 2)
    s = eng.alloc_slot()
    rows = [eng.step([_entry(pe, s, toks[:15], [14])]).clone()]
    for t in toks[15:]:
        rows.append(eng.step([_entry(pe, s, [t], [0])]).clone())
    eng.free_slot(s)
    models.check(key, dtype, toks, torch.cat(rows), range(14, 255), f"{key} decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C"])
@pytest.mark.parametrize("portion", [2, 3, 64, 65, 131])
def test_a_prompt_fed_in_portions(pe, models, key, dtype, portion):
    eng = models.engine(key, dtype)
    toks = _tokens(CONFIGS[key]["vocab"], 280, 3)
    s = eng.alloc_slot()
    rows = []
    for lo in range(0, len(toks), portion):
        part = toks[lo:lo + portion]
        rows.append(eng.step([_entry(pe, s, part, range(len(part)))]).clone())
    eng.free_slot(s)
    models.check(key, dtype, toks, torch.cat(rows), range(len(toks)), f"{key} portions of {portion}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C", "D"])
def test_unequal_batches_on_slots_used_again(pe, models, key, dtype):
    """Two batches in a row on the same slots and pages: unequal prompts in one step (among them one token), then one
    token each until the shorter ones have ended; each request against itself alone in the plain implementation."""
    eng = models.engine(key, dtype)
    vocab = CONFIGS[key]["vocab"]
    seen = []
    for batch in range(2):
        plan = [(1, 9), (200, 4), (65, 12), (33, 1), (130, 7)]
        seqs = [_tokens(vocab, p + dec, 100 * batch + i) for i, (p, dec) in enumerate(plan)]
        slots = [eng.alloc_slot() for _ in plan]
        seen.append(sorted(slots))
        got = {}
        out = eng.step([_entry(pe, s, q[:p], [p - 1]) for s, q, (p, dec) in zip(slots, seqs, plan)])
        for i, (p, dec) in enumerate(plan):
            got[i, p - 1] = out[i].clone()
        for step in range(max(dec for _, dec in plan)):
            live = [i for i, (p, dec) in enumerate(plan) if step < dec]
            out = eng.step([_entry(pe, slots[i], [seqs[i][plan[i][0] + step]], [0]) for i in live])
            for r, i in enumerate(live):
                got[i, plan[i][0] + step] = out[r].clone()
                if step == plan[i][1] - 1:
                    eng.free_slot(slots[i])
        assert not eng.cache.live_slots
        for i, (p, dec) in enumerate(plan):
            rows = torch.stack([got[i, j] for j in range(p - 1, p + dec)])
            models.check(key, dtype, seqs[i], rows, range(p - 1, p + dec), f"{key} batch {batch} request {i}")
        eng.cache.check()
    assert seen[0] == seen[1]


def test_pages_behind_the_window_are_given_back_but_not_the_kept_ones(pe, models):
    """A sequence that decodes far past its window holds the pages of the kept first positions and of the window only."""
    eng = models.engine("B", "float32")
    toks = _tokens(256, 400, 6)
    s = eng.alloc_slot()
    free0 = eng.cache.free_pages()
    eng.step([_entry(pe, s, toks[:390], [])])
    for t in toks[390:]:
        eng.step([_entry(pe, s, [t], [0])])
    window_groups = [g for g in eng.cache.groups if g.request.kind == "kv" and g.request.window]
    assert window_groups and all(g.request.keep_first == 70 for g in window_groups)
    for g in window_groups:
        held = [i for i, p in enumerate(g.pages_of_slot[s]) if p >= 0]
        assert held == [0, 1, 4, 5, 6], held            # positions 0..69 kept; the window of 100 ends at position 399
    eng.free_slot(s)
    assert eng.cache.free_pages() == free0
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("count", [12, 40])
def test_a_decode_batch_of_many(pe, models, dtype, count):
    """More sequences than the weight-streaming products take, inside the captured decode step."""
    key = "B"
    eng = models.engine(key, dtype, max_batch=count, max_cache_tokens=64 * (count + 2))
    vocab = CONFIGS[key]["vocab"]
    seqs = [_tokens(vocab, 3 + i % 13 + 6, 300 + i) for i in range(count)]
    slots = [eng.alloc_slot() for _ in seqs]
    got = {i: [] for i in range(count)}
    out = eng.step([_entry(pe, s, q[:len(q) - 6], [len(q) - 7]) for s, q in zip(slots, seqs)]).clone()
    for i in range(count):
        got[i].append(out[i:i + 1])
    for step in range(6):
        out = eng.step([_entry(pe, s, [q[len(q) - 6 + step]], [0]) for s, q in zip(slots, seqs)]).clone()
        for i in range(count):
            got[i].append(out[i:i + 1])
    for s in slots:
        eng.free_slot(s)
    for i in (0, 5, count - 1):
        n = len(seqs[i])
        models.check(key, dtype, seqs[i], torch.cat(got[i]), range(n - 7, n), f"{key} request {i} of {count}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(pe, models, dtype):
    """``Engine.generate`` with unequal prompts: every generated token must be the plain implementation's best token
    for the sequence so far, or within rounding of it."""
    key = "A"
    eng = models.engine(key, dtype)
    prompts = [_tokens(CONFIGS[key]["vocab"], n, 50 + n) for n in (1, 17, 64, 140)]
    results = eng.generate(prompts, pe.SamplingParams.greedy_params(max_tokens=12))
    for p, r in zip(prompts, results):
        assert len(r.token_ids) == 12
        ref = models.ref(key, p + r.token_ids)
        scale = float(ref.abs().max())
        for j, tok in enumerate(r.token_ids):
            row = ref[len(p) - 1 + j]
            margin = 2 * TOL[dtype] * scale
            if dtype == "bfloat16":      # a logit moves by several times its position's root-mean-square rounding error
                noise = models.noise(key, p + r.token_ids)
                margin = 8.0 * max(float(noise[len(p) - 1 + j]), float(noise.mean()))
            assert float(row.max() - row[tok]) <= margin, (dtype, len(p), j)
    assert not eng.cache.live_slots


def test_a_model_folder_written_at_random_loads_and_runs(pe, tmp_path):
    """config.json and safetensors through the loader, against the plain implementation on the same file."""
    from safetensors.torch import load_file

    cfg = pe.ZonevikConfig.from_dict(CONFIGS["A"])
    folder = pe.write_random_model(str(tmp_path / "m"), cfg, seed=4)
    assert pe.load_config(folder) == cfg
    eng = pe.Engine(folder, dtype="float32", max_context_len=256, max_cache_tokens=512, max_batch=2)
    w = {k: v.float() for k, v in load_file(folder + "/model.safetensors").items()}
    toks = _tokens(131, 90, 8)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(90))]).clone()
    eng.free_slot(s)
    assert rel_err(got.cpu(), plain.forward(CONFIGS["A"], w, toks).float()) < TOL["float32"]
