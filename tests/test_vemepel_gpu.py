"""The Vemepel architecture on the engine against the plain implementation in ``plain_vemepel.py``: mechanisms at kernel
level with inputs made so that a fault shows, every mechanism alone as a one-layer model, then whole models: prompts,
token-by-token decoding, prompts in portions, unequal batches, slots and pages used again, long decoding, generation
through the entry point."""
import math
import random

import pytest
import torch

import plain_vemepel as plain
from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"float32": 3e-5, "bfloat16": 2e-2}
F64 = torch.float64


def _latent(heads, dim, vdim, rank, scale, rot_dim=0, dims=0, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if rot_dim:
        m.update({"rot_dim": rot_dim, "rot": {"base": base, "dims": dims}})
    return {"type": "latent_attention_2" if rot_dim else "latent_attention", "mixer": m}


def _diff(heads, kv, dim, vdim, scale, diff, size=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if size:
        m["mask"] = {"size": size}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# The tests' own models.  A: sizes that are no multiple of 8 or 32, groups of 3 and 1, a chunk that is no multiple of a
# page and a reader with another chunk, a rotated part of which only some features turn, one chosen expert and all experts
# chosen, a layer without feed-forward.  B: rounder sizes, a chunk of exactly a page, two readers of one layer's keys (one
# without a mask), rank and head sizes that differ everywhere.  C: sizes that the tensor-core attentions take in bfloat16
# (cached rows of 128, 192 and 256 features, two maps with heads of 64 in groups of 2), a differential layer first and its
# reader three layers on with another chunk.
CONFIGS = {
    "A": {"architecture": "Vemepel", "vocab": 131, "width": 72, "logit_scale": 0.7, "norm": {"eps": 2e-6},
          "layers": [
              _layer(_diff(6, 2, 20, 12, 0.22, 0.45, size=37), _moe(5, 1, 40)),
              _layer(_latent(3, 20, 28, 36, 0.2, rot_dim=12, dims=8, base=3000.0), _dense(100)),
              _layer(_diff(6, 2, 20, 12, 0.3, 0.7, size=50, kv_from=0), None),
              _layer(_latent(5, 12, 8, 24, 0.3), _moe(3, 3, 24)),
              _layer(_diff(3, 3, 8, 40, 0.35, 0.2), _dense(56))]},
    "B": {"architecture": "Vemepel", "vocab": 256, "width": 128, "logit_scale": 1.0, "norm": {"eps": 1e-5},
          "layers": [
              _layer(_latent(2, 64, 32, 96, 0.1, rot_dim=32, dims=32, base=100000.0), _moe(8, 2, 64)),
              _layer(_diff(4, 1, 32, 64, 0.18, 0.5, size=64), _dense(256)),
              _layer(_diff(4, 1, 32, 64, 0.15, 0.6, size=64, kv_from=1), _moe(4, 2, 96)),
              _layer(_latent(4, 32, 32, 64, 0.17), _dense(192)),
              _layer(_diff(4, 1, 32, 64, 0.2, 0.35, kv_from=1), None)]},
    "C": {"architecture": "Vemepel", "vocab": 200, "width": 96, "logit_scale": 0.5, "norm": {"eps": 1e-5},
          "layers": [
              _layer(_diff(4, 2, 64, 64, 0.125, 0.55, size=96), _dense(160)),
              _layer(_latent(3, 32, 48, 128, 0.15), _moe(6, 2, 48)),
              _layer(_latent(2, 24, 40, 128, 0.16, rot_dim=64, dims=64, base=2000.0), None),
              _layer(_diff(4, 2, 64, 64, 0.11, 0.3, size=40, kv_from=0), _moe(4, 1, 64)),
              _layer(_latent(5, 16, 16, 256, 0.2), _dense(120))]},
}
SEEDS = {"A": 31, "B": 32, "C": 33}


def _tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def _bf16_values(w):
    """Weights as a checkpoint holds them: rounded to bfloat16, so that a bfloat16 engine and the oracle start equal."""
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


def _entry(pe, slot, toks, want):
    return pe.StepEntry(slot, toks, tuple(want))


class Models:
    def __init__(self, pe):
        self.pe = pe
        self.configs = dict(CONFIGS)
        self.seeds = dict(SEEDS)
        self.weights = {}
        self.engines = {}
        self.refs = {}

    def add(self, key, cfg, seed):
        self.configs[key] = cfg
        self.seeds[key] = seed

    def w(self, key):
        if key not in self.weights:
            self.weights[key] = _bf16_values(plain.random_weights(self.configs[key], self.seeds[key]))
        return self.weights[key]

    def engine(self, key, dtype, **kw):
        ident = (key, dtype, tuple(sorted(kw.items())))
        if ident not in self.engines:
            cfg = self.pe.VemepelConfig.from_dict(self.configs[key])
            args = dict(dtype=dtype, max_context_len=1024, max_cache_tokens=64 * 40, max_batch=8)
            args.update(kw)
            self.engines[ident] = self.pe.Engine(None, config=cfg, weights={k: v.to(DEV) for k, v in self.w(key).items()}, **args)
        return self.engines[ident]

    def ref(self, key, toks):
        ident = (key, tuple(toks))
        if ident not in self.refs:
            self.refs[ident] = plain.forward(self.configs[key], self.w(key), toks).float()
        return self.refs[ident]

    def noise(self, key, toks):
        """How far rounding to bfloat16 alone moves each position's logits (root mean square over the vocabulary)."""
        ident = (key, tuple(toks), "noise")
        if ident not in self.refs:
            rounded = plain.forward(self.configs[key], self.w(key), toks, stored=plain.bf16)
            self.refs[ident] = (rounded - self.ref(key, toks).double()).pow(2).mean(dim=1).sqrt()
        return self.refs[ident]

    def check(self, key, dtype, toks, got, positions, what):
        """float32: every logit within 3e-5 of the largest.  bfloat16: the error is held against what rounding alone does
        in the plain implementation: at no more than one position in fifty (or one) above three times the larger of that
        position's own figure and the average, and over the other positions on average no more than twice that."""
        positions = list(positions)
        ref = self.ref(key, toks)[positions]
        got = got.float().cpu()
        assert got.shape == ref.shape, what
        if dtype == "float32":
            err = float((got.double() - ref.double()).abs().max() / ref.double().abs().max())
            assert err < TOL[dtype], f"{what}: error {err:.3e} (limit {TOL[dtype]:.0e})"
            return
        noise = self.noise(key, toks)
        err = (got.double() - ref.double()).pow(2).mean(dim=1).sqrt()
        floor = float(noise.mean())
        allowed = max(1, len(positions) // 50)
        over = err > 3.0 * torch.clamp(noise[positions], min=floor)
        assert int(over.sum()) <= allowed, f"{what}: {int(over.sum())} of {len(positions)} positions beyond three times rounding"
        # the mean is taken over the positions within that bound: a router's close call that rounding turns moves one
        # position's logits by far more than rounding does elsewhere
        rest = err[~over] if int((~over).sum()) else err
        assert float(rest.mean()) <= 2.0 * max(float(noise[positions].mean()), floor), \
            f"{what}: mean error {float(rest.mean()):.3e}, rounding alone {float(noise[positions].mean()):.3e}"


@pytest.fixture(scope="module")
def models(pe):
    return Models(pe)


@pytest.fixture(scope="module")
def ops(pe):
    return pe.kernels.ops


def _status():
    return torch.zeros(4, dtype=torch.int32, device=DEV)


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ---- mechanisms at kernel level ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [72, 256, 1030, 1028, 2052, 5000, 8192, 8196])
def test_norm_and_token_shift_with_kept_rows(ops, dtype, width):
    """Three sequences in one step (a continuing one, a new one, a single token) on slots that hold other rows; then a
    second step that continues all three: the kept row must be the unmoved last row, zeros for a new sequence."""
    g = torch.Generator().manual_seed(width)
    w = (1.0 + 0.3 * torch.randn(width, generator=g)).to(DEV)
    mix = torch.rand(width, generator=g).to(DEV)
    eps = 1e-5
    n_slots = 5
    state = torch.randn(n_slots, width, generator=g).to(DEV)
    slots = [3, 0, 4]
    state[0].zero_()                                        # the new sequence's slot as the cache hands it out
    kept = {s: state[s].double().cpu() for s in slots}
    for q_lens in ([4, 7, 1], [1, 2, 33]):
        n = sum(q_lens)
        x = (3.0 * torch.randn(n, width, generator=g)).to(DEV)
        qstart = [0]
        for q in q_lens:
            qstart.append(qstart[-1] + q)
        token_seq = _i32(sum(([b] * q for b, q in enumerate(q_lens)), []))
        out = torch.empty(n, width, dtype=dtype, device=DEV)
        untouched = state[[1, 2]].clone()
        st = _status()
        ops.norm_token_shift(x, w, eps, mix, state, token_seq, _i32(slots), _i32(qstart), out, st)
        assert st.tolist()[0] == 0
        for b, s in enumerate(slots):
            rows = x[qstart[b]:qstart[b + 1]].double().cpu()
            h = plain.norm_plain(rows, w.double().cpu(), eps)
            want, last = plain.token_shift(h, kept[s], mix.double().cpu())
            kept[s] = last
            tol = 1e-5 if dtype == torch.float32 else 1e-2
            assert rel_err(out[qstart[b]:qstart[b + 1]].cpu(), want) < tol
            assert rel_err(state[s].cpu(), last) < 1e-5
        assert torch.equal(state[[1, 2]], untouched)


def test_depth_average_adds_the_terms_it_is_given(ops):
    g = torch.Generator().manual_seed(5)
    results = torch.randn(6, 33, 72, generator=g).to(DEV)
    coeff = torch.randn(6, generator=g).to(DEV)
    for terms in (2, 5, 6):
        out = torch.zeros(33, 72, device=DEV)
        copy = torch.zeros(33, 72, device=DEV)
        ops.depth_average(results, coeff, terms, out, copy)
        want = plain.depth_average(list(results[:terms].double().cpu()), coeff[:terms].double().cpu())
        assert rel_err(out.cpu(), want) < 1e-6 and torch.equal(out, copy)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [19, 400])
@pytest.mark.parametrize("width", [40, 320, 2050, 4104, 5000, 11000, 40000])
def test_polynorm(ops, dtype, width, rows):
    g = torch.Generator().manual_seed(width)
    z = (2.0 * torch.randn(rows, width, generator=g)).to(dtype).to(DEV)
    coeff = torch.tensor([0.9, -0.4, 0.25, 0.3], device=DEV)
    out = torch.empty_like(z)
    ops.polynorm(z, coeff, 1e-5, out)
    want = plain.polynorm(z.double().cpu(), coeff.cpu(), 1e-5)
    assert rel_err(out.cpu(), want) < (1e-5 if dtype == torch.float32 else 1e-2)


def test_router_by_logits_ties_bias_and_all_experts(ops):
    """The bias moves a choice; equal logits go to the lower index; with ``top`` equal to the number of outputs every
    expert is chosen and the weights are the softmax over all."""
    g = torch.Generator().manual_seed(2)
    for n_all, top in ((5, 1), (16, 4), (3, 3), (70, 6)):
        z = torch.randn(41, n_all, generator=g)
        z[3] = 0.25                                           # all equal: the first `top` indices
        z[4, :] = torch.tensor([1.0] * n_all)
        z[5] = z[5].round()                                   # many ties
        bias = torch.randn(n_all, generator=g)
        bias[n_all - 1] += 3.0                                # the last expert wins often through its bias alone
        zb = (z + bias).to(DEV) - bias.to(DEV)                # what the kernel will add the bias to, in float32
        chosen = torch.zeros(41, top, dtype=torch.int32, device=DEV)
        weight = torch.zeros(41, top, device=DEV)
        ops.moe_route_logits(zb.contiguous(), bias.to(DEV), top, chosen, weight)
        total = (zb + bias.to(DEV)).double().cpu()
        order = torch.sort(total, dim=-1, descending=True, stable=True).indices[:, :top]
        assert torch.equal(chosen.cpu().long(), order)
        want = torch.softmax(torch.gather(total, 1, order), -1)
        assert rel_err(weight.cpu(), want) < 1e-5
        assert top == n_all or int((chosen.cpu() == n_all - 1).sum()) > 41 * top // n_all


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sigmoid_gates_a_head_and_a_feature(ops, dtype):
    g = torch.Generator().manual_seed(12)
    heads, n, dv = 3, 17, 10
    x = torch.randn(heads, n, dv, generator=g).to(dtype).to(DEV)
    wide = torch.randn(n, heads * dv + heads + 7, generator=g).to(dtype).to(DEV)        # gates as columns of a wider row
    xd = x.double().cpu().transpose(0, 1)
    for gate in (wide[:, 2:2 + heads], wide[:, 5:5 + heads * dv]):
        out = torch.zeros(n, heads * dv, dtype=dtype, device=DEV)
        ops.sigmoid_gate(x, gate, out)
        s = torch.sigmoid(gate.double().cpu())
        want = xd * (s[:, :, None] if gate.shape[1] == heads else s.view(n, heads, dv))
        assert rel_err(out.cpu().view(n, heads, dv), want) < (1e-6 if dtype == torch.float32 else 1e-2)
        packed = x.transpose(0, 1).contiguous()                                        # the same heads as packed rows
        out2 = torch.zeros_like(out)
        ops.sigmoid_gate(packed.transpose(0, 1), gate, out2)
        assert torch.equal(out, out2)


def test_the_difference_of_two_maps(ops):
    g = torch.Generator().manual_seed(9)
    for heads, dv, lam, post in ((3, 12, 0.7, 0.55), (4, 96, -0.2, 0.4), (1, 130, 1.3, 1.0)):
        a = torch.randn(21, 2 * heads * dv, generator=g).to(DEV)
        for dtype in (torch.float32, torch.bfloat16):
            out = torch.empty(21, heads * dv, dtype=dtype, device=DEV)
            ops.diff_combine(a, out, heads, dv, lam, 1e-6, post)
            x = a.double().cpu().view(21, 2, heads, dv)
            want = plain.unit_rms(x[:, 0] - lam * x[:, 1], 1e-6) * post
            assert rel_err(out.cpu().view(21, heads, dv), want) < (1e-5 if dtype == torch.float32 else 1e-2)


class Paged:
    """Sequences whose rows lie scattered over shuffled pages of a pool that holds junk elsewhere."""

    def __init__(self, lens, heads, dim, dtype, seed=0):
        self.lens = lens
        rng = random.Random(seed)
        per = [(n + 63) // 64 for n in lens]
        self.num_pages = sum(per) + 4
        order = list(range(self.num_pages))
        rng.shuffle(order)
        self.slots = list(range(len(lens) - 1, -1, -1))
        self.table = torch.full((len(lens) + 1, max(per) + 1), -1, dtype=torch.int32)
        it = iter(order)
        for b, p in enumerate(per):
            for lp in range(p):
                self.table[self.slots[b], lp] = next(it)
        g = torch.Generator().manual_seed(seed)
        self.pages = (50.0 * torch.randn(self.num_pages, heads, 64, dim, generator=g)).to(dtype).to(DEV)
        self.table = self.table.to(DEV)
        self.seq_slot = _i32(self.slots)

    def put(self, b, rows):
        """rows [len, heads, dim] of sequence b into its pages."""
        for lp in range((rows.shape[0] + 63) // 64):
            page = int(self.table[self.slots[b], lp])
            n = min(64, rows.shape[0] - lp * 64)
            self.pages[page, :, :n] = rows[lp * 64: lp * 64 + n].transpose(0, 1).to(self.pages.dtype).to(DEV)


def _attend(ops, decode, q, out, lens, q_lens, nh, nkv, d, dv, scale, kp, vp, table, seq_slot, **kw):
    qstart = [0]
    for n in q_lens:
        qstart.append(qstart[-1] + n)
    past = [L - n for L, n in zip(lens, q_lens)]
    st = _status()
    scratch, splits = None, 0
    if decode:
        splits = -(-max(lens) // 512)
        scratch = torch.zeros(ops.attention_generic_scratch_floats(len(lens), nh, dv, splits), device=DEV)
    ops.attention_generic_masked(decode, q, out, len(lens), max(q_lens), nh, nkv, d, dv, scale, _i32(qstart), _i32(past),
                                 seq_slot, table, kp.shape[0], kp, vp, scratch, 512, splits, st, **kw)
    assert st.tolist()[0] == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk", [37, 64, 130])
def test_chunk_mask_edges_in_prompts_and_decoding(ops, dtype, chunk):
    """Every key scores zero except one that matches the query strongly.  Placed at the first position of the query's
    own block it must take all the weight; one position earlier (the last of the block before) it must not be seen.  The
    queries sit at a block's first, second and last position and right behind a page border, in a prompt and decoding."""
    d, dv, nh, nkv = 16, 24, 2, 1
    length = 3 * chunk + 70
    probes = sorted({chunk, chunk + 1, 2 * chunk - 1, 2 * chunk, 3 * chunk + 5, 128, 129, 191, 192, length - 1})
    for qpos in probes:
        start = qpos // chunk * chunk
        for key_at, seen in ((start, True), (start - 1, False)):
            if key_at < 0:
                continue
            for decode in (False, True):
                k = torch.zeros(qpos + 1, nkv, d)
                k[key_at, 0, 0] = 30.0
                g = torch.Generator().manual_seed(qpos)
                v = torch.randn(qpos + 1, nkv, dv, generator=g)
                kp = Paged([qpos + 1], nkv, d, dtype, seed=1)
                vp = Paged([qpos + 1], nkv, dv, dtype, seed=1)
                kp.put(0, k)
                vp.put(0, v)
                q_len = 1 if decode else min(qpos + 1, 9)
                q = torch.zeros(q_len, nh * d)
                q[-1, 0] = 1.0
                q[-1, d] = 1.0
                out = torch.zeros(q_len, nh * dv, dtype=dtype, device=DEV)
                _attend(ops, decode, q.to(dtype).to(DEV), out, [qpos + 1], [q_len], nh, nkv, d, dv, 1.0, kp.pages, vp.pages,
                        kp.table, kp.seq_slot, chunk=chunk)
                vq = v.to(dtype).double()
                want = vq[key_at, 0] if seen else vq[start:qpos + 1, 0].mean(0)
                got = out[-1].double().cpu().view(nh, dv)
                for h in range(nh):
                    assert (got[h] - want).abs().max() < 2e-2, (chunk, qpos, key_at, decode)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_values_inside_the_key_rows_and_a_far_key(ops, dtype):
    """One kv head whose values are the leading features of its key rows (a latent cache), eleven query heads, random
    rows; and a key 700 positions back that one head matches: against the plain softmax, in prompts and decoding, with a
    float32 output too."""
    row, r, nh = 56, 40, 11
    lens, q_lens = [900, 65, 300], [130, 65, 1]
    g = torch.Generator().manual_seed(4)
    pg = Paged(lens, 1, row, dtype, seed=2)
    rows = [torch.randn(n, 1, row, generator=g) for n in lens]
    rows[0][200, 0, r:] = 0.0
    rows[0][200, 0, 45] = 12.0                             # a feature beyond the value part: only the score sees it
    for b in range(3):
        pg.put(b, rows[b])
    for decode, ql in ((False, q_lens), (True, [1, 1, 1])):
        n = sum(ql)
        q = torch.randn(n, nh * row, generator=g) * 0.5
        q[ql[0] - 1, 3 * row:4 * row] = 0.0
        q[ql[0] - 1, 3 * row + 45] = 5.0                     # head 3 of the first sequence's last query looks far back
        for out_dtype in (dtype, torch.float32):
            out = torch.zeros(n, nh * r, dtype=out_dtype, device=DEV)
            _attend(ops, decode, q.to(dtype).to(DEV), out, lens, ql, nh, 1, row, r, 0.3, pg.pages, pg.pages, pg.table,
                    pg.seq_slot, v_ld=row)
            at = 0
            for b, (L, m) in enumerate(zip(lens, ql)):
                keys = rows[b][:, 0].to(dtype).double()
                pos = torch.arange(L - m, L)
                visible = torch.arange(L)[None, :] <= pos[:, None]
                for h in range(nh):
                    qh = q[at:at + m, h * row:(h + 1) * row].to(dtype).double()
                    want = plain.softmax_attend(qh, keys, keys[:, :r], 0.3, visible)
                    got = out[at:at + m, h * r:(h + 1) * r].double().cpu()
                    assert (got - want).abs().max() < (1e-4 if dtype == torch.float32 else 3e-2), (decode, b, h)
                at += m
            far = out[ql[0] - 1, 3 * r:4 * r].double().cpu()
            assert (far - rows[0][200, 0, :r].to(dtype).double()).abs().max() < 3e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_key_maps_over_one_set_of_values(ops, dtype):
    """Four key heads over two value heads: key head g reads value head g % 2."""
    nh, nkv, nv, d, dv = 8, 4, 2, 12, 20
    lens, q_lens = [150, 70], [150, 3]
    g = torch.Generator().manual_seed(8)
    kp, vp = Paged(lens, nkv, d, dtype, seed=3), Paged(lens, nv, dv, dtype, seed=3)
    ks = [torch.randn(n, nkv, d, generator=g) for n in lens]
    vs = [torch.randn(n, nv, dv, generator=g) for n in lens]
    for b in range(2):
        kp.put(b, ks[b])
        vp.put(b, vs[b])
    n = sum(q_lens)
    q = torch.randn(n, nh * d, generator=g)
    out = torch.zeros(n, nh * dv, device=DEV)
    _attend(ops, False, q.to(dtype).to(DEV), out, lens, q_lens, nh, nkv, d, dv, 0.4, kp.pages, vp.pages, kp.table, kp.seq_slot,
            v_heads=nv)
    at = 0
    for b, (L, m) in enumerate(zip(lens, q_lens)):
        pos = torch.arange(L - m, L)
        visible = torch.arange(L)[None, :] <= pos[:, None]
        for h in range(nh):
            kv = h // (nh // nkv)
            want = plain.softmax_attend(q[at:at + m, h * d:(h + 1) * d].to(dtype).double(), ks[b][:, kv].to(dtype).double(),
                                        vs[b][:, kv % nv].to(dtype).double(), 0.4, visible)
            assert (out[at:at + m, h * dv:(h + 1) * dv].double().cpu() - want).abs().max() < 1e-4
        at += m


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("c0,dk,dv", [(7, 12, 20), (8, 16, 24)])
def test_keys_and_values_into_their_pages_at_once(ops, dtype, c0, dk, dv):
    """Two column ranges of the step's rows into two pools with the same page numbers: what two single copies write, and
    the rows themselves."""
    lens, q_lens = [70, 130, 5], [9, 130, 1]
    nk, nv = 4, 2
    g = torch.Generator().manual_seed(11)
    n = sum(q_lens)
    x = torch.randn(n, c0 + nk * dk + nv * dv, generator=g).to(dtype).to(DEV)
    pos = _i32(sum(([L - m + j for j in range(m)] for L, m in zip(lens, q_lens)), []))
    token_seq = _i32(sum(([b] * m for b, m in enumerate(q_lens)), []))
    single_k, single_v = Paged(lens, nk, dk, dtype, seed=9), Paged(lens, nv, dv, dtype, seed=9)
    both_k, both_v = Paged(lens, nk, dk, dtype, seed=9), Paged(lens, nv, dv, dtype, seed=9)
    st = _status()
    where = (token_seq, pos, single_k.seq_slot, single_k.table, single_k.num_pages)
    ops.rows_to_pages(x, c0, nk, dk, *where, single_k.pages, st)
    ops.rows_to_pages(x, c0 + nk * dk, nv, dv, *where, single_v.pages, st)
    ops.rows_to_pages_pair(x, c0, nk, dk, both_k.pages, c0 + nk * dk, nv, dv, both_v.pages, *where, st)
    assert st.tolist()[0] == 0
    assert torch.equal(single_k.pages, both_k.pages) and torch.equal(single_v.pages, both_v.pages)
    page = int(single_k.table[single_k.slots[1], 1])
    assert torch.equal(both_v.pages[page, 1, 3], x[9 + 64 + 3, c0 + nk * dk + dv:c0 + nk * dk + 2 * dv])
    assert torch.equal(both_k.pages[page, 2, 65 - 64], x[9 + 65, c0 + 2 * dk:c0 + 3 * dk])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rot", [0, 6, 10])
@pytest.mark.parametrize("dr", [10, 16])
def test_latent_rows_and_turned_queries(ops, dtype, rot, dr):
    """The cached row [normed low-rank part | turned shared key part] and the turned part of the queries, for tokens at
    positions around a page border, on pages handed out in shuffled order."""
    nh, d, r = 3, 8, 24
    lens, q_lens = [70, 130], [9, 130]
    pg = Paged(lens, 1, r + dr, dtype, seed=6)
    g = torch.Generator().manual_seed(rot)
    n = sum(q_lens)
    cols = nh * (d + dr) + r + dr + 5
    x = torch.randn(n, cols, generator=g).to(dtype)
    norm_w = 1.0 + 0.3 * torch.randn(r, generator=g)
    base = 500.0
    cos = sin = None
    if rot:
        i = torch.arange(rot // 2, dtype=F64)
        ang = torch.arange(256, dtype=F64)[:, None] * base ** (-2.0 * i / rot)
        cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    pos = torch.tensor(sum(([L - m + j for j in range(m)] for L, m in zip(lens, q_lens)), []))
    token_seq = _i32(sum(([b] * m for b, m in enumerate(q_lens)), []))
    qfull = torch.zeros(n, nh, r + dr, dtype=dtype, device=DEV)
    st = _status()
    ops.latent_prepare(x.to(DEV), 0, nh * (d + dr), nh, d, dr, r, norm_w.to(DEV), 1e-5, cos, sin, rot, token_seq,
                       pos.to(torch.int32).to(DEV), pg.seq_slot, pg.table, pg.num_pages, pg.pages, qfull, True, st)
    assert st.tolist()[0] == 0
    xd = x.double()
    low = xd[:, nh * (d + dr):nh * (d + dr) + r + dr]
    c = plain.norm_plain(low[:, :r], norm_w.double(), 1e-5)
    kr = plain.rotate_pairs(low[:, r:], pos, base, rot) if rot else low[:, r:]
    qr = xd[:, :nh * (d + dr)].view(n, nh, d + dr)[:, :, d:]
    qr = plain.rotate_pairs(qr, pos, base, rot) if rot else qr
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert rel_err(qfull[:, :, r:].cpu(), qr) < tol
    assert float(qfull[:, :, :r].abs().max()) == 0.0              # no absorbed queries were given: left as it was
    absorbed = torch.randn(nh, n, r, generator=g).to(dtype).to(DEV)
    ops.latent_prepare(x.to(DEV), 0, nh * (d + dr), nh, d, dr, r, norm_w.to(DEV), 1e-5, cos, sin, rot, token_seq,
                       pos.to(torch.int32).to(DEV), pg.seq_slot, pg.table, pg.num_pages, pg.pages, qfull, False, st,
                       absorbed=absorbed)
    assert torch.equal(qfull[:, :, :r], absorbed.transpose(0, 1)) and rel_err(qfull[:, :, r:].cpu(), qr) < tol
    at = 0
    for b, (L, m) in enumerate(zip(lens, q_lens)):
        for j in range(m):
            p = L - m + j
            page = int(pg.table[pg.slots[b], p // 64])
            got = pg.pages[page, 0, p % 64].double().cpu()
            assert rel_err(got[:r], c[at + j]) < tol and rel_err(got[r:], kr[at + j]) < tol
        at += m


def _starts_and_pasts(lens, q_lens):
    qstart = [0]
    for n in q_lens:
        qstart.append(qstart[-1] + n)
    return _i32(qstart), _i32([L - n for L, n in zip(lens, q_lens)])


@pytest.mark.parametrize("row,r,nh", [(128, 128, 5), (192, 128, 16), (320, 256, 20), (576, 512, 3), (576, 512, 33)])
def test_cached_rows_on_the_tensor_cores(ops, row, r, nh):
    """The tensor-core kernels over cached rows whose leading features are the values: prompts that start at a page's
    border, in its middle and at position 0, one token, and decoding with more heads than one block takes; one head looks
    700 positions back.  Against the plain softmax on the same bfloat16 inputs."""
    dtype = torch.bfloat16
    assert ops.attention_latent_supported(dtype, row, r)
    lens, q_lens = [900, 65, 300, 192], [130, 65, 1, 64]
    g = torch.Generator().manual_seed(row + nh)
    pg = Paged(lens, 1, row, dtype, seed=2)
    rows = [torch.randn(n, 1, row, generator=g) for n in lens]
    mark = row - 3 if row > r else 7
    rows[0][200, 0] = 0.0
    rows[0][200, 0, mark] = 12.0
    for b in range(len(lens)):
        pg.put(b, rows[b])
    scale = 1.5 / math.sqrt(row)
    look = min(3, nh - 1)
    for decode, ql in ((False, q_lens), (True, [1] * len(lens))):
        n = sum(ql)
        q = torch.randn(n, nh * row, generator=g)
        q[ql[0] - 1, look * row:(look + 1) * row] = 0.0
        q[ql[0] - 1, look * row + mark] = 32.0                # its score stands far above the random ones
        out = torch.zeros(n, nh * r, dtype=dtype, device=DEV)
        qstart, past = _starts_and_pasts(lens, ql)
        st = _status()
        scratch, split_keys, splits, floor = None, 0, 0, 0
        if decode:
            split_keys, splits, floor = ops.attention_latent_decode_ranges(torch.device(DEV), len(lens), nh, max(lens), 128)
            scratch = torch.zeros(ops.attention_generic_scratch_floats(len(lens), nh, r, splits), device=DEV)
        ops.attention_latent(decode, q.to(dtype).to(DEV), out, len(lens), max(ql), nh, row, r, scale, qstart, past, pg.seq_slot,
                             pg.table, pg.num_pages, pg.pages.view(pg.num_pages, 1, 64, row), scratch, split_keys, splits, st,
                             min_range_keys=floor)
        assert st.tolist()[0] == 0
        at = 0
        for b, (L, m) in enumerate(zip(lens, ql)):
            keys = rows[b][:, 0].to(dtype).double()
            pos = torch.arange(L - m, L)
            visible = torch.arange(L)[None, :] <= pos[:, None]
            for h in range(nh):
                qh = q[at:at + m, h * row:(h + 1) * row].to(dtype).double()
                want = plain.softmax_attend(qh, keys, keys[:, :r], scale, visible)
                got = out[at:at + m, h * r:(h + 1) * r].double().cpu()
                assert (got - want).abs().max() < 2e-2, (decode, b, h, float((got - want).abs().max()))
            at += m
        far = out[ql[0] - 1, look * r:(look + 1) * r].double().cpu()
        assert (far - rows[0][200, 0, :r].to(dtype).double()).abs().max() < 7e-2   # bfloat16 steps of 1/16 at 12


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("chunk", [0, 37, 64, 130])
def test_two_key_maps_and_chunks_on_the_tensor_cores(ops, d, chunk):
    """The tensor-core kernels with twice the key heads over one set of value heads, the chunk mask and a float32
    output, weights in two bfloat16 terms: prompts that start inside a chunk, one token, decoding.  Against the plain
    softmax on the same bfloat16 inputs; the weights' second term shows in the tolerance."""
    dtype = torch.bfloat16
    nh, nkv, nv = 12, 4, 2
    assert ops.attention_mma_supported(dtype, d, nh, nkv)
    lens, q_lens = [700, 65, 300, 131], [135, 65, 1, 2]
    g = torch.Generator().manual_seed(d + chunk)
    kp, vp = Paged(lens, nkv, d, dtype, seed=3), Paged(lens, nv, d, dtype, seed=3)
    ks = [torch.randn(n, nkv, d, generator=g) for n in lens]
    vs = [torch.randn(n, nv, d, generator=g) for n in lens]
    for b in range(len(lens)):
        kp.put(b, ks[b])
        vp.put(b, vs[b])
    scale = 1.5 / math.sqrt(d)
    for decode, ql in ((False, q_lens), (True, [1] * len(lens))):
        n = sum(ql)
        q = torch.randn(n, nh * d, generator=g)
        for split_p, tol in ((True, 2e-4), (False, 2e-2)):
            out = torch.zeros(n, nh * d, device=DEV)
            qstart, past = _starts_and_pasts(lens, ql)
            st = _status()
            scratch, split_keys, splits, floor = None, 512, 0, 0
            if decode:
                split_keys, splits, floor = ops.attention_mma_decode_ranges(torch.device(DEV), d, len(lens), nkv, max(lens), 512)
                scratch = torch.zeros(ops.attention_generic_scratch_floats(len(lens), nh, d, splits), device=DEV)
            ops.attention_mma_masked(decode, q.to(dtype).to(DEV), out, len(lens), max(ql), nh, nkv, d, scale, qstart, past,
                                     kp.seq_slot, kp.table, kp.num_pages, kp.pages, vp.pages, scratch, split_keys, splits, st,
                                     min_range_keys=floor, chunk=chunk, v_heads=nv, split_p=split_p)
            assert st.tolist()[0] == 0
            at = 0
            for b, (L, m) in enumerate(zip(lens, ql)):
                pos = torch.arange(L - m, L)
                j = torch.arange(L)
                visible = j[None, :] <= pos[:, None]
                if chunk:
                    visible &= (j[None, :] // chunk) == (pos[:, None] // chunk)
                for h in range(nh):
                    kv = h // (nh // nkv)
                    want = plain.softmax_attend(q[at:at + m, h * d:(h + 1) * d].to(dtype).double(),
                                                ks[b][:, kv].to(dtype).double(), vs[b][:, kv % nv].to(dtype).double(), scale, visible)
                    err = float((out[at:at + m, h * d:(h + 1) * d].double().cpu() - want).abs().max())
                    assert err < tol, (decode, split_p, b, h, err)
                at += m


@pytest.mark.parametrize("chunk", [37, 64, 130])
def test_chunk_edges_on_the_tensor_cores(ops, chunk):
    """One key matches the query strongly: at the first position of the query's own block it takes all the weight, one
    position earlier it is not seen.  Queries at a block's first, second and last position and around page borders."""
    dtype = torch.bfloat16
    d, nh, nkv = 64, 2, 1
    length = 3 * chunk + 70
    for qpos in sorted({chunk, chunk + 1, 2 * chunk - 1, 2 * chunk, 3 * chunk + 5, 128, 129, 191, 192, length - 1}):
        start = qpos // chunk * chunk
        for key_at, seen in ((start, True), (start - 1, False)):
            if key_at < 0:
                continue
            for decode in (False, True):
                k = torch.zeros(qpos + 1, nkv, d)
                k[key_at, 0, 0] = 30.0
                g = torch.Generator().manual_seed(qpos)
                v = torch.randn(qpos + 1, nkv, d, generator=g)
                kp, vp = Paged([qpos + 1], nkv, d, dtype, seed=1), Paged([qpos + 1], nkv, d, dtype, seed=1)
                kp.put(0, k)
                vp.put(0, v)
                q_len = 1 if decode else min(qpos + 1, 9)
                q = torch.zeros(q_len, nh * d)
                q[-1, 0] = 1.0
                q[-1, d] = 1.0
                out = torch.zeros(q_len, nh * d, device=DEV)
                qstart, past = _starts_and_pasts([qpos + 1], [q_len])
                st = _status()
                scratch, split_keys, splits, floor = None, 512, 0, 0
                if decode:
                    split_keys, splits, floor = ops.attention_mma_decode_ranges(torch.device(DEV), d, 1, nkv, qpos + 1, 512)
                    scratch = torch.zeros(ops.attention_generic_scratch_floats(1, nh, d, splits), device=DEV)
                ops.attention_mma_masked(decode, q.to(dtype).to(DEV), out, 1, q_len, nh, nkv, d, 1.0, qstart, past, kp.seq_slot,
                                         kp.table, kp.num_pages, kp.pages, vp.pages, scratch, split_keys, splits, st,
                                         min_range_keys=floor, chunk=chunk, split_p=True)
                assert st.tolist()[0] == 0
                vq = v.to(dtype).double()
                want = vq[key_at, 0] if seen else vq[start:qpos + 1, 0].mean(0)
                got = out[-1].double().cpu().view(nh, d)
                for h in range(nh):
                    assert (got[h] - want).abs().max() < 1e-3, (chunk, qpos, key_at, decode)


# ---- every mechanism alone, as a model of one layer ---------------------------------------------------------------
ONE_LAYER = {
    "latent, one gate a head": _layer(_latent(3, 20, 28, 36, 0.2), None),
    "latent, one head": _layer(_latent(1, 40, 12, 16, 0.15), None),
    "latent with a turned part": _layer(_latent(2, 16, 16, 40, 0.2, rot_dim=16, dims=16, base=50.0), None),
    "latent, part of the turned part turns": _layer(_latent(4, 8, 24, 136, 0.25, rot_dim=20, dims=4, base=1e6), None),
    "two maps, chunk 33, groups of 3": _layer(_diff(6, 2, 24, 8, 0.2, 0.5, size=33), None),
    "two maps, no mask, one kv head": _layer(_diff(4, 1, 8, 72, 0.4, 0.8), None),
    "two maps, chunk of two pages": _layer(_diff(2, 2, 40, 40, 0.15, 0.1, size=128), None),
    "latent, rows the tensor cores take": _layer(_latent(2, 16, 24, 128, 0.2), None),
    "latent with a turned part, rows the tensor cores take": _layer(_latent(3, 16, 16, 128, 0.2, rot_dim=64, dims=64, base=300.0),
                                                                   None),
    "two maps, chunk 33, heads the tensor cores take": _layer(_diff(4, 2, 64, 64, 0.12, 0.5, size=33), None),
    "latent, rows of 512 + 64": _layer(_latent(2, 128, 128, 512, 0.07, rot_dim=64, dims=64, base=1e4), None),
    "two maps, chunk 100, heads of 128": _layer(_diff(4, 2, 128, 128, 0.09, 0.4, size=100), None),
    "dense": _layer(_diff(1, 1, 8, 8, 0.3, 0.5), _dense(90)),
    "one expert of seven": _layer(_latent(1, 8, 8, 8, 0.3), _moe(7, 1, 24)),
    "every expert": _layer(_latent(1, 8, 8, 8, 0.3), _moe(4, 4, 40)),
    "three of twenty": _layer(_latent(1, 8, 8, 8, 0.3), _moe(20, 3, 16)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_each_mechanism_alone_whole_and_token_by_token(pe, models, name, dtype):
    key = "one:" + name
    models.add(key, {"architecture": "Vemepel", "vocab": 97, "width": 48, "logit_scale": 1.3, "norm": {"eps": 1e-5},
                     "layers": [ONE_LAYER[name]]}, 50 + sorted(ONE_LAYER).index(name))
    eng = models.engine(key, dtype)
    toks = _tokens(97, 150, 7)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(150))]).clone()
    eng.free_slot(s)
    models.check(key, dtype, toks, got, range(150), f"{name} whole")
    s = eng.alloc_slot()
    rows = [eng.step([_entry(pe, s, toks[:3], [2])]).clone()]
    for t in toks[3:]:
        rows.append(eng.step([_entry(pe, s, [t], [0])]).clone())
    eng.free_slot(s)
    models.check(key, dtype, toks, torch.cat(rows), range(2, 150), f"{name} token by token")


# ---- whole models -----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_whole_prompt_and_its_first_tokens(pe, models, key, dtype):
    eng = models.engine(key, dtype)
    toks = _tokens(CONFIGS[key]["vocab"], 300, 1)
    ref = models.ref(key, toks)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(300))]).clone()
    eng.free_slot(s)
    models.check(key, dtype, toks, got, range(300), f"{key} whole prompt")
    for first in (1, 2):                               # prompts of one and two tokens, on the slot that was just freed
        s = eng.alloc_slot()
        one = eng.step([_entry(pe, s, toks[:first], range(first))]).clone()
        eng.free_slot(s)
        err = rel_err(one.cpu(), ref[:first])
        assert err < TOL[dtype], f"{key} {first} token(s) on a used slot: {err:.3e}"
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_long_token_by_token_decoding_equals_the_prompt(pe, models, key, dtype):
    """A short prompt, then 240 tokens one by one (over every chunk's edge, over three page borders, through CUDA
    graphs), against the plain implementation of the whole sequence."""
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
@pytest.mark.parametrize("portion", [2, 3, 37, 64, 65, 131])
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
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B", "C"])
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_decode_batch_of_twelve(pe, models, dtype):
    """More sequences than the weight-streaming products take, inside the captured decode step."""
    key = "B"
    eng = models.engine(key, dtype, max_batch=16, max_cache_tokens=64 * 64)
    vocab = CONFIGS[key]["vocab"]
    seqs = [_tokens(vocab, 20 + 11 * i + 6, 300 + i) for i in range(12)]
    slots = [eng.alloc_slot() for _ in seqs]
    got = {i: [] for i in range(12)}
    out = eng.step([_entry(pe, s, q[:len(q) - 6], [len(q) - 7]) for s, q in zip(slots, seqs)]).clone()
    for i in range(12):
        got[i].append(out[i])
    for step in range(6):
        out = eng.step([_entry(pe, s, [q[len(q) - 6 + step]], [0]) for s, q in zip(slots, seqs)]).clone()
        for i in range(12):
            got[i].append(out[i])
    for s in slots:
        eng.free_slot(s)
    for i, q in enumerate(seqs):
        models.check(key, dtype, q, torch.stack(got[i]), range(len(q) - 7, len(q)), f"request {i} among twelve")


def test_pages_behind_a_chunk_are_given_back(pe, models):
    """A model whose only paged layer has a chunk mask gives the pages of finished blocks back while it decodes."""
    key = "chunked layer alone"
    models.add(key, {"architecture": "Vemepel", "vocab": 97, "width": 48, "logit_scale": 1.3, "norm": {"eps": 1e-5},
                     "layers": [ONE_LAYER["two maps, chunk of two pages"]]}, 77)
    eng = models.engine(key, "float32", max_cache_tokens=64 * 6)
    toks = _tokens(97, 400, 11)
    s = eng.alloc_slot()
    rows = [eng.step([_entry(pe, s, toks[:300], range(300))]).clone()]       # five pages at once, more than stay
    assert eng.cache.free_pages() >= 6 - 1
    for t in toks[300:]:
        rows.append(eng.step([_entry(pe, s, [t], [0])]).clone())
        assert eng.cache.free_pages() >= 6 - 2
    eng.free_slot(s)
    eng.cache.check()
    models.check(key, "float32", toks, torch.cat(rows), range(400), "chunked layer with pages given back")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(pe, models, dtype):
    """``Engine.generate`` (scheduler, sampler, CUDA graphs) with unequal prompts: every generated token must be the
    plain implementation's best token for the sequence so far, or within rounding of it."""
    key = "A"
    eng = models.engine(key, dtype)
    vocab = CONFIGS[key]["vocab"]
    prompts = [_tokens(vocab, n, 500 + n) for n in (1, 40, 75)]
    results = eng.generate(prompts, pe.SamplingParams.greedy_params(max_tokens=12))
    for p, r in zip(prompts, results):
        assert len(r.token_ids) == 12
        ref = models.ref(key, p + list(r.token_ids))
        scale = float(ref.abs().max())
        for j, tok in enumerate(r.token_ids):
            row = ref[len(p) - 1 + j]
            margin = 2 * TOL[dtype] * scale
            if dtype == "bfloat16":      # a logit moves by several times its position's root-mean-square rounding error
                noise = models.noise(key, p + list(r.token_ids))
                margin = 8.0 * max(float(noise[len(p) - 1 + j]), float(noise.mean()))
            assert float(row.max() - row[tok]) <= margin, (dtype, len(p), j)
    assert not eng.cache.live_slots


def test_a_model_folder_written_at_random_loads_and_runs(pe, tmp_path):
    """The preset through the random-weights writer, the loader and the engine, against the plain implementation on the
    tensors that were written."""
    from safetensors.torch import load_file
    cfg = pe.preset("vemepel_tiny")
    folder = str(tmp_path / "model")
    pe.write_random_model(folder, cfg, 5)
    assert pe.load_config(folder) == cfg
    w = {k: v.float() for k, v in load_file(f"{folder}/model.safetensors").items()}
    assert set(w) == set(plain.tensor_shapes(cfg.to_dict())) and all(tuple(w[k].shape) == s for k, s in plain.tensor_shapes(cfg.to_dict()).items())
    eng = pe.Engine(folder, dtype="float32", max_context_len=512, max_cache_tokens=64 * 16, max_batch=4)
    toks = _tokens(cfg.vocab, 120, 3)
    s = eng.alloc_slot()
    got = eng.step([_entry(pe, s, toks, range(120))]).clone()
    eng.free_slot(s)
    ref = plain.forward(cfg.to_dict(), w, toks)
    assert rel_err(got.cpu(), ref) < TOL["float32"]
