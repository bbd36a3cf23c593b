"""Vunelix through the engine against the plain implementation (tests/plain_vunelix.py): each mechanism alone, whole
models of several sizes and layer orders, prompts cut in every way, batches, reused pages and state slots, far keys and
page borders, long decoding, and greedy generation through the scheduler."""
import json
import math
import os

import numpy as np
import pytest
import torch

from conftest import random_tokens
import plain_vunelix as plain
from trace_helpers import by_position, mixed, portions, staggered_plan, tail_decode, whole

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# bfloat16: the deepest model here runs eight layers with sixteen norms on sublayers' outputs; its rows differ from the
# float64 model by 2 to 4 per cent of the logits' spread in the median (as the bfloat16 engine differs from the float32 one)
TOL = {"float32": 3e-5, "bfloat16": 5e-2}
F = torch.float64


def latent(heads, dim, rot_dim, vdim, rank, scale, rot_dims=None, base=1e4, scaling=None, mlp=None):
    rot = {"base": base, "dims": rot_dims if rot_dims is not None else rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale, "rot": rot}}


def scan(inner, state, dt_rank, conv, mlp=None):
    return {"type": "mamba1", "mlp": mlp, "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def config(width, vocab, layers, loop=None, cap=None, eps=1e-5):
    out = {"architecture": "Vunelix", "norm": {"eps": eps}, "vocab": vocab, "width": width, "layers": layers, "logit_softcap": cap}
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# Sizes that differ from one another in everything: plain, rotated and value sizes that are unequal, rotation of a part
# and of the whole rotated part, with and without stretched frequencies, one expert a row and several (and all of them),
# with and without a shared expert, layers without feed-forward, a span of layers run twice or three times that starts at
# the first layer or later and ends at the last or earlier, states that are no multiple of the scan's lanes.
MODELS = {
    "latent": config(64, 97, [latent(3, 24, 8, 16, 40, 0.3, mlp=dense(72))], cap=20.0),
    "scan": config(48, 83, [scan(80, 5, 3, 3)], eps=1e-6),
    "moe": config(64, 101, [latent(2, 16, 16, 24, 24, 0.25, rot_dims=8, scaling=(4.0, 64, 8.0, 2.0), mlp=moe(5, 2, 40, shared=24)),
                            scan(96, 16, 4, 2, mlp=moe(3, 3, 24))], cap=15.0),
    "looped": config(96, 211, [scan(128, 9, 5, 4, mlp=dense(80)), latent(4, 12, 12, 20, 48, 0.3, scaling=(8.0, 32, 16.0, 1.0), mlp=moe(6, 2, 32, shared=48)),
                               latent(2, 32, 4, 8, 16, 0.2, base=500.0), scan(64, 24, 2, 3, mlp=moe(4, 1, 56))], loop=(1, 3, 3), cap=12.0),
    "loop-all": config(64, 130, [latent(2, 8, 24, 32, 72, 0.35, rot_dims=12, mlp=dense(40)), scan(72, 12, 6, 4, mlp=moe(2, 2, 48, shared=16))],
                       loop=(0, 2, 2), eps=3e-6),
    "loop-tail": config(80, 77, [latent(5, 16, 8, 16, 32, 0.3, mlp=moe(7, 3, 24)), scan(40, 40, 1, 5, mlp=dense(56)),
                                 latent(1, 48, 16, 40, 136, 0.2, scaling=(2.0, 128, 4.0, 0.5), mlp=dense(64))], loop=(1, 3, 2), cap=30.0),
    # nothing a multiple of anything: odd width, odd sizes everywhere, a prime vocabulary
    "awkward": config(50, 61, [latent(3, 5, 6, 7, 9, 0.4, rot_dims=4, base=777.0, mlp=moe(2, 1, 11, shared=13)), scan(37, 3, 2, 5, mlp=dense(21)),
                               latent(1, 9, 2, 3, 5, 0.5)], loop=(0, 1, 3), cap=9.0),
}
STD = 0.16     # matrices N(0, STD): products keep their input's spread, so scores, gates and routers are far from flat


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from infinicore_infer_b200.config import config_class_for
    from infinicore_infer_b200.weights import index_directory, read_tensor, write_model_folder
    out = {}
    for seed, (name, cfg) in enumerate(MODELS.items()):
        d = str(tmp_path_factory.mktemp("vunelix_" + name))
        write_model_folder(config_class_for(cfg).from_dict(cfg), d, seed=seed + 31, std=STD, norm_std=0.2)
        with open(os.path.join(d, "config.json")) as f:
            disk = json.load(f)
        out[name] = (d, disk, {n: read_tensor(i).float() for n, i in index_directory(d).items()})
    return out


@pytest.fixture(scope="module")
def engines(folders):
    from infinicore_infer_b200.engine import Engine
    cache = {}

    def get(name, dtype, cache_tokens=512, max_requests=3, **kw):
        key = (name, dtype, cache_tokens, max_requests, tuple(sorted(kw.items())))
        if key not in cache:
            cache[key] = Engine.from_folder(folders[name][0], dtype=DTYPES[dtype], max_tokens=512, cache_tokens=cache_tokens,
                                            page_size=16, max_requests=max_requests, max_step_tokens=512, **kw)
        return cache[key]
    return get


_plain = {}
# A row whose router leaves the last chosen expert this close (in the router's output) to the first one left out may go to
# another expert once the activations are rounded to bfloat16: such a row's logits are those of another, equally valid,
# choice, and are not compared.  (float32 reproduces every choice.)
CLOSE_CALL = {"float32": 1e-4, "bfloat16": 0.08}


class Expected(np.ndarray):
    """Logits [T, vocab] with ``margin`` [T]: the smallest router margin of each row over the model's routed layers."""


def expected(folders, name, seed, n):
    key = (name, seed, n)
    if key not in _plain:
        _, cfg, w = folders[name]
        toks = random_tokens(seed, n, cfg["vocab"])
        margins = []
        want = plain.forward(toks, cfg, w, margins=margins).numpy().view(Expected)
        want.margin = torch.stack(margins).min(0).values.numpy() if margins else np.full(n, np.inf)
        _plain[key] = (toks, want)
    return _plain[key]


def run(engine, steps):
    from infinicore_infer_b200.trace import replay
    return by_position(steps, replay(engine, steps))


def check(got, rid, want, tol, what):
    """float32: every logit of every position within ``tol`` of the logits' scale: the sharp test.  bfloat16: the difference
    of a position's logits (its mean taken off, root mean square over the vocabulary) against the spread of the logits.  A
    norm on a sublayer's output brings a row whose output is small up to the size of the others, its rounding error with it,
    so single rows lie far off while a fault of the cache or the state moves most rows: half the rows must lie within
    ``tol``, nine in ten within three times it, all within half the logits' spread.  Rows whose router call is close are left
    out (``CLOSE_CALL``)."""
    loose = tol > 1e-3
    margin = getattr(want, "margin", np.full(len(want), np.inf))
    sure = margin >= CLOSE_CALL["bfloat16" if loose else "float32"]
    assert len(want) < 20 or sure.sum() >= 0.5 * len(want), f"{what}: the router is sure of {int(sure.sum())} of {len(want)} rows only"
    want = np.asarray(want, dtype=np.float64)
    diff = np.stack([got[(rid, p)].astype(np.float64) - want[p] for p in range(len(want))])
    if not loose:
        errs, scale = np.abs(diff).max(1) * sure, np.abs(want).max()
        worst = int(errs.argmax())
        assert errs.max() <= tol * scale, f"{what}: request {rid} position {worst}: error {errs.max():.3e} > {tol * scale:.3e}"
        return
    scale = (want - want.mean(1, keepdims=True)).std()
    errs = ((diff - diff.mean(1, keepdims=True)).std(1) / scale)[sure]
    if not len(errs):
        return
    assert np.median(errs) <= tol, f"{what}: request {rid}: the median row differs by {np.median(errs):.3f} of the logits' spread"
    assert (errs > 3 * tol).sum() <= max(1, len(errs) // 10), f"{what}: request {rid}: {(errs > 3 * tol).sum()} of {len(errs)} rows beyond {3 * tol}"
    assert errs.max() <= 0.5, f"{what}: request {rid}: a row differs by {errs.max():.3f} of the logits' spread"


# ---- whole models ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", list(MODELS))
def test_whole_tail_and_portions_agree_with_the_plain_implementation(folders, engines, name, dtype):
    eng = engines(name, dtype)
    for i, n in enumerate((1, 37, 150)):
        toks, want = expected(folders, name, 300 + i, n)
        for what, steps in (("whole", whole("r", toks)), ("tail", tail_decode("r", toks, tail=20)),
                            ("portions", portions("r", toks)), ("pairs", portions("r", toks, sizes=(2,))),
                            ("uneven", portions("r", toks, sizes=(17, 3, 31, 2, 16)))):
            check(run(eng, steps), "r", want, TOL[dtype], f"{name} {dtype} {what} n={n}")
        eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_every_token_decoded_alone_through_graphs(folders, engines, dtype):
    """Long decoding: every token a step of its own (captured steps), so pages, tails and states move one position at a
    time, and from 256 positions on the keys of a row are cut into ranges."""
    for name in ("looped", "loop-tail", "moe"):
        toks, want = expected(folders, name, 77, 300)
        eng = engines(name, dtype)
        before = eng.steps_run
        check(run(eng, tail_decode("r", toks, tail=len(toks))), "r", want, TOL[dtype], f"{name} {dtype} token by token")
        assert eng.steps_run - before >= 300


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", ["looped", "loop-all", "awkward"])
def test_batches_of_unequal_requests_in_a_small_pool(folders, name, dtype):
    """Up to three live requests, portions beside single tokens; the pool holds three requests, so the pages and state
    slots of finished requests are the next ones handed out.  Every row equals the request run alone."""
    from infinicore_infer_b200.engine import Engine
    lengths = [70, 9, 33, 50, 2, 41, 64]
    reqs, wants = {}, {}
    for i, n in enumerate(lengths):
        toks, want = expected(folders, name, 500 + i, n)
        reqs[f"q{i}"], wants[f"q{i}"] = toks, want
    steps = mixed(reqs, staggered_plan(reqs, live=3, portion=6, tail=5))
    eng = Engine.from_folder(folders[name][0], dtype=DTYPES[dtype], max_tokens=128, cache_tokens=3 * 80, page_size=16,
                             max_requests=3, max_step_tokens=128)
    got = run(eng, steps)
    for rid, want in wants.items():
        check(got, rid, want, TOL[dtype], f"{name} {dtype} mixed")
    eng.cache.check_invariants()
    assert eng.cache.slots.available == 3 and all(g.pool.in_use == 0 for g in eng.cache.groups)


def test_a_reused_slot_starts_from_zero_state(folders, engines):
    """The same request twice in a row lands in the slot (and pages) that its first run left."""
    toks, want = expected(folders, "looped", 9, 45)
    eng = engines("looped", "float32", max_requests=1)
    check(run(eng, whole("r", toks)), "r", want, TOL["float32"], "first run")
    check(run(eng, portions("r", toks, sizes=(5, 2))), "r", want, TOL["float32"], "second run in the same slot")


def test_passes_of_a_span_keep_caches_and_states_apart(folders):
    from infinicore_infer_b200.config import read_config
    from infinicore_infer_b200.parts import cache_needs, state_needs
    spec = read_config(folders["looped"][0], max_tokens=64).model_spec()
    assert [e.layer for e in spec.order] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [e.cache for e in spec.order] == list(range(8)) and all(e.writes_cache for e in spec.order)
    assert [e.before.step_index if e.before else None for e in spec.order] == [None, 0, None, 1, None, 2, None, None]
    needs, tails = cache_needs(spec), state_needs(spec)
    assert needs[0].shape == (128, 9) and tails[0].shape == (3, 128) and needs[7].shape == (64, 24) and tails[1] is None
    assert needs[1].head_dim == 48 + 12 and needs[1].v_head_dim == 48 and needs[1].values_in_keys and needs[2].head_dim == 16 + 4


# ---- mechanisms alone -------------------------------------------------------------------------------------------------------
def scrambled_pages(rows, page, dev, dtype, spare=2):
    """Rows [T, D] of one request into pages handed out in a scrambled order; (pages, table [1, blocks])."""
    T, D = rows.shape
    blocks = (T + page - 1) // page
    order = torch.randperm(blocks + spare, generator=torch.Generator().manual_seed(3))[:blocks] + 1
    pages = torch.zeros(blocks + spare + 1, 1, page, D, dtype=dtype, device=dev)
    for t in range(T):
        pages[order[t // page], 0, t % page] = rows[t].to(dtype)
    return pages, order.to(torch.int32).view(1, -1).to(dev)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,R,dr,page", [(3, 40, 8, 8), (9, 128, 32, 16), (1, 5, 2, 4), (2, 260, 0, 16)])
def test_latent_attention_finds_one_far_key_at_any_place(dtype, H, R, dr, page):
    """Among hundreds of cached rows one far row gets a score that stands out, for queries in a prompt and for a single
    decoded row, with the far row at a page's first place, its last place, at position 0 and right before the query;
    whole keys and keys cut into ranges agree.  float32 runs on the CUDA cores, bfloat16 on the tensor cores."""
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    g = torch.Generator().manual_seed(H + R)
    T, D = 333, R + dr
    rows = 0.3 * torch.randn(T, D, generator=g, dtype=F)
    q = torch.randn(T, H, D, generator=g, dtype=F)
    far = {T - 1: 0, T - 2: page - 1, T - 3: page, T - 4: T - 5, 100: 2 * page - 1, 17: 16, 5: 5}
    for i, j in far.items():                      # head 0 of row i looks for row j
        q[i, 0] = 25.0 * rows[j] / (rows[j] @ rows[j])
    if dt == torch.bfloat16:
        rows, q = rows.to(dt).double(), q.to(dt).double()
    scores = torch.einsum("thd,sd->hts", q, rows)
    causal = torch.arange(T).view(1, T, 1) >= torch.arange(T).view(1, 1, T)
    want = torch.einsum("hts,sd->thd", torch.softmax(scores.masked_fill(~causal, -math.inf), -1), rows[:, :R])
    pages, table = scrambled_pages(rows, page, dev, dt)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    tol = 2e-5 if dt == torch.float32 else 2e-2
    for splits in (1, 3, 7):
        out = torch.empty(T, H, R, dtype=dt, device=dev)
        starts = torch.tensor([0, T], dtype=torch.int32, device=dev)
        K.latent_attention(q.to(dt).to(dev).contiguous(), pages, out, pos, torch.zeros_like(pos), table, H, R, dr, 1.0, splits=splits, req_start=starts)
        err = (out.double().cpu() - want).abs().max().item()
        assert err <= tol * want.abs().max().item(), f"prompt rows, {splits} ranges: {err}"
        for i in far:                             # the same rows one by one, as a decode step sees them
            one = torch.empty(1, H, R, dtype=dt, device=dev)
            K.latent_attention(q[i:i + 1].to(dt).to(dev).contiguous(), pages, one, pos[i:i + 1], torch.zeros(1, dtype=torch.int32, device=dev),
                               table, H, R, dr, 1.0, splits=splits, req_start=torch.tensor([0, 1], dtype=torch.int32, device=dev))
            assert (one.double().cpu()[0] - want[i]).abs().max().item() <= tol * want.abs().max().item(), f"decoded row {i}, {splits} ranges"
    for i, j in far.items() if D >= 40 else ():   # the far row decides head 0's output
        assert (want[i, 0] - rows[j, :R]).abs().max() < 0.05 * rows[j, :R].abs().max() + 0.02


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_queries_and_cache_rows_of_the_latent_attention(dtype):
    """Two requests side by side at unequal positions in scrambled pages: plain query parts, rotated parts behind the
    latent part's room, normed latent vectors and rotated shared key parts in the pages, with stretched frequencies and a
    rotation of fewer elements than the rotated part has."""
    from infinicore_infer_b200 import kernels as K
    from infinicore_infer_b200.config import FrequencyRampSpec, PairRotarySpec
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    H, dn, dr, R, dims, page, eps = 3, 10, 12, 14, 8, 8, 1e-4
    scaling = {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 1.0}
    spec = PairRotarySpec(dims=dims, base=300.0, scaling=FrequencyRampSpec(4.0, 32.0, 4.0, 1.0))
    f, mag = spec.frequencies()
    pf, pm = plain.rotary_frequencies(dims, 300.0, scaling)
    assert np.allclose(f, pf.numpy(), rtol=1e-12) and abs(mag - pm) < 1e-12 and abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-12
    assert f[0] == 1.0 and abs(f[-1] - 300.0 ** (-6 / 8) / 4.0) < 1e-12          # the fastest pair keeps its frequency, the slowest is stretched
    g = torch.Generator().manual_seed(2)
    starts, n = (3, 41), 30
    ld = H * (dn + dr) + R + dr + 5
    q_off, kv_off = 2, 2 + H * (dn + dr)
    u = torch.randn(2 * n, ld, generator=g, dtype=F)
    w = 1 + 0.3 * torch.randn(R, generator=g, dtype=F)
    pos = torch.cat([torch.arange(s, s + n) for s in starts])
    blocks = (max(starts) + n + page - 1) // page
    table = torch.tensor([[2 * b + 2 for b in range(blocks)], [2 * b + 1 for b in range(blocks)]], dtype=torch.int32, device=dev)
    pages = torch.zeros(2 * blocks + 1, 1, page, R + dr, dtype=dt, device=dev)
    q_plain = torch.empty(2 * n, H * dn, dtype=dt, device=dev)
    q_full = torch.zeros(2 * n, H, R + dr, dtype=dt, device=dev)
    K.latent_qkv(u.float().to(dev), q_off, kv_off, H, dn, dr, R, dims, torch.tensor(f, dtype=torch.float32, device=dev), mag,
                 w.float().to(dev), eps, pos.to(torch.int32).to(dev), torch.tensor([0] * n + [1] * n, dtype=torch.int32, device=dev), table,
                 page, q_plain, q_full, pages)
    uf = u.float().double()
    q = uf[:, q_off:q_off + H * (dn + dr)].view(2 * n, H, dn + dr)
    tol = 2e-5 if dt == torch.float32 else 2e-2
    assert (q_plain.double().cpu().view(2 * n, H, dn) - q[..., :dn]).abs().max() < tol * q.abs().max()
    assert (q_full.double().cpu()[..., R:] - plain.rotate_pairs(q[..., dn:], pos, pf, pm)).abs().max() < tol * q.abs().max()
    assert torch.all(q_full[..., :R] == 0)
    c = plain.rms_norm(uf[:, kv_off:kv_off + R], w, eps)
    kr = plain.rotate_pairs(uf[:, kv_off + R:kv_off + R + dr], pos, pf, pm)
    for r in range(2 * n):
        row = pages[table[r // n, pos[r] // page].item(), 0, pos[r] % page].double().cpu()
        assert (row[:R] - c[r]).abs().max() < tol * c.abs().max() and (row[R:] - kr[r]).abs().max() < tol * kr.abs().max(), f"cache row of row {r}"


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,n,k", [(3, 40, 24), (1, 7, 130), (5, 65, 5), (2, 128, 64)])
def test_products_per_head_with_and_without_a_gate(H, n, k, dtype):
    """float32 on the CUDA cores, bfloat16 on the tensor cores; sizes that are no multiple of a tile, of eight or of two."""
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    g = torch.Generator().manual_seed(n)
    tol = 1e-5 if dt == torch.float32 else 1e-2
    for T in (1, 70, 133):
        x = torch.randn(T, H, k, generator=g).to(dt).double()
        w = torch.randn(H, n, k, generator=g).to(dt).double()
        gate = torch.randn(T, H * n + 3, generator=g, dtype=F)
        want = torch.einsum("thk,hnk->thn", x, w)
        out = torch.zeros(T, H, n + 2, dtype=dt, device=dev)
        K.head_linear(x.to(dt).to(dev), w.to(dt).to(dev), out, n + 2)
        assert (out[..., :n].double().cpu() - want).abs().max() < tol * want.abs().max() and torch.all(out[..., n:] == 0)
        gated = torch.empty(T, H, n, dtype=dt, device=dev)
        K.head_linear(x.to(dt).to(dev), w.to(dt).to(dev), gated, n, gate=gate.float().to(dev), gate_ld=H * n + 3)
        want_g = want * torch.sigmoid(gate.float().double()[:, :H * n]).view(T, H, n)
        assert (gated.double().cpu() - want_g).abs().max() < tol * want.abs().max()


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("E,N,K_,J", [(80, 5, 3, 3), (37, 22, 11, 4), (8, 70, 1, 2), (130, 16, 9, 1), (96, 16, 40, 3)])
def test_convolution_and_scan_carry_their_state_across_cuts_and_slots(E, N, K_, J, dtype):
    """Two sequences cut into portions (down to one row, shorter and longer than the taps) that go through state slots
    side by side; an early input is made large and its channel's decay slow, so that a lost state or a wrong decay moves
    late outputs.  The state, the step sizes and the sums are float32 in both modes; bfloat16 rounds the output and has the
    step sizes' weights as a 16-bit checkpoint stores them (their product then runs on the tensor cores, unrounded rows)."""
    from infinicore_infer_b200 import kernels as K
    dev, dt_ = torch.device("cuda:0"), DTYPES[dtype]
    g = torch.Generator().manual_seed(E)
    T = 150
    ld = 2 * E + 3
    us = [torch.randn(T, ld, generator=g, dtype=F) for _ in range(2)]
    us[0][1, :E] *= 8.0
    taps, bias = torch.randn(E, J, generator=g, dtype=F) * 0.5, 0.1 * torch.randn(E, generator=g, dtype=F)
    w_x = torch.randn(K_ + 2 * N, E, generator=g, dtype=F) * E ** -0.5
    w_dt, b_dt = (torch.randn(E, K_, generator=g) * 0.5).to(torch.bfloat16).double(), torch.randn(E, generator=g, dtype=F) - 2.0
    a_log, skip = torch.randn(E, N, generator=g, dtype=F) - 2.0, torch.randn(E, generator=g, dtype=F)

    def plain_y(u):
        x = plain.silu(plain.causal_conv(u[:, :E], taps, bias))
        low = x @ w_x.T
        dt = torch.nn.functional.softplus(low[:, :K_] @ w_dt.T + b_dt)
        return plain.selective_scan(x, dt, -torch.exp(a_log), low[:, K_:K_ + N], low[:, K_ + N:], skip) * plain.silu(u[:, E:2 * E])

    want = [plain_y(u.float().double()) for u in us]
    state = torch.zeros(4, E, N, dtype=torch.float32, device=dev)
    tail = torch.zeros(4, max(J - 1, 1), E, dtype=torch.float32, device=dev)
    state[0] = 7.0                               # slot 0 is nobody's; what lies there must not matter
    slots = torch.tensor([3, 1], dtype=torch.int32, device=dev)
    A = (-torch.exp(a_log)).float().to(dev)
    got = [[], []]
    cuts = [0, 1, 2, 3, 5, 40, 41, 120, T]
    for a, b in zip(cuts, cuts[1:]):
        n = b - a
        rows = torch.cat([us[0][a:b], us[1][a:b]]).float().to(dev)
        req_start = torch.tensor([0, n, 2 * n], dtype=torch.int32, device=dev)
        row_req = torch.tensor([0] * n + [1] * n, dtype=torch.int32, device=dev)
        x32 = torch.empty(2 * n, E, dtype=torch.float32, device=dev)
        K.causal_conv(rows, 0, E, taps.float().to(dev), bias.float().to(dev), K.ACT_SILU, tail if J > 1 else None, row_req, req_start, slots, x32, None)
        low = (x32.double().cpu() @ w_x.T).float().to(dev)          # the small projection, here on the host
        out = torch.empty(2 * n, E, dtype=dt_, device=dev)
        K.selective_scan(x32, low, K_, N, rows[:, E:], ld, w_dt.to(dt_).to(dev), b_dt.float().to(dev), A, skip.float().to(dev), state,
                         req_start, slots, out, dt_buf=torch.empty(2 * n, E, dtype=torch.float32, device=dev) if a % 2 else None)
        got[0].append(out[:n].float().cpu()); got[1].append(out[n:].float().cpu())
    for i in range(2):
        err = (torch.cat(got[i]).double() - want[i]).abs().max().item() / want[i].abs().max().item()
        assert err < (3e-5 if dt_ == torch.float32 else 6e-3), f"sequence {i}: relative error {err}"
    assert torch.all(state[0] == 7.0) and torch.all(state[2] == 0.0)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("experts,top,ff,shared", [(5, 2, 40, True), (3, 3, 24, False), (9, 1, 88, True), (70, 4, 9, False)])
def test_routed_experts_choose_scale_and_add_up(dtype, experts, top, ff, shared):
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    g = torch.Generator().manual_seed(experts)
    d = 48
    for T in (1, 5, 200):
        h = torch.randn(T, d, generator=g, dtype=F)
        if dt == torch.bfloat16:
            h = h.to(dt).double()
        W = {"router": torch.randn(experts, d, generator=g, dtype=F)}
        for e in range(experts):            # matrices as a 16-bit checkpoint holds them
            W[f"e{e}.gate"] = (torch.randn(ff, d, generator=g) * d ** -0.5).to(torch.bfloat16).double()
            W[f"e{e}.up"] = (torch.randn(ff, d, generator=g) * d ** -0.5).to(torch.bfloat16).double()
            W[f"e{e}.down"] = (torch.randn(d, ff, generator=g) * ff ** -0.5).to(torch.bfloat16).double()
        base = torch.randn(T, d, generator=g, dtype=F) if shared else torch.zeros(T, d, dtype=F)
        want = base + plain.routed_ff(h, {"router": {"experts": experts, "top": top}}, W, "")
        delta = base.float().to(dev) if shared else torch.full((T, d), 9.0, dtype=torch.float32, device=dev)
        w_gu = torch.cat([W[f"e{e}.{n}"] for e in range(experts) for n in ("gate", "up")]).to(dt).to(dev).contiguous()
        w_dn = torch.cat([W[f"e{e}.down"] for e in range(experts)]).to(dt).to(dev).contiguous()
        K.routed_experts(h.to(dt).to(dev).contiguous(), W["router"].float().to(dev), w_gu, w_dn, delta, shared, experts, top, K.ACT_SILU)
        err = (delta.double().cpu() - want).abs().max().item()
        assert err <= (3e-5 if dt == torch.float32 else 2e-2) * max(want.abs().max().item(), 1.0), f"{T} rows: {err}"


def test_norm_that_adds_and_norms_again_relu_unit_and_cap():
    from infinicore_infer_b200 import kernels as K
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(4)
    for d in (5, 96, 1000):
        x = torch.randn(7, d, generator=g, dtype=F) * 3 + 1.5
        delta = torch.randn(7, d, generator=g, dtype=F) * 2 - 4
        w, w2 = torch.randn(d, generator=g, dtype=F), torch.randn(d, generator=g, dtype=F)
        want = x + plain.rms_norm(delta, w, 1e-5)
        xs = x.float().to(dev)
        K.norm_add(delta.float().to(dev), xs, w.float().to(dev), 1e-5)
        assert (xs.double().cpu() - want).abs().max() < 1e-5 * want.abs().max()
        xs, h = x.float().to(dev), torch.empty(7, d, dtype=torch.float32, device=dev)
        K.norm_add(delta.float().to(dev), xs, w.float().to(dev), 1e-5, next_weight=w2.float().to(dev), next_eps=1e-3, out=h)
        want_h = plain.rms_norm(want, w2, 1e-3)
        assert (xs.double().cpu() - want).abs().max() < 1e-5 * want.abs().max() and (h.double().cpu() - want_h).abs().max() < 1e-5 * want_h.abs().max()
        hb = torch.empty(7, d, dtype=torch.bfloat16, device=dev)
        xs = x.float().to(dev)
        K.norm_add(delta.float().to(dev), xs, w.float().to(dev), 1e-5, out=hb)
        assert torch.equal(hb, xs.to(torch.bfloat16))
        gu = torch.randn(7, 2 * d, generator=g, dtype=F) * 2
        out = torch.empty(7, d, dtype=torch.float32, device=dev)
        K.glu(gu.float().to(dev), out, K.ACT_RELU)
        assert (out.double().cpu() - torch.relu(gu[:, :d]) * gu[:, d:]).abs().max() < 1e-5
        z = (torch.randn(7, d, generator=g, dtype=F) * 30).float().to(dev)
        want_z = 11.0 * torch.tanh(z.double().cpu() / 11.0)
        assert (K.softcap(z, 11.0).double().cpu() - want_z).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_the_relu_unit_in_the_fused_products_of_few_and_many_rows(folders, engines, dtype):
    """The dense feed-forward's gate/up product takes another kernel for few rows, many rows and float32; all of them
    apply relu."""
    eng = engines("latent", dtype)
    for n in (3, 40, 300):
        toks, want = expected(folders, "latent", 40 + n, n)
        check(run(eng, whole("r", toks)), "r", want, TOL[dtype], f"relu unit, {n} rows")


# ---- generation through the scheduler ---------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler_matches_the_plain_model(folders):
    """Requests of unequal length through ``Generator`` (admission, portions of 16 tokens, decoding beside prompts, three
    slots for five requests): every generated token is the plain model's argmax given the tokens before it."""
    from infinicore_infer_b200.engine import Engine, Generator
    d, cfg, w = folders["looped"]
    eng = Engine.from_folder(d, dtype=torch.float32, max_tokens=160, cache_tokens=3 * 96, page_size=16, max_requests=3, max_step_tokens=64)
    gen = Generator(eng, chunk_size=16)
    prompts = [random_tokens(900 + i, n, cfg["vocab"]) for i, n in enumerate((40, 3, 25, 61, 12))]
    outs = gen.generate(prompts, max_new_tokens=12)
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        logits = plain.forward(p + o, cfg, w).numpy()
        for j, tok in enumerate(o):
            row = logits[len(p) + j - 1]
            best = int(row.argmax())
            assert tok == best or row[best] - row[tok] < 1e-4 * np.abs(row).max(), f"token {j} of a prompt of {len(p)}"
    eng.cache.check_invariants()


def test_command_line_runs_a_small_model_with_random_weights(tmp_path):
    """``--random vunelix-tiny`` with three prompts through the scheduler, greedy: the printed tokens are the plain model's."""
    import re
    import subprocess
    import sys
    from infinicore_infer_b200.config import PRESETS, VunelixConfig
    from infinicore_infer_b200.weights import index_directory, read_tensor, write_model_folder
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    preset = PRESETS["vunelix-tiny"]
    proc = subprocess.run([sys.executable, "-m", "infinicore_infer_b200.jiuge", "--nvidia", "--random", "vunelix-tiny", "--seed", "3",
                           "--prompt-lens", "2,19,40", "--chunk-size", "11", "--num-pages", "24", "--max-batch", "3",
                           "--max-tokens-per-step", "24", "--temperature", "0", "--max-steps", "8", "--dtype", "float32"],
                          capture_output=True, text=True, cwd=root, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = {int(m.group(1)): [int(t) for t in m.group(2).split()] for m in re.finditer(r"request (\d+): ([\d ]*)", proc.stdout)}
    assert sorted(got) == [0, 1, 2]
    cfg = VunelixConfig.from_dict(preset.config)
    write_model_folder(cfg, str(tmp_path), seed=3, std=preset.std, norm_std=preset.norm_std)
    w = {n: read_tensor(i).float() for n, i in index_directory(str(tmp_path)).items()}
    for k, n in enumerate((2, 19, 40)):
        prompt = torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(3 + k)).tolist()
        assert len(got[k]) == 8
        logits = plain.forward(prompt + got[k], cfg.to_dict(), w).numpy()
        for j, tok in enumerate(got[k]):
            row = logits[n + j - 1]
            assert tok == int(row.argmax()) or row.max() - row[tok] < 1e-4 * np.abs(row).max(), f"request {k}, token {j}"
