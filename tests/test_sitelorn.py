"""Sitelorn through the engine against the plain implementation (tests/plain_sitelorn.py): each mixer alone, whole models
of other sizes and layer orders, prompts cut in every way, batches, reused pages and state slots, window edges, long
decoding, and greedy generation through the scheduler."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import random_tokens
import plain_sitelorn as plain
from trace_helpers import by_position, mixed, portions, staggered_plan, tail_decode, whole

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 3e-2}


def lightning(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def gla(heads, dim, vdim, tau, rank, ff=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def attention(heads, kv_heads, dim, vdim, conv, rot_dims, base, scale, window, kv_from=None, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "rot": {"dims": rot_dims, "base": base},
         "scale": scale, "mask": {"size": window}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(width, vocab, layers, scale=3.0, eps=1e-5):
    return {"architecture": "Sitelorn", "embedding": {"scale": scale}, "norm": {"eps": eps}, "vocab": vocab, "width": width,
            "layers": layers}


# Sizes that differ from one another in everything: key and value sizes that are unequal (and neither a power of two),
# one head and several, grouped and ungrouped key heads, rotation of a part and of the whole head, two, three and one
# taps, a borrowing layer with a wider window than its lender's, layers without feed-forward, attention first and last.
MODELS = {
    "lightning": config(64, 97, [lightning(3, 24, 16, [0.5, 0.97, 0.999], ff=72)]),
    "gla": config(48, 83, [gla(2, 16, 40, 5.0, 6, ff=56)], scale=2.0, eps=1e-6),
    "attention": config(64, 101, [attention(4, 2, 24, 40, 3, 8, 1e4, 0.4, 9, ff=80)]),
    "borrowed": config(64, 90, [attention(2, 1, 32, 16, 2, 32, 5e3, 0.3, 7), attention(2, 1, 32, 16, 4, 32, 5e3, 0.25, 19, kv_from=0, ff=40)]),
    "mixed-a": config(96, 211, [attention(6, 2, 16, 24, 3, 6, 2e5, 0.35, 21, ff=120), gla(3, 16, 24, 9.0, 5, ff=120),
                                attention(6, 2, 16, 24, 2, 6, 2e5, 0.3, 33, kv_from=0), lightning(3, 24, 16, [0.6, 0.9, 0.9995], ff=88),
                                gla(2, 24, 32, 3.0, 4)], scale=5.0),
    "mixed-b": config(64, 130, [lightning(1, 40, 72, [0.98], ff=48), attention(2, 2, 16, 16, 1, 16, 1e3, 0.5, 5, ff=48),
                                lightning(4, 8, 8, [0.3, 0.8, 0.99, 1.0]), attention(3, 3, 20, 12, 5, 0, 1e4, 0.45, 64, ff=96)],
                       scale=1.0, eps=3e-6),
    # head sizes that the tensor-core attention kernels take (64 and 128: tcgen05 tiles and the grouped decode kernel; 32: the
    # mma.sync tiles and the per-head decode kernel), keys and values of one size
    "heads64": config(128, 140, [attention(4, 2, 64, 64, 3, 32, 1e4, 0.2, 70, ff=96), gla(2, 64, 64, 4.0, 8),
                                 attention(4, 2, 64, 64, 2, 32, 1e4, 0.15, 131, kv_from=0, ff=96)], scale=2.0),
    "heads128": config(128, 99, [attention(2, 1, 128, 128, 4, 64, 5e5, 0.12, 40, ff=64), lightning(2, 128, 128, [0.9, 0.999], ff=64)]),
    "heads32": config(64, 77, [attention(6, 2, 32, 32, 2, 8, 1e4, 0.3, 23, ff=64), attention(6, 2, 32, 32, 3, 8, 1e4, 0.3, 11, kv_from=0)]),
    # nothing a multiple of anything: an odd width, odd head sizes, an odd feed-forward, a vocabulary that is prime
    "awkward": config(50, 61, [gla(3, 5, 9, 2.5, 3, ff=37), attention(3, 1, 9, 7, 3, 4, 777.0, 0.4, 6, ff=37),
                               lightning(2, 7, 5, [0.8, 0.99]), attention(3, 1, 9, 7, 2, 4, 777.0, 0.4, 13, kv_from=1, ff=21)], scale=2.5),
}
STD = 0.16     # matrices N(0, STD): products keep their input's spread, so scores and gates are far from flat


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from infinicore_infer_b200.config import config_class_for
    from infinicore_infer_b200.weights import index_directory, read_tensor, write_model_folder
    out = {}
    for seed, (name, cfg) in enumerate(MODELS.items()):
        d = str(tmp_path_factory.mktemp("sitelorn_" + name))
        write_model_folder(config_class_for(cfg).from_dict(cfg), d, seed=seed + 11, std=STD, norm_std=0.2)
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


def expected(folders, name, seed, n):
    key = (name, seed, n)
    if key not in _plain:
        _, cfg, w = folders[name]
        toks = random_tokens(seed, n, cfg["vocab"])
        _plain[key] = (toks, plain.forward(cfg, w, toks).numpy())
    return _plain[key]


def run(engine, steps):
    from infinicore_infer_b200.trace import replay
    return by_position(steps, replay(engine, steps))


def check(got, rid, want, tol, what):
    """Every position within ``tol`` of the logits' scale.  In bfloat16 the norm on a sublayer's output turns the rounding
    of a small output into a large relative error now and then (the same position stands out whole and token by token):
    one position in fifty may lie beyond ``tol``, none beyond three times it."""
    scale = np.abs(want).max()
    errs = np.array([np.abs(got[(rid, p)].astype(np.float64) - want[p]).max() for p in range(len(want))])
    loose = tol > 1e-3
    worst = int(errs.argmax())
    assert errs.max() <= (3 if loose else 1) * tol * scale, f"{what}: request {rid} position {worst}: error {errs.max():.3e} > {tol * scale:.3e}"
    if loose:
        over = int((errs > tol * scale).sum())
        assert over <= max(1, len(want) // 50), f"{what}: request {rid}: {over} of {len(want)} positions beyond {tol * scale:.3e}"


def test_config_reads_every_size_and_the_registry_finds_it(folders):
    from infinicore_infer_b200.config import SitelornConfig, read_config
    d, cfg, _ = folders["mixed-a"]
    c = read_config(d, max_tokens=256)
    assert isinstance(c, SitelornConfig) and c.max_positions == 256 and c.width == 96 and len(c.layers) == 5
    spec = c.model_spec()
    assert [e.cache for e in spec.order] == [0, 1, 0, 3, 4] and [e.writes_cache for e in spec.order] == [True, True, False, True, True]
    from infinicore_infer_b200.parts import cache_needs, state_needs
    needs = cache_needs(spec)
    assert needs[0].window == 33 and needs[0].v_head_dim == 24          # kept for the wider of the two windows
    assert needs[2] is None and needs[1].shape == (3, 16, 24)
    tails = state_needs(spec)
    assert tails[0].shape == (2, 6 * 16 + 2 * 16 + 2 * 24) and tails[2].shape == (1, 6 * 16) and tails[1] is None


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


def test_sink_and_gate_in_the_legacy_tensor_core_tiles(folders):
    """The mma.sync prefill tiles (what runs where the tcgen05 kernel is not built) with heads of 64."""
    from infinicore_infer_b200.engine import Engine
    eng = Engine.from_folder(folders["heads64"][0], dtype=torch.bfloat16, max_tokens=512, cache_tokens=512, page_size=16,
                             max_requests=2, max_step_tokens=512)
    eng.runtime.legacy_tensor_cores = True
    toks, want = expected(folders, "heads64", 302, 150)
    for what, steps in (("whole", whole("r", toks)), ("uneven", portions("r", toks, sizes=(17, 3, 31, 2, 16)))):
        check(run(eng, steps), "r", want, TOL["bfloat16"], f"legacy tiles {what}")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_every_token_decoded_alone_through_graphs(folders, engines, dtype):
    """Long decoding: every token a step of its own, so windows, pages and tails are passed one position at a time."""
    for name in ("mixed-a", "mixed-b", "heads64", "heads32", "heads128"):       # the last three: the split-key decode kernels
        toks, want = expected(folders, name, 77, 140)
        eng = engines(name, dtype)
        check(run(eng, tail_decode("r", toks, tail=len(toks))), "r", want, TOL[dtype], f"{name} {dtype} token by token")
        assert eng.steps_run >= 140


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", ["mixed-a", "mixed-b", "borrowed"])
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
    """The same request twice in a row lands in the slot (and pages) that its first run left: equal logits, bit for bit."""
    toks, want = expected(folders, "mixed-a", 9, 45)
    eng = engines("mixed-a", "float32", max_requests=1)
    a = run(eng, whole("r", toks))
    b = run(eng, portions("r", toks, sizes=(5, 2)))
    check(a, "r", want, TOL["float32"], "first run")
    check(b, "r", want, TOL["float32"], "second run in the same slot")


# ---- mechanisms alone, with inputs made so that one key decides ------------------------------------------------------------
def paged(k, v, page, dev, dtype):
    """Keys [T, G, dk] and values [T, G, dv] of one request into pages handed out in a scrambled order."""
    T, G, dk = k.shape
    blocks = (T + page - 1) // page
    order = torch.randperm(blocks, generator=torch.Generator().manual_seed(3)) + 1
    kp = torch.zeros(blocks + 1, G, page, dk, dtype=dtype, device=dev)
    vp = torch.zeros(blocks + 1, G, page, v.shape[-1], dtype=dtype, device=dev)
    for t in range(T):
        kp[order[t // page], :, t % page] = k[t].to(dtype)
        vp[order[t // page], :, t % page] = v[t].to(dtype)
    return kp, vp, order.to(torch.int32).view(1, -1).to(dev)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("window,page", [(7, 8), (16, 16), (33, 8)])
def test_window_edge_sink_and_gate_of_the_row_attention(dtype, window, page):
    """For chosen rows i the key just inside the window (i - W + 1) gets a large score and the key just outside (i - W)
    a larger one: a window that is one off in either direction changes the row's output from one value to another."""
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    g = torch.Generator().manual_seed(window)
    T, H, G, dk, dv = 120, 4, 2, 24, 40
    q = torch.randn(T, H, dk, generator=g, dtype=torch.float64)
    k = 0.3 * torch.randn(T, G, dk, generator=g, dtype=torch.float64)
    v = torch.randn(T, G, dv, generator=g, dtype=torch.float64)
    gate = torch.randn(T, H + 3, generator=g, dtype=torch.float64)
    for i in range(window + 2, T, 5):          # query head 0 reads key head 0
        unit = q[i, 0] / (q[i, 0] @ q[i, 0])
        k[i - window, 0] = 14.0 * unit
        k[i - window + 1, 0] = 9.0 * unit
    if dt == torch.bfloat16:
        q, k, v = (t.to(dt).double() for t in (q, k, v))
    want = plain.windowed_sink_attention(q, k, v, 1.0, window) * torch.sigmoid(gate[:, :H]).unsqueeze(-1)
    kp, vp, table = paged(k, v, page, dev, dt)
    out = torch.empty(T, H, dv, dtype=dt, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    K.attention_rows(q.to(dt).to(dev).contiguous(), kp, vp, out, pos, torch.zeros_like(pos), table, T, H, 1.0, window, sink=True,
                     gate=gate.float().to(dev)[:, :H + 3])
    err = (out.double().cpu() - want).abs().max().item()
    assert err <= (2e-5 if dt == torch.float32 else 3e-2), f"row attention differs by {err}"
    no_sink = torch.empty_like(out)
    K.attention_rows(q.to(dt).to(dev).contiguous(), kp, vp, no_sink, pos, torch.zeros_like(pos), table, T, H, 1.0, window)
    assert (no_sink.double().cpu()[:3].abs().sum() > out.double().cpu()[:3].abs().sum() * 0 ) and not torch.allclose(no_sink.float(), out.float())


def scan_inputs(T, H, dk, dv, rank, seed):
    g = torch.Generator().manual_seed(seed)
    ld = 2 * H * dk + 2 * H * dv + rank
    u = torch.randn(T, ld, generator=g, dtype=torch.float64)
    return u, ld


@pytest.mark.parametrize("H,dk,dv", [(1, 40, 72), (3, 24, 16), (2, 128, 128), (5, 7, 3)])
@pytest.mark.parametrize("projected", [False, True])
def test_recurrence_carries_its_state_across_cuts_and_slots(H, dk, dv, projected):
    """One sequence run whole, and cut into portions (one of a single row) that go through a state slot; a second
    sequence in another slot in the same launches.  A key of the first rows is made large so that losing the state, or
    decaying it wrongly, moves late outputs."""
    from infinicore_infer_b200 import kernels as K
    dev = torch.device("cuda:0")
    from infinicore_infer_b200.parts import LinearAttention
    rank, tau = 5, 6.0
    T = 230
    u, ld = scan_inputs(T, H, dk, dv, rank, 5)
    u2, _ = scan_inputs(T, H, dk, dv, rank, 6)
    u[1, H * dk: 2 * H * dk] *= 6.0           # an early key that late rows still see
    g = torch.Generator().manual_seed(1)
    decay = torch.tensor([0.999, 0.6, 0.95, 0.9, 1.0][:H], dtype=torch.float64)
    w2 = 0.5 * torch.randn(H * dk, rank, generator=g, dtype=torch.float64)
    b2 = 2.0 + torch.randn(H * dk, generator=g, dtype=torch.float64)
    offs = (0, H * dk, 2 * H * dk)
    r_off = 2 * H * dk + 2 * H * dv

    def plain_o(x):
        q = x[:, :H * dk].view(T, H, dk) * 0.5
        k = x[:, H * dk: 2 * H * dk].view(T, H, dk)
        v = x[:, 2 * H * dk: 2 * H * dk + H * dv].view(T, H, dv)
        if projected:
            a = torch.exp(torch.nn.functional.logsigmoid(x[:, r_off:] @ w2.T + b2) / tau).view(T, H, dk)
        else:
            a = decay.view(1, H, 1).expand(T, H, dk)
        return plain.linear_recurrence(q, k, v, a).reshape(T, H * dv)

    want = [plain_o(u), plain_o(u2)]
    state = torch.zeros(4, H, dk, dv, dtype=torch.float32, device=dev)
    state[0] = 7.0                              # slot 0 is nobody's; what lies there must not matter
    slots = torch.tensor([3, 1], dtype=torch.int32, device=dev)
    got = [[], []]
    cuts = [0, 1, 2, 30, 31, 160, 225, T]       # 129 rows in one portion: two whole pieces and one row more
    for a, b in zip(cuts, cuts[1:]):
        n = b - a
        rows = torch.cat([u[a:b], u2[a:b]]).float().to(dev)
        out = torch.empty(2 * n, H * dv, dtype=torch.float32, device=dev)
        caps = LinearAttention.step_list_capacity(2 * n, 2)
        arrays = {name: np.zeros(max(1, c), dtype=np.int32) for name, c in caps.items()}
        counts = LinearAttention.fill_step_lists(2, 2, [n, n], [a, a], arrays)
        lists = {name: torch.from_numpy(arrays[name][:max(1, counts[name][0] * w)]).to(dev) if counts[name][0] else None
                 for name, w in (("direct", 1), ("pieces", 2), ("piece_reqs", 3))}
        K.linear_scan(rows, offs, H, dk, dv, K.ACT_NONE, 0.5, None if projected else decay.float().to(dev),
                      w2.float().to(dev) if projected else None, b2.float().to(dev) if projected else None, r_off, tau, state,
                      torch.tensor([0, n, 2 * n], dtype=torch.int32, device=dev), slots, out, direct=lists["direct"],
                      pieces=lists["pieces"], piece_reqs=lists["piece_reqs"])
        got[0].append(out[:n].cpu()); got[1].append(out[n:].cpu())
    for i in range(2):
        o = torch.cat(got[i]).double()
        err = (o - want[i]).abs().max().item() / want[i].abs().max().item()
        assert err < 2e-5, f"sequence {i}: relative error {err}"
    assert torch.all(state[0] == 7.0) and torch.all(state[2] == 0.0)


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_convolution_norm_and_rotation_across_cuts(dtype):
    """Projections cut into portions shorter and longer than the taps, two requests side by side in scrambled pages:
    queries, cached keys and cached values equal the plain functions over the whole sequences."""
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    H, G, dk, dv, taps, rot, page = 3, 1, 10, 6, 4, 6, 8
    nq, nk, nv = H * dk, G * dk, G * dv
    T = 37
    g = torch.Generator().manual_seed(2)
    us = [torch.randn(T, nq + nk + nv + 2, generator=g, dtype=torch.float64) for _ in range(2)]
    conv = [torch.randn(n, taps, generator=g, dtype=torch.float64) for n in (nq, nk, nv)]
    norm = [1 + 0.3 * torch.randn(n, generator=g, dtype=torch.float64) for n in (nq, nk)]
    base, eps = 300.0, 1e-4
    freq = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(dev)
    blocks = (T + page - 1) // page
    kp = torch.zeros(2 * blocks + 1, G, page, dk, dtype=dt, device=dev)
    vp = torch.zeros(2 * blocks + 1, G, page, dv, dtype=dt, device=dev)
    table = torch.tensor([[2 * b + 2 for b in range(blocks)], [2 * b + 1 for b in range(blocks)]], dtype=torch.int32, device=dev)
    tail = torch.zeros(3, taps - 1, nq + nk + nv, dtype=torch.float32, device=dev)
    slots = torch.tensor([2, 1], dtype=torch.int32, device=dev)
    qs = [[], []]
    cuts = [0, 1, 3, 4, 12, 14, 29, T]
    for a, b in zip(cuts, cuts[1:]):
        n = b - a
        rows = torch.cat([us[0][a:b], us[1][a:b]]).float().to(dev)
        pos = torch.cat([torch.arange(a, b), torch.arange(a, b)]).to(torch.int32).to(dev)
        row_req = torch.tensor([0] * n + [1] * n, dtype=torch.int32, device=dev)
        q_out = torch.empty(2 * n, nq, dtype=dt, device=dev)
        K.conv_qkv(rows, (0, nq, nq + nk), H, G, dk, dv, True, [c.float().to(dev) for c in conv], taps, [w.float().to(dev) for w in norm],
                   eps, freq, rot, tail, pos, row_req, torch.tensor([0, n, 2 * n], dtype=torch.int32, device=dev), slots, table, page,
                   q_out, kp, vp)
        qs[0].append(q_out[:n].cpu()); qs[1].append(q_out[n:].cpu())
    tol = 2e-5 if dt == torch.float32 else 2e-2
    for i in range(2):
        u = us[i]
        q = plain.rotate_pairs((plain.rms(plain.short_conv(u[:, :nq], conv[0]), eps) * norm[0]).view(T, H, dk), {"dims": rot, "base": base})
        k = plain.rotate_pairs((plain.rms(plain.short_conv(u[:, nq:nq + nk], conv[1]), eps) * norm[1]).view(T, G, dk), {"dims": rot, "base": base})
        v = plain.short_conv(u[:, nq + nk:nq + nk + nv], conv[2]).view(T, G, dv)
        assert (torch.cat(qs[i]).double().view(T, H, dk) - q).abs().max() < tol * q.abs().max()
        for t in range(T):
            pg = table[i, t // page].item()
            assert (kp[pg, :, t % page].double().cpu() - k[t]).abs().max() < tol * k.abs().max(), f"key {t} of request {i}"
            assert (vp[pg, :, t % page].double().cpu() - v[t]).abs().max() < tol * v.abs().max(), f"value {t} of request {i}"


def test_layer_norm_and_gated_unit_kernels():
    from infinicore_infer_b200 import kernels as K
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(4)
    for d in (5, 96, 1000):
        x = torch.randn(7, d, generator=g, dtype=torch.float64) * 3 + 1.5
        delta = torch.randn(7, d, generator=g, dtype=torch.float64) * 2 - 4
        w, b = torch.randn(d, generator=g, dtype=torch.float64), torch.randn(d, generator=g, dtype=torch.float64)
        xs = x.float().to(dev)
        h = torch.empty(7, d, dtype=torch.bfloat16, device=dev)
        K.layernorm(delta.float().to(dev), w.float().to(dev), b.float().to(dev), 1e-5, out=h, add_into=xs)
        want = x + plain.layer_norm(delta, w, b, 1e-5)
        assert (xs.double().cpu() - want).abs().max() < 1e-5 * want.abs().max()
        assert torch.equal(h, xs.to(torch.bfloat16))
        rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=dev)
        out = torch.empty(3, d, dtype=torch.float32, device=dev)
        K.layernorm(x.float().to(dev), w.float().to(dev), b.float().to(dev), 1e-5, out=out, rows=rows)
        want = plain.layer_norm(x[[6, 0, 3]], w, b, 1e-5)
        assert (out.double().cpu() - want).abs().max() < 1e-5 * want.abs().max()
        gu = torch.randn(7, 2 * d, generator=g, dtype=torch.float64) * 2
        out = torch.empty(7, d, dtype=torch.float32, device=dev)
        K.glu(gu.float().to(dev), out, K.ACT_GELU_TANH)
        want = plain.gelu_tanh(gu[:, :d]) * gu[:, d:]
        assert (out.double().cpu() - want).abs().max() < 1e-5 * want.abs().max()


# ---- generation through the scheduler ---------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler_matches_the_plain_model(folders):
    """Requests of unequal length through ``Generator`` (admission, portions of 16 tokens, decoding beside prompts, three
    slots for five requests): every generated token is the plain model's argmax given the tokens before it."""
    from infinicore_infer_b200.engine import Engine, Generator
    name = "mixed-a"
    d, cfg, w = folders[name]
    eng = Engine.from_folder(d, dtype=torch.float32, max_tokens=160, cache_tokens=3 * 96, page_size=16, max_requests=3, max_step_tokens=64)
    gen = Generator(eng, chunk_size=16)
    prompts = [random_tokens(900 + i, n, cfg["vocab"]) for i, n in enumerate((40, 3, 25, 61, 12))]
    outs = gen.generate(prompts, max_new_tokens=12)
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        logits = plain.forward(cfg, w, p + o).numpy()
        for j, tok in enumerate(o):
            row = logits[len(p) + j - 1]
            best = int(row.argmax())
            assert tok == best or row[best] - row[tok] < 1e-4 * np.abs(row).max(), f"token {j} of a prompt of {len(p)}"
    eng.cache.check_invariants()
