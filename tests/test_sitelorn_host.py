"""Sitelorn's host side without a GPU: the configuration (keys, errors, what the specification says), the cache needs of
its layers, the manager's bookkeeping with state slots, the recurrence's work lists, the plain implementation's parts
against one another."""
import numpy as np
import pytest
import torch

import plain_sitelorn as plain
from test_sitelorn import MODELS, attention, config, gla, lightning


def typed(cfg, **kw):
    from infinicore_infer_b200.config import config_class_for
    return config_class_for(cfg).from_dict(cfg, **kw)


def test_the_registry_finds_the_design_by_its_architecture_key():
    from infinicore_infer_b200.config import SitelornConfig
    c = typed(MODELS["mixed-b"], max_tokens=99)
    assert isinstance(c, SitelornConfig) and c.max_positions == 99 and c.vocab == 130
    assert typed(c.to_dict(), max_tokens=99) == c


def test_specification_follows_the_layers_one_by_one():
    spec = typed(MODELS["mixed-b"]).model_spec()
    kinds = [type(b.mixer).__name__ for b in spec.layers]
    assert kinds == ["LinearAttentionSpec", "ConvAttentionSpec", "LinearAttentionSpec", "ConvAttentionSpec"]
    assert spec.layers[2].feed_forward is None and spec.layers[2].ffn_norm is None
    a = spec.layers[3].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.v_head_dim, a.conv_taps, a.window, a.position) == (3, 3, 20, 12, 5, 64, None)
    assert a.sink and a.head_gate and a.qk_norm and not a.shares_kv
    l = spec.layers[0].mixer
    assert l.decay == (0.98,) and l.qkv_act == "silu" and not l.norm_per_head and l.gate_act == "sigmoid"
    g = typed(MODELS["gla"]).model_spec().layers[0].mixer
    assert g.decay is None and g.decay_rank == 6 and g.decay_tau == 5.0 and g.q_scale == 16 ** -0.5 and g.norm_per_head


def test_the_decay_projection_takes_its_width_from_the_checkpoints_shapes():
    cfg = config(32, 50, [gla(2, 8, 8, 4.0, 3)])
    del cfg["layers"][0]["mixer"]["rank"]
    c = typed(cfg, shapes={"l0.mix.a1": (7, 32)})
    assert c.model_spec().layers[0].mixer.decay_rank == 7
    from infinicore_infer_b200.config import ConfigError
    with pytest.raises(ConfigError):
        typed(cfg).model_spec()


@pytest.mark.parametrize("break_it, word", [
    (lambda c: c["layers"][0].__setitem__("type", "mamba"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("decay", [0.5]), "decay"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 0), "kv_from"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "experts"), "mlp.kind"),
])
def test_a_configuration_that_does_not_fit_says_where(break_it, word):
    import copy
    from infinicore_infer_b200.config import ConfigError
    cfg = copy.deepcopy(config(32, 50, [lightning(2, 8, 8, [0.5, 0.9], ff=16), attention(2, 1, 8, 8, 2, 4, 1e4, 0.3, 9, ff=16)]))
    break_it(cfg)
    with pytest.raises(ConfigError) as e:
        typed(cfg)
    assert word in str(e.value)


def test_manifest_names_the_checkpoints_tensors():
    from infinicore_infer_b200.parts import model_manifest
    m = model_manifest(typed(MODELS["borrowed"]).model_spec())
    assert {"embed", "head", "final.norm", "final.norm.b", "l0.mix.k.conv", "l0.mix.q.norm", "l0.mix.g", "l1.mix.q.conv",
            "l1.norm2.b", "l1.mlp.down"} <= set(m)
    assert not any(n.startswith(("l1.mix.k", "l1.mix.v", "l0.mlp", "l0.norm2")) for n in m)
    assert m["l1.mix.q.conv"].shape == (64, 4) and m["l0.mix.g"].shape == (2, 64) and m["l0.mix.v"].shape == (16, 64)


def test_cache_bookkeeping_with_state_slots_and_a_shared_cache():
    from infinicore_infer_b200.cache import CacheManager
    from infinicore_infer_b200.parts import cache_needs, state_needs
    spec = typed(MODELS["mixed-a"]).model_spec()
    mgr = CacheManager(cache_needs(spec), num_pages=12, page_size=8, max_requests=2, max_positions=200, device=None,
                       entry_states=state_needs(spec))
    assert len(mgr.groups) == 1 and mgr.groups[0].need.window == 33
    mgr.admit("a")
    mgr.reserve("a", 90); mgr.commit("a", 90)
    # the window group gives back what no later query of either layer can see
    assert mgr.groups[0].pool.in_use == len([b for b in range(12) if b >= (90 - 33 + 1) // 8])
    mgr.release("a")
    mgr.check_invariants()
    assert mgr.slots.available == 2


def test_recurrence_work_lists():
    from infinicore_infer_b200.kernels import host
    from infinicore_infer_b200.parts import LinearAttention
    piece = host.scan_piece()
    lens = [3, 2 * piece + 5, 1, piece, piece + 1]
    caps = LinearAttention.step_list_capacity(sum(lens), len(lens) + 1)
    arrays = {n: np.zeros(max(1, c), dtype=np.int32) for n, c in caps.items()}
    got = LinearAttention.fill_step_lists(len(lens), len(lens) + 1, lens, [0] * len(lens), arrays)
    assert got["direct"] == (4, False) and list(arrays["direct"][:4]) == [0, 2, 3, 5]        # the padding request runs directly
    assert got["pieces"][0] == 5 and got["piece_reqs"][0] == 2
    rows = np.cumsum([0] + lens)
    assert arrays["pieces"][:10].reshape(5, 2).tolist() == [[rows[1], piece], [rows[1] + piece, piece], [rows[1] + 2 * piece, 5],
                                                            [rows[4], piece], [rows[4] + piece, 1]]
    assert arrays["piece_reqs"][:6].reshape(2, 3).tolist() == [[1, 0, 3], [4, 3, 2]]
    all_direct = LinearAttention.fill_step_lists(2, 4, [1, 1], [5, 9], arrays)
    assert all_direct["direct"] == (4, True) and all_direct["pieces"][0] == 0


def test_plain_recurrence_equals_its_unrolled_sum():
    g = torch.Generator().manual_seed(0)
    T, H, dk, dv = 9, 2, 3, 4
    q, k = torch.randn(T, H, dk, generator=g, dtype=torch.float64), torch.randn(T, H, dk, generator=g, dtype=torch.float64)
    v = torch.randn(T, H, dv, generator=g, dtype=torch.float64)
    a = torch.rand(T, H, dk, generator=g, dtype=torch.float64)
    o = plain.linear_recurrence(q, k, v, a)
    for t in (0, 4, 8):
        want = torch.zeros(H, dv, dtype=torch.float64)
        for s in range(t + 1):
            decay = torch.ones(H, dk, dtype=torch.float64)
            for r in range(s + 1, t + 1):
                decay = decay * a[r]
            want += torch.einsum("hk,hk,hv->hv", q[t], decay * k[s], v[s])
        assert torch.allclose(o[t], want, atol=1e-12)


def test_plain_attention_sees_exactly_its_window_and_the_sink_takes_weight():
    T = 12
    q = torch.ones(T, 1, 2, dtype=torch.float64)
    k = torch.zeros(T, 1, 2, dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64).view(T, 1, 1)
    o = plain.windowed_sink_attention(q, k, v, 1.0, 3)          # all scores 0: each seen key and the sink weigh the same
    assert torch.allclose(o[0, 0, 0], torch.tensor(0.0, dtype=torch.float64))
    assert torch.allclose(o[5, 0, 0], torch.tensor((3 + 4 + 5) / 4.0, dtype=torch.float64))
    assert torch.allclose(o[1, 0, 0], torch.tensor((0 + 1) / 3.0, dtype=torch.float64))


def test_more_windows_than_block_tables_share_groups_by_size():
    from infinicore_infer_b200.cache import CacheManager, PagedKV
    from infinicore_infer_b200.kernels.host import max_cache_groups
    n = max_cache_groups() + 3
    needs = [PagedKV(2, 16, 8 + 4 * i) for i in range(n)] + [PagedKV(1, 32, None, 8)]
    mgr = CacheManager(needs, num_pages=16, page_size=4, max_requests=2, max_positions=128, device=None)
    assert len(mgr.groups) == 2 and mgr.groups[0].need.window == 8 + 4 * (n - 1) and mgr.groups[1].need.v_head_dim == 8
    assert [v.group_index for v in mgr.views] == [0] * n + [1]
