"""Vadonex without a GPU: the configuration's reader and its errors, the model as data (schedule, cache and
state needs), the cache manager with one-plane groups, sizes taken from tensor shapes, and the plain
implementation's own checks against formulas written out element by element."""
import json
import math
import os

import pytest
import torch

from vadonex_util import attention_layer, config, delta_layer, dense, moe, write_model


def build(cfg_dict):
    from nanoinfer_b200.config import VadonexConfig
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture

    cfg = VadonexConfig.from_dict(json.loads(json.dumps(cfg_dict)))
    return Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)


def test_the_architecture_is_registered_and_named_by_one_string():
    from nanoinfer_b200 import architectures
    from nanoinfer_b200.config.base import architecture_name

    assert "Vadonex" in architectures() and "GPT2LMHeadModel" in architectures()
    assert architecture_name({"architecture": "Vadonex"}) == "Vadonex"
    assert architecture_name({"architectures": ["GPT2LMHeadModel"]}) == "GPT2LMHeadModel"


def test_all_problems_of_a_configuration_come_in_one_error():
    from nanoinfer_b200.config import ConfigError, VadonexConfig

    bad = config([attention_layer(kv_from=0), delta_layer(), dict(type="conv", mixer={}), attention_layer(mlp=moe(experts=2, top=3))])
    del bad["layers"][1]["mixer"]["heads"]
    bad["norm"] = {}
    with pytest.raises(ConfigError) as e:
        VadonexConfig.from_dict(bad)
    text = str(e.value)
    for piece in ("norm.eps", "layers[0].mixer.kv_from", "layers[1].mixer.heads", "layers[2].type", "router.top"):
        assert piece in text, (piece, text)


def test_a_reader_of_another_layers_cache_must_fit_it():
    from nanoinfer_b200.config import ConfigError, VadonexConfig

    ok = config([attention_layer(), delta_layer(), attention_layer(kv_from=0, window=40, heads=3, dim=8, vdim=8)])
    VadonexConfig.from_dict(ok)
    for change in (dict(kv_rank=16), dict(rot_dim=4, rot_dims=4)):
        bad = config([attention_layer(), attention_layer(kv_from=0, **change)])
        with pytest.raises(ConfigError):
            VadonexConfig.from_dict(bad)
    with pytest.raises(ConfigError):      # a reader of a reader
        VadonexConfig.from_dict(config([attention_layer(), attention_layer(kv_from=0), attention_layer(kv_from=1)]))


def test_schedule_cache_groups_and_state_of_a_mixed_stack():
    from nanoinfer_b200.cache import CacheManager

    m = build(config([delta_layer(heads=3, dim=16), attention_layer(window=24), attention_layer(kv_from=1, window=56),
                      attention_layer(window=0, kv_rank=16, mlp=dense()), delta_layer(mlp=moe()),
                      attention_layer(kv_from=3, window=8, kv_rank=16)]))
    assert [e.cache_of for e in m.schedule] == [None, None, 1, None, None, 3]
    needs = dict(m.kv_needs())
    # the owner's pages are kept for the widest window that reads them; no window at all is the widest
    assert needs[1].window == 56 and needs[3].window == 0 and set(needs) == {1, 3}
    assert all(s.planes == 1 and s.n_kv_head == 1 for s in needs.values())
    assert needs[1].head_dim == 32 + 8 and needs[3].head_dim == 16 + 8
    assert [(i, tuple(s.shape)) for i, s in m.state_needs()] == [(0, (3, 16, 16)), (4, (2, 16, 16))]
    assert m.capture_safe()
    cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=128, max_requests=2, page_size=16,
                         dtype=torch.float32, device=torch.device("cpu"), padding=True)
    shapes = sorted(tuple(g.tensor.shape) for g in cache.groups)
    assert shapes == [(1, 9, 1, 1, 16, 24), (1, 9, 1, 1, 16, 40)]
    assert sorted(g.bytes_per_page(4) for g in cache.groups) == [16 * 24 * 4, 16 * 40 * 4]
    r = cache.open_request()
    cache.append([(r, 100)])
    cache.commit(r, 100)
    held = {g.spec.window: sum(p >= 0 for p in blocks) for g, blocks in zip(cache.groups, r.blocks)}
    assert held[0] == 7 and held[56] == 7 - (100 - 56 + 1) // 16     # pages behind the widest window went back
    cache.close_request(r)
    cache.check()


def test_a_layer_without_feed_forward_has_no_second_norm():
    m = build(config([attention_layer(mlp=None), delta_layer(mlp=dense())]))
    names = {b.ref.name for b in m.bindings()}
    assert "l0.norm2" not in names and "l1.norm2" in names and {"l0.dwa", "l1.dwa", "final.norm", "head"} <= names
    assert m.layers[0].feed_forward is None and m.layers[1].feed_forward is not None


def test_the_decay_rank_comes_from_the_tensor_when_the_file_does_not_give_it(tmp_path):
    from nanoinfer_b200 import load_config
    from nanoinfer_b200.config import ConfigError, VadonexConfig
    from nanoinfer_b200.models.vadonex import build_vadonex_spec

    d = write_model(config([delta_layer(decay_rank=12), attention_layer()]), str(tmp_path))
    with open(os.path.join(d, "config.json")) as fh:
        raw = json.load(fh)
    del raw["layers"][0]["mixer"]["decay_rank"]
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(raw, fh)
    assert load_config(d).layers[0]["mixer"]["decay_rank"] == 12
    with pytest.raises(ConfigError):
        build_vadonex_spec(VadonexConfig.from_dict(raw))      # no folder was seen: the size is unknown


def test_random_weights_round_trip_and_parameter_count(tmp_path):
    from nanoinfer_b200.measure import parameter_count_of_spec
    from plain_vadonex import PlainVadonex

    cfg = config([delta_layer(mlp=dense()), attention_layer(mlp=moe()), attention_layer(kv_from=1)], vocab=50, width=32)
    d = write_model(cfg, str(tmp_path))
    plain = PlainVadonex(d)
    assert parameter_count_of_spec(build(cfg)) == sum(t.numel() for t in plain.W.values())
    logits = plain.logits([1, 2, 3, 4, 5])
    assert logits.shape == (5, 50) and torch.isfinite(logits).all()


# ------------------------------------------------------------------ the plain implementation against element-wise formulas
def test_plain_delta_rule_against_scalar_loops():
    from plain_vadonex import general_delta

    torch.manual_seed(0)
    n, C, H, d, R, eps = 5, 6, 2, 3, 2, 1e-5
    m = dict(heads=H, dim=d)
    W = {k: torch.randn(H * d, C, dtype=torch.float64) for k in ("r", "k", "v", "g", "a")}
    W.update({"a.b": torch.randn(H * d, dtype=torch.float64), "w1": torch.randn(R, C, dtype=torch.float64),
              "w2": torch.randn(H * d, R, dtype=torch.float64), "w0": torch.randn(H * d, dtype=torch.float64),
              "norm": torch.randn(H * d, dtype=torch.float64), "o": torch.randn(C, H * d, dtype=torch.float64)})
    h = torch.randn(n, C, dtype=torch.float64)
    got = general_delta(h, W, "", m, eps)
    sig = lambda z: 1.0 / (1.0 + math.exp(-z))
    out = torch.zeros(n, H * d, dtype=torch.float64)
    S = [[[0.0] * d for _ in range(d)] for _ in range(H)]
    for t in range(n):
        proj = {k: (W[k] @ h[t]).tolist() for k in ("r", "k", "v", "g", "a")}
        wl = (W["w2"] @ torch.tanh(W["w1"] @ h[t]) + W["w0"]).tolist()
        for hh in range(H):
            sl = slice(hh * d, (hh + 1) * d)
            r, k, v = proj["r"][sl], proj["k"][sl], proj["v"][sl]
            w = [math.exp(-math.exp(-0.5) * sig(z)) for z in wl[sl]]
            a = [sig(z + b) for z, b in zip(proj["a"][sl], W["a.b"][sl].tolist())]
            nk = math.sqrt(sum(z * z for z in k) + 1e-6)
            u = [z / nk for z in k]
            uS = [sum(u[i] * S[hh][i][j] for i in range(d)) for j in range(d)]
            S[hh] = [[w[i] * S[hh][i][j] - a[i] * u[i] * uS[j] + k[i] * v[j] for j in range(d)] for i in range(d)]
            o = [sum(S[hh][i][j] * r[i] for i in range(d)) for j in range(d)]
            scale = math.sqrt(sum(z * z for z in o) / d + eps)
            for j in range(d):
                out[t, hh * d + j] = o[j] / scale * float(W["norm"][hh * d + j]) * sig(proj["g"][sl][j])
    assert torch.allclose(got, out @ W["o"].T, atol=1e-10)


def test_plain_window_sees_exactly_its_size():
    from plain_vadonex import visible

    v = visible(6, 6, 0, 3)
    assert v.tolist() == [[j <= i and i - j < 3 for j in range(6)] for i in range(6)]
    assert visible(2, 8, 5, 0).tolist() == [[j <= 5 + i for j in range(8)] for i in range(2)]


def test_plain_rotation_pairs_neighbours_and_leaves_the_rest():
    from plain_vadonex import rotate_pairs

    v = torch.arange(12, dtype=torch.float64).view(2, 6) + 1
    out = rotate_pairs(v, torch.tensor([0, 3]), 100.0, 4)
    assert torch.equal(out[0], v[0]) and torch.equal(out[1, 4:], v[1, 4:])
    for i in range(2):
        a = 3 * 100.0 ** (-2 * i / 4)
        u, w = float(v[1, 2 * i]), float(v[1, 2 * i + 1])
        assert abs(float(out[1, 2 * i]) - (u * math.cos(a) - w * math.sin(a))) < 1e-12
        assert abs(float(out[1, 2 * i + 1]) - (w * math.cos(a) + u * math.sin(a))) < 1e-12


def test_plain_router_weights_are_the_scores_themselves():
    from plain_vadonex import gelu_erf, routed_ff

    torch.manual_seed(1)
    C, E, F = 5, 4, 3
    W = {"router": torch.randn(E, C, dtype=torch.float64) * 3}
    for e in range(E):
        W[f"e{e}.up"], W[f"e{e}.down"] = torch.randn(F, C, dtype=torch.float64), torch.randn(C, F, dtype=torch.float64)
    h = torch.randn(7, C, dtype=torch.float64)
    got = routed_ff(h, W, "", dict(router=dict(experts=E, top=2), expert=dict(ff=F)))
    for t in range(7):
        s = torch.softmax(W["router"] @ h[t], 0)
        best = sorted(range(E), key=lambda e: -float(s[e]))[:2]
        want = sum(s[e] * (W[f"e{e}.down"] @ gelu_erf(W[f"e{e}.up"] @ h[t])) for e in best)
        assert torch.allclose(got[t], want, atol=1e-12)
        assert float(sum(s[e] for e in best)) < 1.0


def test_block_tables_grow_when_a_request_behind_a_window_outgrows_the_pool():
    from nanoinfer_b200.cache import CacheManager, PoolExhausted
    from nanoinfer_b200.parts.base import KVCacheSpec

    cache = CacheManager([(0, KVCacheSpec(1, 8, window=20, planes=1))], [], max_tokens=64, max_requests=2, page_size=16)
    assert cache.max_blocks == [4]
    a, b = cache.open_request(), cache.open_request()
    cache.append([(b, 3)])
    cache.commit(b, 3)
    for _ in range(300):                       # 300 positions through a pool of 4 pages, one of them b's
        cache.append([(a, 1)])
        cache.commit(a, 1)
        cache.check()
        assert cache.pages_used()[0] <= 4
    assert cache.max_blocks[0] >= 19 and cache.table_generation >= 1
    assert len(a.table_rows[0]) == len(b.table_rows[0]) == cache.max_blocks[0]
    assert [i for i, p in enumerate(a.table_rows[0]) if p >= 0] == [17, 18] and b.table_rows[0][0] >= 0
    # without a window nothing can outgrow the pool: the pool runs out first, and nothing changes
    plain = CacheManager([(0, KVCacheSpec(1, 8, window=0, planes=1))], [], max_tokens=64, max_requests=1, page_size=16)
    r = plain.open_request()
    with pytest.raises(PoolExhausted):
        plain.append([(r, 65)])
    assert plain.max_blocks == [4] and plain.table_generation == 0
