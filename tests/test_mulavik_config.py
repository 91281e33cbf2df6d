"""Mulavik without a GPU: the configuration's reader and its errors, the model as data (parts, tensors, cache and
state needs), and the plain implementation's own checks against formulas written out element by element."""
import json
import math

import pytest
import torch

from mulavik_util import attention_layer, config, dense, memory_layer, moe, write_model


def build(cfg_dict):
    from nanoinfer_b200.config import MulavikConfig
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture

    cfg = MulavikConfig.from_dict(json.loads(json.dumps(cfg_dict)))
    return Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)


def test_the_architecture_is_registered():
    from nanoinfer_b200 import architectures
    from nanoinfer_b200.config.base import architecture_name

    assert {"Mulavik", "Vadonex", "GPT2LMHeadModel"} <= set(architectures())
    assert architecture_name({"architecture": "Mulavik"}) == "Mulavik"


def test_all_problems_of_a_configuration_come_in_one_error():
    from nanoinfer_b200.config import ConfigError, MulavikConfig

    bad = config([attention_layer(heads=3, kv_heads=2), memory_layer(), dict(type="conv", mixer={}),
                  attention_layer(mlp=moe(experts=2, top=3)), attention_layer(dim=8, rot_dims=10)])
    del bad["layers"][1]["mixer"]["gate_cap"]
    bad["norm"] = {}
    del bad["embedding"]["scale"]
    with pytest.raises(ConfigError) as e:
        MulavikConfig.from_dict(bad)
    text = str(e.value)
    for piece in ("norm.eps", "embedding.scale", "layers[0].mixer.heads", "layers[1].mixer.gate_cap", "layers[2].type",
                  "router.top", "layers[4].mixer.rot.dims"):
        assert piece in text, (piece, text)


def test_defaults_of_keys_that_may_be_left_out():
    cfg = config([attention_layer(rot_dims=None), attention_layer(mlp=moe(shared=0))])
    del cfg["layers"][0]["mixer"]["kv_heads"]
    m = build(cfg)
    att = m.layers[0].mixer
    assert att.n_kv_head == att.n_head and att.position is None and att.sink
    assert m.layers[1].feed_forward.shared_inner == 0 and not m.layers[1].feed_forward.shared_row_gate


def test_parts_tensors_cache_and_state_of_a_mixed_stack():
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.kernels.ops import mlstm_state_floats

    layers = [memory_layer(heads=2, dim=24, vdim=40, mlp=dense(80)), attention_layer(heads=4, kv_heads=2, dim=16, vdim=40, mlp=moe()),
              attention_layer(heads=4, kv_heads=2, dim=48, vdim=8, mlp=None), memory_layer(heads=3, dim=20, vdim=8, mlp=None)]
    m = build(config(layers, vocab=99, width=64))
    names = {b.ref.name for b in m.bindings()}
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.i.b", "l0.mix.norm",
            "l1.mix.q", "l1.mlp.router", "l1.mlp.e5.gate", "l1.mlp.shared.sg", "l2.norm1b", "l3.mix.f"} <= names
    assert "l2.norm2" not in names and "l2.mlp.up" not in names and "l1.mix.g" not in names
    shapes = {b.ref.name: tuple(b.spec.shape) for b in m.bindings()}
    assert shapes["l1.mix.q"] == (64, 64) and shapes["l1.mix.k"] == (32, 64) and shapes["l1.mix.v"] == (80, 64)
    assert shapes["l1.mix.o"] == (64, 160) and shapes["l0.mix.i"] == (2, 64) and shapes["l1.mlp.shared.sg"] == (1, 64)
    # keys and values of unequal sizes share pages of the larger one, rounded up to 16; layers of one size share a group
    kv = dict(m.kv_needs())
    assert kv[1].head_dim == 48 and kv[2].head_dim == 48 and kv[1].n_kv_head == 2 and kv[1].window == 0 and kv[1].planes == 2
    st = dict(m.state_needs())
    assert set(st) == {0, 3} and st[0].shape == (2 * mlstm_state_floats(24, 40),) and st[3].shape == (3 * mlstm_state_floats(20, 8),)
    assert mlstm_state_floats(24, 40) == 41 * 32 + 4
    assert m.capture_safe() and m.max_positions is None
    cm = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=128, max_requests=2, page_size=16, dtype=torch.float32,
                      device=None, max_positions=None)
    assert len(cm.groups) == 1
    r = cm.open_request()
    cm.append([(r, 40)])
    cm.commit(r, 40)
    assert cm.pages_used() == [3]
    cm.close_request(r)
    assert cm.pages_used() == [0]


def test_a_model_folder_round_trips_through_the_configuration(tmp_path):
    from nanoinfer_b200.registry import load_config

    cfg = config([memory_layer(mlp=moe()), attention_layer(mlp=dense())], vocab=77, width=32, scale=3.5, eps=2e-6)
    d = write_model(cfg, str(tmp_path), torch.float32)
    back = load_config(d)
    assert back.architecture == "Mulavik" and back.embedding_scale == 3.5 and back.eps == 2e-6 and back.n_layer == 2
    assert back.to_dict()["layers"] == cfg["layers"]


# ------------------------------------------------------------------ the plain implementation's own checks
def test_plain_sink_softmax_and_grouped_heads_element_by_element():
    from plain_mulavik import rotate_pairs, sink_attention

    torch.manual_seed(0)
    n, C, H, G, d, dv, dims, base = 6, 10, 4, 2, 6, 4, 4, 7.0
    W = {"q": torch.randn(H * d, C, dtype=torch.float64), "k": torch.randn(G * d, C, dtype=torch.float64),
         "v": torch.randn(G * dv, C, dtype=torch.float64), "o": torch.randn(C, H * dv, dtype=torch.float64)}
    h = torch.randn(n, C, dtype=torch.float64)
    m = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=0.3, rot=dict(base=base, dims=dims))
    got = sink_attention(h, W, "", m)

    def turn(vec, p):
        out = list(vec)
        for i in range(dims // 2):
            a = p * base ** (-2 * i / dims)
            u, w = vec[2 * i], vec[2 * i + 1]
            out[2 * i], out[2 * i + 1] = u * math.cos(a) - w * math.sin(a), w * math.cos(a) + u * math.sin(a)
        return out

    q, k, v = (h @ W["q"].T).tolist(), (h @ W["k"].T).tolist(), (h @ W["v"].T).tolist()
    heads = torch.zeros(n, H * dv, dtype=torch.float64)
    for t in range(n):
        for a in range(H):
            g = a // (H // G)
            qt = turn(q[t][a * d:(a + 1) * d], t)
            s = [0.3 * sum(x * y for x, y in zip(qt, turn(k[j][g * d:(g + 1) * d], j))) for j in range(t + 1)]
            den = 1.0 + sum(math.exp(x) for x in s)
            for c in range(dv):
                heads[t, a * dv + c] = sum(math.exp(s[j]) / den * v[j][g * dv + c] for j in range(t + 1))
    assert float((got - heads @ W["o"].T).abs().max()) < 1e-10
    # the first token sees itself and the sink only; its weight is below one
    x = torch.randn(1, 2, 8, dtype=torch.float64)
    assert torch.equal(rotate_pairs(x, torch.tensor([0]), 10.0, 8), x)


def test_plain_matrix_memory_element_by_element_and_in_two_halves():
    from plain_mulavik import mlstm

    torch.manual_seed(1)
    n, C, H, d, dv, cap, eps = 7, 9, 2, 3, 4, 2.5, 1e-5
    W = {k: torch.randn(s, C, dtype=torch.float64) for k, s in dict(q=H * d, k=H * d, v=H * dv, g=H * dv, i=H, f=H).items()}
    W.update({"i.b": torch.randn(H, dtype=torch.float64), "f.b": torch.randn(H, dtype=torch.float64) + 2,
              "norm": torch.rand(H * dv, dtype=torch.float64) + 0.5, "o": torch.randn(C, H * dv, dtype=torch.float64)})
    h = torch.randn(n, C, dtype=torch.float64) * 2
    m = dict(heads=H, dim=d, vdim=dv, gate_cap=cap)
    got = mlstm(h, W, "", m, eps)
    y = torch.zeros(n, H * dv, dtype=torch.float64)
    for a in range(H):
        S = [[0.0] * dv for _ in range(d)]
        nn, mx = [0.0] * d, 0.0
        for t in range(n):
            ht = h[t]
            q = [float(W["q"][a * d + i] @ ht) / math.sqrt(d) for i in range(d)]
            k = [float(W["k"][a * d + i] @ ht) for i in range(d)]
            v = [float(W["v"][a * dv + j] @ ht) for j in range(dv)]
            gi = cap * math.tanh((float(W["i"][a] @ ht) + float(W["i.b"][a])) / cap)
            zf = cap * math.tanh((float(W["f"][a] @ ht) + float(W["f.b"][a])) / cap)
            gf = -math.log1p(math.exp(-zf))
            new = max(gf + mx, gi)
            keep, take = math.exp(gf + mx - new), math.exp(gi - new)
            for i in range(d):
                nn[i] = keep * nn[i] + take * k[i]
                for j in range(dv):
                    S[i][j] = keep * S[i][j] + take * k[i] * v[j]
            mx = new
            den = max(abs(sum(nn[i] * q[i] for i in range(d))), math.exp(-mx)) + 1e-6
            o = [sum(S[i][j] * q[i] for i in range(d)) / den for j in range(dv)]
            r = math.sqrt(sum(x * x for x in o) / dv + eps)
            for j in range(dv):
                gate = 1 / (1 + math.exp(-float(W["g"][a * dv + j] @ ht)))
                y[t, a * dv + j] = o[j] / r * float(W["norm"][a * dv + j]) * gate
    assert float((got - y @ W["o"].T).abs().max()) < 1e-9
    # the state carries: two halves give what the whole gives
    first, st = mlstm(h[:4], W, "", m, eps, return_state=True)
    second = mlstm(h[4:], W, "", m, eps, state=st)
    assert float((torch.cat([first, second]) - got).abs().max()) < 1e-12
    # the running maximum starts at 0, not at minus infinity: with gates far below zero the first token's
    # denominator is the floor exp(-0) = 1, not |n . q|
    W2 = dict(W)
    W2["i.b"] = torch.full((H,), -50.0, dtype=torch.float64)
    m2 = dict(m, gate_cap=60.0)
    one = mlstm(h[:1], W2, "", m2, eps, return_state=True)[1]
    assert float(one[2].min()) > -20.0             # mx is f + 0 (a little below 0), not i = -50


def test_plain_feed_forwards_element_by_element():
    from plain_mulavik import dense_ff, routed_ff

    torch.manual_seed(2)
    n, C, F, E, top, Fs = 5, 6, 4, 5, 2, 3
    h = torch.randn(n, C, dtype=torch.float64)
    W = {"up": torch.randn(F, C, dtype=torch.float64), "down": torch.randn(C, F, dtype=torch.float64)}
    want = torch.zeros(n, C, dtype=torch.float64)
    for t in range(n):
        z = [max(float(W["up"][f] @ h[t]), 0.0) ** 2 for f in range(F)]
        for c in range(C):
            want[t, c] = sum(float(W["down"][c, f]) * z[f] for f in range(F))
    assert float((dense_ff(h, W, "") - want).abs().max()) < 1e-10
    W = {"router": torch.randn(E, C, dtype=torch.float64) * 2, "shared.sg": torch.randn(1, C, dtype=torch.float64)}
    for name, f in [(f"e{e}", F) for e in range(E)] + [("shared", Fs)]:
        W[f"{name}.gate"], W[f"{name}.up"] = torch.randn(f, C, dtype=torch.float64), torch.randn(f, C, dtype=torch.float64)
        W[f"{name}.down"] = torch.randn(C, f, dtype=torch.float64)
    mlp = dict(router=dict(experts=E, top=top), expert=dict(ff=F), shared=dict(ff=Fs))
    margins = []
    got = routed_ff(h, W, "", mlp, margins)

    def expert(name, x):
        f = W[f"{name}.gate"].shape[0]
        g = [float(W[f"{name}.gate"][i] @ x) for i in range(f)]
        u = [float(W[f"{name}.up"][i] @ x) for i in range(f)]
        mid = [g[i] / (1 + math.exp(-g[i])) * u[i] for i in range(f)]
        return torch.tensor([sum(float(W[f"{name}.down"][c, i]) * mid[i] for i in range(f)) for c in range(C)], dtype=torch.float64)

    for t in range(n):
        s = [1 / (1 + math.exp(-float(W["router"][e] @ h[t]))) for e in range(E)]
        best = sorted(range(E), key=lambda e: -s[e])[:top]
        out = sum(expert(f"e{e}", s[e] * h[t]) for e in best)          # the score scales what the expert reads
        out = out + expert("shared", h[t]) / (1 + math.exp(-float(W["shared.sg"][0] @ h[t])))
        assert float((got[t] - out).abs().max()) < 1e-10
        zs = sorted((float(W["router"][e] @ h[t]) for e in range(E)), reverse=True)
        assert abs(float(margins[0][t]) - (zs[top - 1] - zs[top]) / math.sqrt(sum(v * v for v in zs) / E)) < 1e-12
    # scaling the input is not scaling the output
    e0 = best[0]
    assert float((expert(f"e{e0}", s[e0] * h[-1]) - s[e0] * expert(f"e{e0}", h[-1])).abs().max()) > 1e-3


def test_the_plain_model_puts_norms_on_both_sides_of_a_sublayer(tmp_path):
    from plain_mulavik import PlainMulavik, dense_ff, mlstm, rms_norm

    cfg = config([memory_layer(heads=1, dim=8, vdim=8, mlp=dense(16))], vocab=30, width=16, scale=3.0)
    d = write_model(cfg, str(tmp_path), torch.float32)
    p = PlainMulavik(d)
    t = [3, 9, 27, 1]
    logits = p.logits(t)
    W, eps = p.W, p.eps
    x = W["embed"][torch.tensor(t)] * 3.0
    x = x + rms_norm(mlstm(rms_norm(x, W["l0.norm1"], eps), W, "l0.mix.", cfg["layers"][0]["mixer"], eps), W["l0.norm1b"], eps)
    x = x + rms_norm(dense_ff(rms_norm(x, W["l0.norm2"], eps), W, "l0.mlp."), W["l0.norm2b"], eps)
    assert float((p.streams[0] - x).abs().max()) < 1e-12
    assert float((logits - rms_norm(x, W["final.norm"], eps) @ W["head"].T).abs().max()) < 1e-12
    assert p.greedy(t, 3) == p.greedy(t, 3) and len(p.greedy(t, 3)) == 3
