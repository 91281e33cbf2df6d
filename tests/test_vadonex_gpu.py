"""Vadonex on the GPU: every new kernel alone against plain torch, every mechanism alone as a one-layer
model, and whole models through the step function, cut into steps every way, against the plain
implementation (tests/plain_vadonex.py).  Test weights are made so that faults show (vadonex_util.write_model);
where random values would still hide one (a window's edge), the kernel test builds queries and keys by hand."""
import json
import math
import os
import random
from types import SimpleNamespace

import pytest
import torch

from vadonex_util import TOL, attention_layer, clear_rows, config, delta_layer, dense, moe, rel_err, write_model

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda"


def toks(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# =============================================================================== kernels alone
@pytest.mark.parametrize("C", [40, 264, 1536])
def test_stream_kernels_against_torch(C):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(C)
    T, R, eps = 9, 12, 3e-5
    x0 = torch.randn(R, C, device=DEV) * 3
    w = torch.rand(C, device=DEV) + 0.5
    rows = torch.tensor([5, 0, 8, 8], dtype=torch.int32, device=DEV)
    out = torch.zeros(4, C, device=DEV)
    ops.rmsnorm(x0, w, eps, out, 4, rows)
    ref = lambda v: (v.double() / torch.sqrt((v.double() ** 2).mean(-1, keepdim=True) + eps) * w.double())
    assert float((out - ref(x0[rows.long()])).abs().max()) < 1e-5
    for dt in (torch.float32, torch.bfloat16):
        x, xn, lv0 = x0.clone(), torch.zeros(R, C, device=DEV, dtype=dt), torch.zeros(R, C, device=DEV)
        ops.stream_enter(x, xn, 1.75, T, lv0)
        assert torch.equal(x[:T], 1.75 * x0[:T]) and torch.equal(x[T:], x0[T:]) and torch.equal(lv0[:T], x0[:T])
        assert torch.equal(xn[:T], x0[:T].to(dt)) and not xn[T:].any()
        # norm, the level's store, the sum over levels, the next sublayer's input and scale: one kernel
        levels = torch.randn(4, R, C, device=DEV)
        keep = levels.clone()
        mix = torch.tensor([0.4, -0.3, 0.7, 9.9], device=DEV)
        x = x0.clone()
        ops.post_norm(x, w, eps, T, xn=xn, alpha_next=0.5, levels=levels, n_levels=3, mix=mix)
        y = ref(x0[:T])
        z = 0.4 * keep[0, :T].double() + -0.3 * keep[1, :T].double() + 0.7 * y
        assert float((levels[2, :T] - y).abs().max()) < 1e-5 and torch.equal(levels[3], keep[3]) and torch.equal(levels[:2], keep[:2])
        assert float((x[:T] - 0.5 * z).abs().max()) < 1e-5 and torch.equal(x[T:], x0[T:])
        assert float((xn[:T].double() - z).abs().max()) < (1e-5 if dt == torch.float32 else 0.05)
        x = x0.clone()
        ops.post_norm(x, w, eps, T)
        assert float((x[:T] - y).abs().max()) < 1e-5


def test_unary_kernels_against_torch():
    from nanoinfer_b200.kernels import ops
    from plain_vadonex import xielu

    torch.manual_seed(3)
    src = torch.randn(11, 50, device=DEV) * 3
    prm = torch.tensor([0.3, -1.2], device=DEV)
    out = torch.zeros(11, 20, device=DEV)
    ops.unary(src[:, 30:], out, 7, ops.UNARY_TANH)
    assert float((out[:7] - torch.tanh(src[:7, 30:].double())).abs().max()) < 1e-6 and not out[7:].any()
    want = xielu(src.double(), 0.3, -1.2)
    buf = src.clone()
    ops.unary(buf, buf, 11, ops.UNARY_XIELU, prm)
    assert float((buf - want).abs().max() / want.abs().max()) < 1e-6
    b16 = src.to(torch.bfloat16)
    want16 = xielu(b16.double(), 0.3, -1.2)
    ops.unary(b16, b16, 11, ops.UNARY_XIELU, prm)
    assert float(((b16.double() - want16).abs() / (want16.abs() + 1e-2)).max()) < 1e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_product_per_head_against_torch(dtype):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(5)
    M, H, N, K, pad = 37, 3, 20, 12, 5
    a = torch.randn(40, H * (K + pad), device=DEV).to(DT[dtype])
    w = torch.randn(H, N, K, device=DEV).to(DT[dtype])
    for out_dt in {torch.float32, DT[dtype]}:
        out = torch.zeros(40, H * (N + 3), device=DEV, dtype=out_dt)
        ops.linear_heads(a, K + pad, w, out, N + 3, M)
        ref = torch.einsum("mhk,hnk->mhn", a.double().view(40, H, K + pad)[:M, :, :K], w.double())
        got = out.double().view(40, H, N + 3)
        assert float((got[:M, :, :N] - ref).abs().max()) < (1e-4 if out_dt == torch.float32 else 0.06)
        assert not got[M:].any() and not got[:, :, N:].any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,C,F", [(5, 1, 40, 12), (4, 4, 64, 33), (12, 3, 88, 24)])
def test_routing_kernels_against_torch(E, top, C, F, dtype):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(E * 10 + top)
    dt, T = DT[dtype], 19
    h = torch.randn(T + 2, C, device=DEV).to(dt)
    wr = (torch.randn(E, C, device=DEV) * 0.5).to(dt)
    ids = torch.full((T + 2, top), -7, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T + 2, top, device=DEV)
    ops.moe_route(h, wr, T, top, False, ids, wts)
    s = torch.softmax(h[:T].double() @ wr.double().T, -1)
    score, chosen = torch.topk(s, top, -1)
    assert torch.equal(ids[:T].long(), chosen) and (ids[T:] == -7).all()
    assert float((wts[:T] - score).abs().max()) < 1e-5
    ops.moe_route(h, wr, T, top, True, ids, wts)
    assert float((wts[:T] - score / score.sum(-1, keepdim=True)).abs().max()) < 1e-5
    ops.moe_route(h, wr, T, top, False, ids, wts)
    up = (torch.randn(E, F, C, device=DEV) * 0.2).to(dt)
    down = (torch.randn(E, C, F, device=DEV) * 0.2).to(dt)
    inner = torch.zeros((T + 2) * top, F, device=DEV, dtype=dt)
    ops.moe_up(h, up, ids, inner, T, top, ops.ACT_GELU_ERF)
    pre = torch.einsum("tc,tkfc->tkf", h[:T].double(), up.double()[chosen])
    mid = 0.5 * pre * (1 + torch.erf(pre / math.sqrt(2)))
    tol = 1e-5 if dtype == "float32" else 0.03
    assert float((inner[:T * top].double().view(T, top, F) - mid).abs().max()) < tol
    x0 = torch.randn(T + 2, C, device=DEV)
    x = x0.clone()
    ops.moe_down(inner, down, ids, wts, x, T, top)
    add = torch.einsum("tk,tkf,tkcf->tc", score, inner[:T * top].double().view(T, top, F), down.double()[chosen])
    assert float((x[:T] - (x0[:T] + add)).abs().max()) < 1e-4 and torch.equal(x[T:], x0[T:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,C,F", [(4, 2, 72, 50), (3, 1, 130, 33), (8, 3, 256, 96)])
def test_experts_row_by_row_expert_by_expert_and_all_at_once_agree(E, top, C, F, dtype):
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.base import Workspace

    torch.manual_seed(E + C)
    dt, T = DT[dtype], 150
    h = torch.randn(T, C, device=DEV).to(dt)
    up, down = (torch.randn(E, F, C, device=DEV) * 0.2).to(dt), (torch.randn(E, C, F, device=DEV) * 0.2).to(dt)
    ids = torch.stack([torch.randperm(E)[:top] for _ in range(T)]).to(torch.int32).to(DEV)
    wts = torch.rand(T, top, device=DEV)
    x0 = torch.randn(T + 10, C, device=DEV)
    got = {}
    for form, (dense, grouped) in {"row by row": (False, False), "expert by expert": (False, True),
                                   "all experts at once": (True, True)}.items():
        ops.MOE_DENSE, ops.MOE_GROUPED = dense, grouped
        try:
            x, inner = x0.clone(), torch.zeros(T * top, F, device=DEV, dtype=dt)
            ops.moe_experts(h, up, down, ids, wts, inner, x, T, top, ops.ACT_GELU_ERF, Workspace(torch.device(DEV)))
            got[form] = x
        finally:
            ops.MOE_DENSE = ops.MOE_GROUPED = True
    pre = torch.einsum("tc,tkfc->tkf", h.double(), up.double()[ids.long()])
    mid = 0.5 * pre * (1 + torch.erf(pre / math.sqrt(2)))
    want = x0[:T].double() + torch.einsum("tk,tkf,tkcf->tc", wts.double(), mid, down.double()[ids.long()])
    # (in bfloat16 the inner activations, in one form times their weight, are rounded to 8 bits: the bound goes
    # with the size of the sums)
    tol = 1e-4 if dtype == "float32" else 0.01 * float(want.abs().max())
    for form, x in got.items():
        assert float((x[:T] - want).abs().max()) < tol, form
        assert torch.equal(x[T:], x0[T:]), form


@pytest.mark.parametrize("dim", [16, 40, 48, 64, 128])
def test_delta_rule_kernel_carries_its_state_in_the_slot(dim):
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(dim)
    H, eps, lens, slots = 3, 1e-5, [1, 7, 33], [4, 0, 2]
    N, T = H * dim, sum(lens)
    proj = torch.randn(T + 3, 5 * N + 6, device=DEV)
    wl = torch.randn(T + 3, N, device=DEV) * 2 - 2
    w0, ab, nw = torch.randn(N, device=DEV), torch.randn(N, device=DEV), torch.rand(N, device=DEV) + 0.5
    state0 = torch.randn(6, H, dim, dim, device=DEV) * 0.3

    def plain(rows, S):
        r, k, v, g, a = (proj[rows, i * N:(i + 1) * N].double().view(-1, H, dim) for i in range(5))
        w = torch.exp(-math.exp(-0.5) * torch.sigmoid(wl[rows].double() + w0.double())).view(-1, H, dim)
        a = torch.sigmoid(a + ab.double().view(H, dim))
        u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        S, out = S.double().clone(), []
        for t in range(len(rows)):
            uS = torch.einsum("hi,hij->hj", u[t], S)
            S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
            o = torch.einsum("hij,hi->hj", S, r[t])
            o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
            out.append(o.reshape(N) * nw.double() * torch.sigmoid(g[t].reshape(N)))
        return torch.stack(out), S

    def run(cuts, with_unit=True):
        """every entry's rows in portions: one launch per round of portions"""
        state = state0.clone()
        out = torch.zeros(T + 3, N, device=DEV)
        first = [sum(lens[:i]) for i in range(len(lens))]
        at = [0] * len(lens)
        while any(at[i] < lens[i] for i in range(len(lens))):
            # rows of the entries that still have some, packed in entry order into a fresh buffer
            rows, starts, sl = [], [0], []
            for i in range(len(lens)):
                n = min(cuts, lens[i] - at[i])
                if n > 0:
                    rows += list(range(first[i] + at[i], first[i] + at[i] + n))
                    starts.append(len(rows))
                    sl.append(slots[i])
                    at[i] += n
            idx = torch.tensor(rows, device=DEV)
            ctx = SimpleNamespace(n_rows=len(rows), n_entries=len(sl),
                                  entry_start=torch.tensor(starts, dtype=torch.int32, device=DEV),
                                  entry_slot=torch.tensor(sl, dtype=torch.int32, device=DEV))
            o = torch.zeros(len(rows), N, device=DEV)
            unit = torch.zeros(len(rows), N, device=DEV) if with_unit else None
            ops.delta_rule(proj[idx].contiguous(), (0, N, 2 * N, 3 * N, 4 * N), wl[idx].contiguous(), w0, ab, nw, state,
                           ctx, H, dim, eps, o, unit)
            out[idx] = o
        return out, state

    want, want_state = torch.zeros(T, N, dtype=torch.float64, device=DEV), state0.double().clone()
    at = 0
    for n, s in zip(lens, slots):
        o, S = plain(list(range(at, at + n)), state0[s])
        want[at:at + n], want_state[s] = o, S
        at += n
    for cuts, with_unit in ((1000, True), (1000, False), (1, True), (2, True), (5, True), (5, False)):
        got, state = run(cuts, with_unit)
        assert float((got[:T] - want).abs().max()) < 2e-4, (cuts, with_unit)
        assert float((state - want_state).abs().max()) < 2e-4, (cuts, with_unit)   # untouched slots stay as they were


def _latent_case(dtype, kv_rank, rot, page, window, positions, hot, n_splits=None):
    """One request's rows at ``positions`` over a cache whose pages lie in a scrambled order; the key at
    ``hot[i]`` is made to tower over row i's other scores."""
    from nanoinfer_b200.kernels import ops

    torch.manual_seed(11)
    D, H, n_keys = kv_rank + rot, 3, max(positions) + 1
    n_blocks = -(-n_keys // page)
    table = torch.randperm(n_blocks + 3)[:n_blocks].to(torch.int32)
    cache = torch.zeros(n_blocks + 3, 1, 1, page, D, device=DEV, dtype=dtype)
    lat = torch.randn(n_keys, D) * 0.3
    q = torch.randn(len(positions) + 1, H, D) * 0.3
    for i, j in enumerate(hot):
        if j is not None:
            q[i] += 6.0 * lat[j] / lat[j].norm()
    for j in {j for j in hot if j is not None}:
        lat[j] *= 4.0
    lat = lat.to(dtype)
    for j in range(n_keys):
        cache[int(table[j // page]), 0, 0, j % page] = lat[j].to(DEV)
    T = len(positions) + 1                                      # the last row belongs to no request
    from nanoinfer_b200.parts.base import Workspace
    ctx = SimpleNamespace(n_rows=T, workspace=Workspace(torch.device(DEV)),
                          row_entry=torch.tensor([0] * (T - 1) + [-1], dtype=torch.int32, device=DEV),
                          positions=torch.tensor(list(positions) + [0], dtype=torch.int32, device=DEV),
                          status=torch.zeros(1, dtype=torch.int32, device=DEV), host_entry_pos0=[], host_entry_start=[0])
    out = torch.full((T, H * kv_rank), 7.0, device=DEV, dtype=dtype)
    ops.latent_attention(q.to(DEV), cache[:, :, :, :, :], out, table.view(1, -1).to(DEV).contiguous(), ctx, H, kv_rank,
                         0.8, window, n_splits=n_splits)
    assert int(ctx.status) == 0 and (out[-1] == 7.0).all()
    ref, weight_on_hot = [], []
    for i, p in enumerate(positions):
        lo = max(0, p - window + 1) if window else 0
        keys = lat[lo:p + 1].double()
        s = torch.einsum("hd,jd->hj", q[i].double(), keys) * 0.8
        pr = torch.softmax(s, -1)
        ref.append((pr @ keys[:, :kv_rank]).reshape(-1))
        weight_on_hot.append(float(pr[:, hot[i] - lo].min()) if hot[i] is not None and lo <= hot[i] <= p else None)
    return out[:-1].double().cpu(), torch.stack(ref), weight_on_hot


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_splits", [1, 3, None])      # the keys whole, in three pieces, and as a step of few rows cuts them
@pytest.mark.parametrize("kv_rank,rot,page,window", [(32, 8, 16, 24), (20, 6, 16, 17), (80, 24, 32, 36), (40, 0, 16, 0),
                                                      (64, 16, 16, 1), (48, 16, 16, 100)])
def test_latent_attention_kernel_at_the_windows_edges(kv_rank, rot, page, window, n_splits, dtype):
    w = window or 1000
    positions = [0, 1, page - 1, page, w - 1, w, w + 1, 3 * page + 5, 130, 131]
    # a towering key just inside the window (the last one it keeps), just outside it, and at the row itself
    inside = [max(0, p - w + 1) for p in positions]
    got, ref, hot_w = _latent_case(DT[dtype], kv_rank, rot, page, window, positions, inside, n_splits)
    tol = 2e-5 if dtype == "float32" else 0.03
    assert float((got - ref).abs().max()) < tol
    if window != 1:
        assert min(x for x in hot_w if x is not None) > 0.5          # the edge key carries the row: losing it would show
    outside = [p - w if p - w >= 0 else None for p in positions]
    got, ref, _ = _latent_case(DT[dtype], kv_rank, rot, page, window, positions, outside, n_splits)
    assert float((got - ref).abs().max()) < tol                      # a key one behind the window must weigh nothing


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_prep_and_rotation_against_torch(dtype):
    from nanoinfer_b200.kernels import ops
    from plain_vadonex import rms_norm, rotate_pairs

    torch.manual_seed(2)
    dt, T, qr, kr, rd, dims, page, eps = DT[dtype], 6, 24, 20, 10, 6, 16, 1e-5
    proj = torch.randn(T, qr + kr + rd, device=DEV)
    wq, wkv = torch.rand(qr, device=DEV) + 0.5, torch.rand(kr, device=DEV) + 0.5
    freqs = (777.0 ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)).to(DEV)
    pos = [5, 6, 7, 1000, 15, 16]
    ent = [0, 0, 0, 1, -1, 2]
    table = torch.tensor([[3, -1] + [-1] * 62, [-1] * 62 + [1, -1], [2, 0] + [-1] * 62], dtype=torch.int32, device=DEV)
    cache = torch.zeros(5, 1, 1, page, kr + rd, device=DEV, dtype=dt)
    cq = torch.zeros(T, qr, device=DEV, dtype=dt)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.latent_prep(proj, qr, kr, rd, dims, freqs, wq, wkv, eps, cq, cache, table,
                    torch.tensor(ent, dtype=torch.int32, device=DEV), torch.tensor(pos, dtype=torch.int32, device=DEV), T, status)
    tol = 1e-5 if dtype == "float32" else 0.03
    assert int(status) == 0
    assert float((cq.double() - rms_norm(proj[:, :qr].double(), wq.double(), eps)).abs().max()) < tol
    c = rms_norm(proj[:, qr:qr + kr].double(), wkv.double(), eps)
    k_rot = rotate_pairs(proj[:, qr + kr:].double().cpu(), torch.tensor(pos), 777.0, dims).to(DEV)
    where = {0: (3, 5), 1: (3, 6), 2: (3, 7), 3: (1, 1000 % 16), 5: (0, 0)}
    for t, (pg, slot) in where.items():
        assert float((cache[pg, 0, 0, slot].double() - torch.cat([c[t], k_rot[t]])).abs().max()) < tol, t
    filled = torch.zeros(5, page, dtype=torch.bool)
    for pg, slot in where.values():
        filled[pg, slot] = True
    assert not cache[:, 0, 0][~filled.to(DEV)].any()                  # the row of no request wrote nothing
    # the queries' rotated part, behind the absorbed part of every head
    H, nope = 2, 4
    q = torch.randn(T, H * (nope + rd), device=DEV).to(dt)
    full = torch.zeros(T, H, kr + rd, device=DEV)
    ops.rope_heads(q, nope, rd, dims, freqs, torch.tensor(pos, dtype=torch.int32, device=DEV), full, kr, H, T)
    want = rotate_pairs(q.double().cpu().view(T, H, nope + rd)[..., nope:], torch.tensor(pos), 777.0, dims)
    assert float((full[..., kr:].double().cpu() - want).abs().max()) < 1e-5 and not full[..., :kr].any()


# =============================================================================== models through the step function
class Harness:
    def __init__(self, cfg, tmp_path, dtype, max_tokens=512, slots=4, page=16, max_rows=256, seed=1, sharpen=8.0,
                 long_memory=False):
        from nanoinfer_b200 import load_model
        from nanoinfer_b200.cache import CacheManager
        from nanoinfer_b200.engine import ModelRunner
        from plain_vadonex import PlainVadonex

        self.dir = write_model(cfg, str(tmp_path), DT[dtype], seed=seed, sharpen=sharpen, long_memory=long_memory)
        self.plain = PlainVadonex(self.dir)
        self.model = load_model(self.dir, DT[dtype], DEV)
        self.cache = CacheManager(self.model.kv_needs(), self.model.state_needs(), max_tokens=max_tokens,
                                  max_requests=slots, page_size=page, dtype=DT[dtype], device=torch.device(DEV),
                                  max_positions=None, padding=True)
        self.runner = ModelRunner(self.model, self.cache, max_rows=max_rows, max_entries=slots, check_status=True)
        self.dtype, self.vocab = dtype, cfg["vocab"]

    def alone(self, tokens, cuts):
        """One request cut into portions of the sizes in ``cuts`` (cycled), all logits back."""
        from nanoinfer_b200.engine import StepItem

        r, at, k, rows = self.cache.open_request(), 0, 0, []
        while at < len(tokens):
            n = min(cuts[k % len(cuts)], len(tokens) - at)
            rows.append(self.runner.step([StepItem(r, tokens[at:at + n], list(range(n)))]).clone())
            at, k = at + n, k + 1
        self.cache.close_request(r)
        return torch.cat(rows)

    def check(self, got, tokens, what=""):
        ref = self.plain.logits(tokens)
        ok = clear_rows(self.plain, self.dtype)
        assert int(ok.sum()) >= 0.5 * len(tokens), f"{what}: the test's weights make too many close calls"
        e = rel_err(got[ok.to(got.device)], ref[ok])
        assert e <= TOL[self.dtype], f"{what}: {e:.3e}"
        return e


ONE_LAYER = {
    "attention": [attention_layer()],
    "attention, one head, all keys": [attention_layer(heads=1, window=0, dim=8, vdim=24)],
    "attention, part of the rotated dims rotated": [attention_layer(rot_dim=12, rot_dims=8, base=50.0, kv_rank=24, window=9)],
    "attention, sizes no multiple of 8": [attention_layer(heads=3, dim=12, rot_dim=6, vdim=10, q_rank=20, kv_rank=28, window=21)],
    "delta rule": [delta_layer()],
    "delta rule, one head of 40": [delta_layer(heads=1, dim=40, decay_rank=3)],
    "dense feed-forward": [delta_layer(mlp=dense(72))],
    "routed feed-forward with a shared expert": [attention_layer(mlp=moe())],
    "routed, one expert a row, none shared": [delta_layer(mlp=moe(experts=5, top=1, shared=0))],
    "routed, every expert chosen": [delta_layer(mlp=moe(experts=3, top=3, ff=40, shared=8))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ONE_LAYER))
def test_each_mechanism_alone_as_a_one_layer_model(name, dtype, tmp_path):
    h = Harness(config(ONE_LAYER[name], vocab=150, width=48), tmp_path, dtype)
    t = toks(150, 75, 3)
    h.check(h.alone(t, [1000]), t, name)
    h.check(h.alone(t, [40, 1, 1, 2, 3, 1]), t, name + " in portions")


FULL = [delta_layer(heads=2, dim=24, mlp=dense(80)), attention_layer(window=24, mlp=moe()),
        attention_layer(window=24, mlp=None), attention_layer(kv_from=2, window=40, heads=3, dim=8, vdim=8, mlp=moe(experts=4, top=2, shared=0)),
        delta_layer(heads=4, dim=16, mlp=moe(experts=7, top=3, ff=16, shared=24)), attention_layer(kv_from=1, window=7, mlp=dense(40))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_token_by_token_and_portions_agree(dtype, tmp_path):
    h = Harness(config(FULL, vocab=190, width=64, alpha=2.2, eps=1e-6), tmp_path, dtype)
    t = toks(190, 97, 5)
    whole = h.alone(t, [1000])
    h.check(whole, t, "whole")
    ways = {"one by one": [1], "portions of two": [2], "3 and 5": [3, 5], "17, 16, 1, 31": [17, 16, 1, 31],
            "most of it, then single tokens": [60] + [1] * 40}
    for what, cuts in ways.items():
        got = h.alone(t, cuts)
        h.check(got, t, what)
        if dtype == "float32":     # how the prompt was cut shows in rounding only
            assert rel_err(got, whole) < 2e-5, what
    assert h.runner.graph_replays > 50            # single tokens ran as replayed graphs, state and all
    assert h.cache.pages_used() == [0] * len(h.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_together_equal_each_alone_and_pages_and_slots_come_back(dtype, tmp_path):
    from nanoinfer_b200.engine import StepItem

    h = Harness(config(FULL, vocab=170, width=64), tmp_path, dtype, max_tokens=4 * 64, slots=3)
    lens = [3, 120, 41, 64, 17, 88, 1]
    prompts = [toks(170, n, 20 + i) for i, n in enumerate(lens)]
    cuts = [[3], [50, 1, 1, 30, 2], [1, 40], [16, 16, 1], [17], [2, 2, 2, 80, 1], [1]]
    waiting, live, got = list(range(len(lens))), {}, {i: [] for i in range(len(lens))}
    slot_users, page_users, tick = {}, {}, 0
    while waiting or live:
        while waiting and len(live) < 3:
            i = waiting.pop(0)
            live[i] = [h.cache.open_request(), 0, 0]
            slot_users.setdefault(live[i][0].slot, set()).add(i)
        items, meta = [], []
        for j, (i, (req, at, k)) in enumerate(list(live.items())):
            if (tick + j) % 4 == 3 and len(live) > 1:
                continue                                   # sits this step out and goes on later
            n = min(cuts[i][k % len(cuts[i])], lens[i] - at)
            if not h.cache.can_append([(it.request, len(it.tokens)) for it in items] + [(req, n)]):
                continue
            items.append(StepItem(req, prompts[i][at:at + n], list(range(n))))
            meta.append((i, n))
        tick += 1
        if not items:
            continue
        out = h.runner.step(items)
        row = 0
        for i, n in meta:
            got[i].append(out[row:row + n].clone())
            row += n
            live[i][1] += n
            live[i][2] += 1
            for g, blocks in enumerate(live[i][0].blocks):
                for p in blocks:
                    if p >= 0:
                        page_users.setdefault((g, p), set()).add(i)
            if live[i][1] == lens[i]:
                h.cache.close_request(live[i][0])
                del live[i]
        h.cache.check()
    for i, t in enumerate(prompts):
        h.check(torch.cat(got[i]), t, f"request {i}")
    assert max(len(u) for u in slot_users.values()) >= 2 and max(len(u) for u in page_users.values()) >= 2
    assert h.cache.pages_used() == [0] * len(h.cache.groups) and h.cache.slots.n_free == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lengths_around_page_and_window_edges(dtype, tmp_path):
    layers = [attention_layer(window=24, mlp=None), delta_layer(mlp=None), attention_layer(kv_from=0, window=17, mlp=None)]
    h = Harness(config(layers, vocab=120, width=40), tmp_path, dtype, sharpen=12.0)
    for n in (1, 2, 15, 16, 17, 18, 23, 24, 25, 26, 32, 33, 41, 48, 49):
        t = toks(120, n + 3, n)
        h.check(h.alone(t, [n, 1, 1, 1]), t, f"{n} tokens, then three alone")
        h.check(h.alone(t, [1, 1, 1, n]), t, f"three alone, then {n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_hands_pages_back_behind_the_window(dtype, tmp_path):
    from nanoinfer_b200.engine import StepItem

    layers = [delta_layer(mlp=dense()), attention_layer(window=24, mlp=moe()), attention_layer(kv_from=1, window=24)]
    h = Harness(config(layers, vocab=100, width=48), tmp_path, dtype, max_tokens=64, slots=2)
    t = toks(100, 330, 9)
    r = h.cache.open_request()
    rows = [h.runner.step([StepItem(r, t[:5], list(range(5)))]).clone()]
    for p in range(5, len(t)):                    # 330 positions through a pool of 4 pages
        rows.append(h.runner.step([StepItem(r, t[p:p + 1], [0])]).clone())
        assert h.cache.pages_used()[0] <= 3
    h.cache.close_request(r)
    h.check(torch.cat(rows), t, "330 positions")
    assert h.runner.graph_replays > 300


def test_a_token_far_back_shows_through_the_state(tmp_path):
    """The decays of the test weights let some channels remember for hundreds of tokens: two prompts that
    differ in their first token only still differ 120 tokens on, and the engine follows the plain model in both."""
    h = Harness(config([delta_layer(heads=2, dim=32, mlp=None)], vocab=90, width=64), tmp_path, "float32",
                long_memory=True)
    a = toks(90, 120, 4)
    b = [(a[0] + 1) % 90] + a[1:]
    la, lb = h.plain.logits(a)[-1], h.plain.logits(b)[-1]
    assert rel_err(la[None], lb[None]) > 10 * TOL["float32"]
    for t in (a, b):
        h.check(h.alone(t, [90, 7, 1]), t)


def random_config(rnd):
    width = rnd.choice([32, 40, 64, 72, 96, 100])
    layers = []
    for i in range(rnd.randint(1, 5)):
        mlp = rnd.choice([None, dense(rnd.choice([24, 50, 64])),
                          moe(experts=rnd.choice([2, 5, 8]), top=rnd.choice([1, 2]), ff=rnd.choice([8, 20, 32]),
                              shared=rnd.choice([0, 12, 32]))])
        owners = [j for j, l in enumerate(layers) if l["type"] == "latent_attention" and "kv_from" not in l["mixer"]]
        if rnd.random() < 0.4:
            layers.append(delta_layer(heads=rnd.choice([1, 2, 3]), dim=rnd.choice([8, 16, 20, 32, 48]),
                                      decay_rank=rnd.choice([1, 4, 8, 16]), mlp=mlp))
        elif owners and rnd.random() < 0.5:
            src = rnd.choice(owners)
            o = layers[src]["mixer"]
            layers.append(attention_layer(heads=rnd.choice([1, 2, 4]), dim=rnd.choice([4, 8, 16]), rot_dim=o["rot_dim"],
                                          vdim=rnd.choice([8, 12, 16]), q_rank=rnd.choice([8, 16, 24]), kv_rank=o["kv_rank"],
                                          window=rnd.choice([0, 1, 5, 16, 33, 64]), rot_dims=o["rot"]["dims"],
                                          base=o["rot"]["base"], kv_from=src, scale=rnd.choice([0.1, 0.25, 0.4]), mlp=mlp))
        else:
            rd = rnd.choice([0, 4, 8, 16])
            layers.append(attention_layer(heads=rnd.choice([1, 2, 3, 5]), dim=rnd.choice([4, 8, 12, 16, 32]), rot_dim=rd,
                                          vdim=rnd.choice([4, 8, 16, 24]), q_rank=rnd.choice([8, 12, 32]),
                                          kv_rank=rnd.choice([8, 16, 20, 32, 48, 72]), window=rnd.choice([0, 2, 16, 24, 50]),
                                          rot_dims=rnd.choice([rd, rd // 4 * 2 if rd >= 8 else rd]),
                                          base=rnd.choice([10.0, 10000.0, 500000.0]), scale=rnd.choice([0.1, 0.25, 0.4]), mlp=mlp))
    return config(layers, vocab=rnd.choice([97, 256, 1001]), width=width, alpha=rnd.choice([1.0, 1.5, 2.5, 3.0]),
                  eps=rnd.choice([1e-6, 1e-5, 3e-4]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", range(12))
def test_random_configuration_cut_at_random(case, dtype, tmp_path):
    from nanoinfer_b200.engine import StepItem

    rnd = random.Random(4200 + case)
    cfg = random_config(rnd)
    page = rnd.choice([16, 32, 48])
    lens = [rnd.randint(1, 150) for _ in range(rnd.randint(2, 6))]
    pages_of = lambda n: -(-n // page)
    pages = max(max(pages_of(n) for n in lens) + 2, int(0.6 * sum(pages_of(n) for n in lens)))
    h = Harness(cfg, tmp_path, dtype, max_tokens=pages * page, slots=3, page=page, max_rows=rnd.choice([64, 160]),
                seed=case + 1, sharpen=rnd.choice([4.0, 8.0]))
    prompts = [[rnd.randrange(cfg["vocab"]) for _ in range(n)] for n in lens]
    want, clear = [], []
    for t in prompts:
        want.append(h.plain.logits(t))
        clear.append(clear_rows(h.plain, dtype))
    pending, live, got = list(range(len(lens))), {}, {}
    while pending or live:
        while pending and len(live) < 3:
            live[pending.pop(0)] = [h.cache.open_request(), 0]
        items, meta, rows = [], [], 0
        for i, (req, at) in list(live.items()):
            if rnd.random() < 0.2 and len(live) > 1:
                continue
            n = min(lens[i] - at, rnd.choice([1, 1, 2, 3, 7, 16, 17, 33, 64, 100]), h.runner.max_rows - rows)
            if n <= 0 or not h.cache.can_append([(it.request, len(it.tokens)) for it in items] + [(req, n)]):
                continue
            places = sorted(rnd.sample(range(n), min(n, rnd.randint(0, 3))))
            items.append(StepItem(req, prompts[i][at:at + n], places))
            meta.append((i, at, n, places))
            rows += n
        if not items:
            # nothing fits beside what is held: the newest request gives way and starts again later
            i = max(live)
            h.cache.close_request(live.pop(i)[0])
            pending.insert(0, i)
            got = {k: v for k, v in got.items() if k[0] != i}
            continue
        out = h.runner.step(items)
        k = 0
        for i, at, n, places in meta:
            for j in places:
                got[(i, at + j)] = out[k].clone()
                k += 1
            live[i][1] = at + n
            if at + n == lens[i]:
                h.cache.close_request(live.pop(i)[0])
    h.cache.check()
    assert got and h.cache.pages_used() == [0] * len(h.cache.groups)
    compared = 0
    for (i, p), row in got.items():
        if not clear[i][p]:
            continue                        # (bfloat16 only) at or behind a router's close call
        compared += 1
        e = rel_err(row[None], want[i][p][None])
        assert e <= TOL[dtype], f"case {case} {json.dumps(cfg)}: request {i}, position {p}: {e:.3e}"
    assert compared >= 0.5 * len(got)


def test_greedy_generation_through_the_engine_and_its_scheduler(tmp_path):
    import nanoinfer_b200 as nb

    cfg = config(FULL, vocab=130, width=64)
    d = write_model(cfg, str(tmp_path), torch.float32, seed=3)
    from plain_vadonex import PlainVadonex
    plain = PlainVadonex(d)
    prompts = [toks(130, n, 40 + n) for n in (1, 9, 30, 55, 17)]
    eng = nb.Engine(d, dtype="float32", max_tokens=3 * 128, max_batch=3, max_rows=64)
    outs = eng.generate(prompts, nb.SamplingParams(max_new_tokens=20))
    for p, o in zip(prompts, outs):
        assert o == plain.greedy(p, 20)
    assert eng.runner.graph_replays > 0 and eng.cache.pages_used() == [0] * len(eng.cache.groups)


def test_trace_replay_of_a_model_folder(tmp_path):
    from trace_util import TraceSession

    cfg = config(FULL[:4], vocab=110, width=48)
    d = write_model(cfg, str(tmp_path / "m"), torch.float32, seed=8)
    from plain_vadonex import PlainVadonex
    plain = PlainVadonex(d)
    reqs = {f"r{i}": toks(110, n, 60 + i) for i, n in enumerate((50, 3, 64, 20, 33, 9))}
    s = TraceSession(d, "float32", tmp_path / "out", 4 * 64, 110)
    order, live, at = list(reqs), [], {r: 0 for r in reqs}
    k = 0
    while order or live:
        while order and len(live) < 4:
            live.append(order.pop(0))
        entries, ended = [], []
        for r in list(live):
            n = min([7, 1, 20, 2][k % 4], len(reqs[r]) - at[r])
            k += 1
            entries.append((r, reqs[r][at[r]:at[r] + n], range(n)))
            at[r] += n
            if at[r] == len(reqs[r]):
                ended.append(r)
                live.remove(r)
        s.step(entries, end=ended)
    s.close()
    for r, t in reqs.items():
        assert rel_err(s.stacked(r, len(t)), plain.logits(t)) <= TOL["float32"], r


def test_command_line_writes_a_folder_generates_from_it_and_profiles(tmp_path, capsys):
    """The command line as for the other architecture: random-weights from the preset, generate (the tokens
    of the entry point, which are the plain model's), and the per-op profile of a prefill and a decode step."""
    import nanoinfer_b200 as nb
    from nanoinfer_b200 import cli
    from plain_vadonex import PlainVadonex

    d = str(tmp_path / "m")
    assert cli.main(["random-weights", "--config", "vadonex-tiny", "--seed", "6", "--out", d, "--dtype", "float32"]) == 0
    capsys.readouterr()
    prompt = toks(512, 12, 77)
    assert cli.main(["--weights", d, "generate", "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
                     "--tokens", "10", "--temperature", "0.0", "--profile"]) == 0
    captured = capsys.readouterr()
    printed = [int(t) for t in captured.out.split()]
    assert printed == PlainVadonex(d).greedy(prompt, 10)
    assert "delta_rule" in captured.err and "attn" in captured.err and "experts_up" in captured.err
