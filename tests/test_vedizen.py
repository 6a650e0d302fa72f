"""The Vedizen decoder in the engine against the plain implementation (tests/plain_vedizen.py): each mechanism's
kernels alone, then whole models of several small shapes through the step function, the scheduler and the
replay tool: whole prompts, token-by-token decoding, portions down to two tokens, unequal batches, slots and
pages used again, chunk edges, far keys and long decoding."""
from __future__ import annotations

import math
import random

import numpy as np
import pytest
import torch

import plain_vedizen as P
from helpers import Replay, assert_close, bf16_noise, random_tokens

F64 = torch.float64


# ----------------------------------------------------------------------------- small shapes
def shape_s1() -> dict:
    """Odd sizes everywhere: a width no tensor-core product takes, key rows (2*16) unlike value rows (24), a layer
    without a feed-forward, a loop in the middle of the stack run twice, chunks of 37 and 11 positions."""
    return P.make_config(vocab=160, width=100, scale=1.7, eps=3e-5, loop=(1, 3, 2), layers=[
        P.attention_layer(6, 3, 16, 24, chunk=37, ff=72, limit=1.2, diff=0.35),
        P.gla_layer(3, 24, 40, tau=7.0),
        P.attention_layer(2, 2, 8, 16, chunk=11, softcap=5.0, diff=0.6, ff=56, limit=0.8),
        P.gla_layer(2, 40, 16, tau=2.5, ff=88, limit=2.5)])


def shape_s2() -> dict:
    """Sizes the tensor-core products take in bfloat16 (multiples of 16), no loop at all, one KV head."""
    return P.make_config(vocab=192, width=128, scale=0.8, layers=[
        P.gla_layer(2, 32, 64, tau=12.0, ff=160, limit=2.0),
        P.attention_layer(4, 1, 16, 48, chunk=64, softcap=30.0, diff=0.2, ff=96, limit=1.0),
        P.attention_layer(2, 2, 32, 32, chunk=24, softcap=50.0, diff=0.5)])


SHAPES = {"s1": (shape_s1, 8, 6), "s2": (shape_s2, 16, 16)}        # name -> (config, page size, decay rank)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (make, page, rank) in SHAPES.items():
        cfg = make()
        W = P.random_weights(cfg, seed=len(name) * 7 + 1, rank=rank)
        out[name] = (P.write_folder(str(tmp_path_factory.mktemp(name)), cfg, W), cfg, W, page)
    return out


def engine(folder, dtype, page, tokens=512, batch=256, reqs=4):
    import airun_b200
    return airun_b200.Engine.from_folder(folder, dtype=dtype, page_size=page, cache_tokens=tokens, max_batch_tokens=batch,
                                         max_requests=reqs, max_context=tokens)


def run_schedule(eng, seqs, schedule):
    """schedule: steps, each a list of (request index, tokens to take); wants every token's logits.  Returns
    {request: [T, vocab]} and frees a request when its tokens are used up."""
    from airun_b200 import StepEntry
    at = {i: 0 for i in range(len(seqs))}
    got = {i: [] for i in range(len(seqs))}
    for step in schedule:
        entries = []
        for i, n in step:
            if at[i] == 0:
                eng.manager.add_request(f"q{i}")
            entries.append(StepEntry(f"q{i}", seqs[i][at[i]:at[i] + n], tuple(range(n))))
        out = eng.runner.step(entries).cpu().numpy()
        eng.runner.raise_on_device_error()
        row = 0
        for i, n in step:
            got[i].append(out[row:row + n])
            row += n
            at[i] += n
            if at[i] == len(seqs[i]):
                eng.manager.free_request(f"q{i}")
    eng.manager.check_invariants()
    return {i: np.concatenate(v) for i, v in got.items() if v}


def expect(cfg, W, seq, dtype):
    exact = P.plain_forward(cfg, W, seq).numpy()
    if dtype == "float32":
        return exact, None
    rounded = P.plain_forward(cfg, W, seq, rnd=P.to_bf16_and_back).numpy()
    return rounded, bf16_noise(rounded, exact)


def compare(got, cfg, W, seq, dtype, what):
    want, noise = expect(cfg, W, seq, dtype)
    assert_close(got, want.astype(np.float32), dtype, what, noise)


# ----------------------------------------------------------------------------- without a GPU
def test_config_reads_sizes_order_and_rank():
    from airun_b200.config import VedizenConfig, architecture_name, lookup_architecture
    d = shape_s1()
    assert architecture_name(d) == "Vedizen" and lookup_architecture("Vedizen")[0] is VedizenConfig
    c = VedizenConfig.from_dict(d)
    assert (c.vocab_size, c.hidden_size, c.embedding_scale, c.norm_eps) == (160, 100, 1.7, 3e-5)
    order = c.execution_order()
    assert [(o.layer, o.add_row) for o in order] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert c.order_table() == ("loop.step", 2)
    c2 = c.with_tensor_shapes({"l1.mix.a1": (6, 100), "l3.mix.a1": (9, 100)})
    assert c2.decay_ranks == (0, 6, 0, 9)
    assert [s.mixer_args.get("decay_rank") for s in c2.layer_specs()] == [None, 6, None, 9]
    assert VedizenConfig.from_dict(c2.to_dict()).to_dict() == c2.to_dict()
    specs = c.layer_specs()
    assert specs[1].feed_forward == "" and specs[0].feed_forward == "clamped_glu" and specs[0].arrangement == "parallel"
    assert specs[2].mixer_args["chunk"] == 11 and specs[2].mixer_args["soft_cap"] == 5.0
    nol = VedizenConfig.from_dict(shape_s2())
    assert nol.order_table() is None and [o.layer for o in nol.execution_order()] == [0, 1, 2]


def test_config_lists_every_problem():
    from airun_b200.config import ConfigError, VedizenConfig
    d = shape_s1()
    d["layers"][0]["mixer"]["kv_heads"] = 4
    d["layers"][1]["mixer"]["tau"] = 0
    d["loop"] = dict(start=3, stop=2, times=1)
    with pytest.raises(ConfigError) as e:
        VedizenConfig.from_dict(d)
    for text in ("multiple of kv_heads", "tau", "loop"):
        assert text in str(e.value)


def test_declared_tensors_are_the_files_tensors():
    from airun_b200.config import VedizenConfig
    from airun_b200.engine.model import DecoderModel
    for make, _, rank in SHAPES.values():
        cfg = make()
        shapes = P.tensor_shapes(cfg, rank)
        c = VedizenConfig.from_dict(cfg).with_tensor_shapes(shapes)
        specs = {s.name: tuple(s.shape) for s in DecoderModel(c, torch.float32, "cpu").weight_specs()}
        assert specs == {n: tuple(s) for n, s in shapes.items()}


def test_cache_groups_keep_value_rows_of_their_own_size():
    from airun_b200.cache.manager import CacheManager
    from airun_b200.config import VedizenConfig
    from airun_b200.engine.model import DecoderModel
    from airun_b200.parts.base import PagedKVSpec, StateSpec
    m = DecoderModel(VedizenConfig.from_dict(shape_s1()), torch.float32, "cpu")
    specs, src = m.cache_specs()
    assert specs[0] == PagedKVSpec(3, 32, 0, value_dim=24) and specs[2] == PagedKVSpec(2, 16, 0, value_dim=0)
    assert specs[1] == StateSpec((3, 24, 40), torch.float32) and specs[1] == specs[3] and specs[5] == StateSpec((2, 40, 16), torch.float32)
    mgr = CacheManager(specs, src, page_size=8, num_pages=16, max_requests=4)
    assert [b.kind for b in mgr.bindings] == ["paged", "state", "paged", "state", "paged", "state"]
    assert len(mgr.paged) == 2 and len(mgr.state) == 2 and mgr.bindings[3].index == 1      # each pass has its own state


def test_plain_recurrence_equals_its_closed_form():
    g = torch.Generator().manual_seed(3)
    T, Hh, D, Dv = 23, 2, 5, 3
    q, k = torch.randn(T, Hh, D, generator=g, dtype=F64), torch.randn(T, Hh, D, generator=g, dtype=F64)
    v, a = torch.randn(T, Hh, Dv, generator=g, dtype=F64), torch.rand(T, Hh, D, generator=g, dtype=F64) * 0.6 + 0.4
    o, S = P.plain_gla_recurrence(q, k, v, a)
    assert torch.allclose(o, P.plain_gla_closed_form(q, k, v, a), atol=1e-12)
    o2, _ = P.plain_gla_recurrence(q[9:], k[9:], v[9:], a[9:], state=P.plain_gla_recurrence(q[:9], k[:9], v[:9], a[:9])[1])
    assert torch.allclose(o[9:], o2, atol=1e-12)


def test_plain_mask_counts_chunks_from_position_zero():
    vis = P.plain_visible(6, chunk=4, first=2)           # positions 2..7: 2, 3 | 4, 5, 6, 7
    assert vis.int().tolist() == [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [0, 0, 1, 0, 0, 0], [0, 0, 1, 1, 0, 0],
                                  [0, 0, 1, 1, 1, 0], [0, 0, 1, 1, 1, 1]]


# ----------------------------------------------------------------------------- kernels alone
gpu = pytest.mark.gpu


def dev(t, dtype=torch.float32):
    return t.to("cuda", dtype).contiguous()


@gpu
def test_dyt_norm_kernel_with_delta_row_offset_and_gather():
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    T, n = 9, 70
    x, d, vec = torch.randn(T, n, generator=g) * 3, torch.randn(T, n, generator=g), torch.randn(n, generator=g)
    w, b, alpha = torch.randn(n, generator=g), torch.randn(n, generator=g), torch.tensor([0.37])
    xd, out = dev(x), torch.empty(T, n, device="cuda")
    ops.dyt_norm(xd, dev(alpha), dev(w), dev(b), out, delta=dev(d), add_vec=dev(vec))
    s = x.double() + d.double() + vec.double()
    assert torch.allclose(xd.cpu().double(), s, atol=1e-6)                      # the sum became the residual
    assert torch.allclose(out.cpu().double(), P.plain_dyt(s, w.double(), b.double(), alpha.double()), atol=2e-6)
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    xd2, out2 = dev(x), torch.empty(3, n, device="cuda", dtype=torch.bfloat16)
    ops.dyt_norm(xd2, dev(alpha), dev(w), dev(b), out2, delta=dev(d), rows=rows)
    assert torch.equal(xd2.cpu(), x)                                            # a gathered norm leaves x alone
    want = P.plain_dyt((x + d)[[7, 0, 3]].double(), w.double(), b.double(), alpha.double())
    assert torch.allclose(out2.cpu().double(), want, atol=2e-2, rtol=1e-2)


@gpu
def test_clamped_gated_unit_kernel_into_a_column_slice():
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    T, I, group = 5, 48, 16
    gate, up = torch.randn(T, I, generator=g) * 3, torch.randn(T, I, generator=g) * 3
    gu = torch.stack([gate.view(T, I // group, group), up.view(T, I // group, group)], dim=2).reshape(T, 2 * I)
    buf = torch.full((T, I + 10), 9.0, device="cuda")
    ops.glu_clamped(dev(gu), buf[:, 10:], group, limit=1.5, slope=1.702)
    gg, uu = gate.double().clamp(max=1.5), up.double().clamp(-1.5, 1.5)
    assert torch.allclose(buf[:, 10:].cpu().double(), gg * torch.sigmoid(1.702 * gg) * (uu + 1), atol=1e-5)
    assert (buf[:, :10] == 9.0).all()


@gpu
@pytest.mark.parametrize("heads,D,Dv", [(3, 24, 40), (2, 130, 33), (1, 8, 8), (2, 64, 96)])
def test_gla_kernels_carry_state_across_steps_and_requests(heads, D, Dv):
    """Three requests of unequal length in one batch, each cut in two steps at another place, slots out of order."""
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(heads * 100 + D)
    lens, cuts, slots = [13, 1, 37], [5, 0, 36], [2, 0, 3]
    rank, tau, eps = 5, 3.0, 1e-5
    data = []
    for n in lens:
        data.append(dict(q=torch.randn(n, heads * D, generator=g), k=torch.randn(n, heads * D, generator=g) * 0.5,
                         v=torch.randn(n, heads * Dv, generator=g), gate=torch.randn(n, heads * Dv, generator=g),
                         low=torch.randn(n, rank, generator=g)))
    w2, b2, wn = torch.randn(heads * D, rank, generator=g), torch.randn(heads * D, generator=g) + 2.0, torch.randn(Dv, generator=g)
    state = torch.zeros(4, heads, D, Dv, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = [[] for _ in lens]
    for part in (0, 1):
        spans = [(0, c) if part == 0 else (c, n) for n, c in zip(lens, cuts)]
        rows = [i for i, (a, b) in enumerate(spans) if b > a]
        cat = lambda key: torch.cat([data[i][key][spans[i][0]:spans[i][1]] for i in rows])
        width = 2 * heads * D + 2 * heads * Dv + rank
        proj = dev(torch.cat([cat("q"), cat("k"), cat("v"), cat("gate"), cat("low")], dim=1))
        T = proj.shape[0]
        kd, vd = heads * D, heads * Dv
        cu = torch.tensor(np.cumsum([0] + [spans[i][1] - spans[i][0] for i in rows]), dtype=torch.int32, device="cuda")
        req = torch.repeat_interleave(torch.arange(len(rows), dtype=torch.int32), (cu[1:] - cu[:-1]).cpu()).to("cuda", torch.int32)
        sl = torch.tensor([slots[i] for i in rows], dtype=torch.int32, device="cuda")
        logd = torch.empty(T, kd, device="cuda")
        ops.gla_decay(proj[:, 2 * kd + 2 * vd:], dev(w2), dev(b2), tau, logd, req)
        o = torch.empty(T, vd, device="cuda")
        ops.gla_recurrent(proj[:, :kd], proj[:, kd:2 * kd], proj[:, 2 * kd:2 * kd + vd], logd, state, cu, sl, len(rows), o,
                          heads, D, Dv, D ** -0.5, err)
        act = torch.empty(T, vd + 3, device="cuda")
        ops.gla_out_gate(o, proj[:, 2 * kd + vd:2 * kd + 2 * vd], dev(wn), eps, act[:, 3:], heads, Dv, req)
        for j, i in enumerate(rows):
            got[i].append(act[cu[j]:cu[j + 1], 3:].cpu())
    assert int(err.item()) == 0
    for i, n in enumerate(lens):
        d = {k: t.double() for k, t in data[i].items()}
        a = torch.exp(torch.nn.functional.logsigmoid(d["low"] @ w2.double().T + b2.double()) / tau).view(n, heads, D)
        o, S = P.plain_gla_recurrence(d["q"].view(n, heads, D) * D ** -0.5, d["k"].view(n, heads, D), d["v"].view(n, heads, Dv), a)
        want = (P.plain_rms_unit(o, eps) * wn.double()).reshape(n, -1) * (d["gate"] * torch.sigmoid(d["gate"]))
        assert torch.allclose(torch.cat(got[i]).double(), want, atol=2e-4, rtol=2e-4), f"request {i}"
        assert torch.allclose(state[slots[i]].cpu().double(), S, atol=2e-4, rtol=2e-4)
    assert (state[1] == 0).all()                                   # a slot nobody used stays as it was


@gpu
def test_gla_remembers_a_token_from_far_back():
    """Decays a hair below one: what token 0 wrote must still be read 700 tokens on, decoded one at a time."""
    from airun_b200.kernels import ops
    heads, D, Dv, n = 1, 16, 32, 700
    q, k, v = torch.zeros(n, D), torch.zeros(n, D), torch.zeros(n, Dv)
    k[0, 3], v[0] = 4.0, torch.arange(Dv) - 10.0
    q[:, 3] = 1.0
    k[1:, 5], v[1:, 0] = 0.01, 1.0                                  # later tokens write elsewhere
    logd = torch.full((n, D), 0.9995)
    state = torch.zeros(1, heads, D, Dv, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    cu, sl = torch.tensor([0, 1], dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
    proj, o = dev(torch.cat([q, k, v], 1)), torch.empty(1, Dv, device="cuda")
    for t in range(n):
        row = proj[t:t + 1]
        ops.gla_recurrent(row[:, :D], row[:, D:2 * D], row[:, 2 * D:], dev(logd[t:t + 1]), state, cu, sl, 1, o, heads, D, Dv, 1.0, err)
    want = 4.0 * 0.9995 ** (n - 1) * v[0].double()
    assert torch.allclose(o[0].cpu().double(), want, rtol=1e-3, atol=1e-3)


def paged_attention_case(seq_lens, new_lens, heads, kvh, D, Dv, chunk, page, dtype, seed, spike=None, bias=0.2):
    """Fills a paged cache through the store kernel (pages handed out in a scrambled order) with the first
    len - new tokens of every request, then runs the last ``new`` tokens of each as one batch."""
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    kd, qw = 2 * D, heads * 2 * D
    width = qw + kvh * (kd + Dv)
    reqs = []
    for n in seq_lens:
        proj = torch.randn(n, width, generator=g)
        if spike is not None:
            spike(proj, n)
        reqs.append(proj)
    bq, bk, bv = (torch.randn(w, generator=g) * bias for w in (qw, kvh * kd, kvh * Dv))
    blocks = [(n + page - 1) // page for n in seq_lens]
    num_pages = sum(blocks) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    bt = torch.full((len(seq_lens), max(blocks)), -1, dtype=torch.int32)
    for r, nb in enumerate(blocks):
        for b in range(nb):
            bt[r, b] = perm.pop()
    pool = torch.zeros(num_pages, page * kvh * (kd + Dv), device="cuda", dtype=dtype)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    btd = bt.cuda()
    outs = []
    for phase in (0, 1):
        spans = [(0, n - m) if phase == 0 else (n - m, n) for n, m in zip(seq_lens, new_lens)]
        rows = [r for r, (a, b) in enumerate(spans) if b > a]
        if not rows:
            continue
        proj = dev(torch.cat([reqs[r][spans[r][0]:spans[r][1]] for r in rows]))
        pos = torch.cat([torch.arange(*spans[r]) for r in rows]).to("cuda", torch.int32)
        req = torch.cat([torch.full((spans[r][1] - spans[r][0],), r) for r in rows]).to("cuda", torch.int32)
        q = torch.empty(proj.shape[0], qw, device="cuda", dtype=dtype)
        ops.qkv_bias_store(proj, dev(bq), dev(bk), dev(bv), q, pool, btd, pos, req, len(seq_lens), page, qw, kvh, kd, Dv, err)
        outs.append((rows, spans, q, pos, req))
    return dict(reqs=reqs, bq=bq, bk=bk, bv=bv, pool=pool, bt=btd, err=err, last=outs[-1], page=page)


def plain_attention_rows(case, r, heads, kvh, D, Dv, scale, cap, lam, chunk, eps, out_scale, rnd=None):
    proj = case["reqs"][r].double()
    n, qw, kd = proj.shape[0], heads * 2 * D, 2 * D
    rr = (lambda t: t) if rnd is None else rnd
    q = rr(proj[:, :qw] + case["bq"].double()).view(n, heads, 2, D)
    k = rr(proj[:, qw:qw + kvh * kd] + case["bk"].double()).view(n, kvh, 2, D)
    v = rr(proj[:, qw + kvh * kd:] + case["bv"].double()).view(n, kvh, Dv)
    vis = P.plain_visible(n, chunk)
    out = torch.zeros(n, heads, Dv, dtype=F64)
    for h in range(heads):
        gi, maps = h // (heads // kvh), []
        for m in range(2):
            s = (q[:, h, m] @ k[:, gi, m].T) * scale
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            maps.append(torch.softmax(s.masked_fill(~vis, -math.inf), -1) @ v[:, gi])
        out[:, h] = P.plain_rms_unit(maps[0] - lam * maps[1], eps) * out_scale
    return out.reshape(n, heads * Dv)


@gpu
@pytest.mark.parametrize("heads,kvh,D,Dv,chunk,page", [(6, 3, 16, 24, 37, 8), (2, 2, 8, 16, 11, 16), (4, 1, 40, 72, 0, 24),
                                                         (3, 1, 130, 200, 50, 16)])
def test_differential_attention_kernel_over_scrambled_pages(heads, kvh, D, Dv, chunk, page):
    from airun_b200.kernels import ops
    lens, new = [75, 9, 41, 1], [75, 1, 5, 1]          # a whole prompt, single tokens, a short portion
    scale, cap, lam, eps, osc = D ** -0.5, 6.0, 0.45, 1e-5, 0.7
    case = paged_attention_case(lens, new, heads, kvh, D, Dv, chunk, page, torch.float32, seed=heads + D)
    rows, spans, q, pos, req = case["last"]
    out = torch.empty(q.shape[0], heads * Dv + 5, device="cuda")
    ops.diff_attention(q, out[:, 5:], case["pool"], case["bt"], pos, req, len(lens), page, heads, kvh, D, Dv, scale, cap,
                       chunk, 0, lam, eps, osc, case["err"])
    assert int(case["err"].item()) == 0
    at = 0
    for r in rows:
        a, b = spans[r]
        want = plain_attention_rows(case, r, heads, kvh, D, Dv, scale, cap, lam, chunk, eps, osc)[a:b]
        assert torch.allclose(out[at:at + b - a, 5:].cpu().double(), want, atol=3e-5, rtol=1e-4), f"request {r}"
        at += b - a


def tensor_core_attention(case, lens, new, heads, kvh, D, Dv, scale, cap, lam, chunk, eps, osc):
    """The batch of ``paged_attention_case`` through the tensor-core kernel; returns [rows, heads*Dv] float64."""
    from types import SimpleNamespace as NS
    from airun_b200.kernels import fast
    rows, spans, q, pos, req = case["last"]
    counts = [spans[r][1] - spans[r][0] if r in rows else 0 for r in range(len(lens))]
    ctx = NS(cu_tokens=torch.tensor(np.cumsum([0] + counts), dtype=torch.int32, device="cuda"),
             context_lens=torch.tensor(lens, dtype=torch.int32, device="cuda"), num_reqs=len(lens), err=case["err"])
    part = NS(D=D, Dv=Dv, nh=heads, nkv=kvh, scale=scale, cap=cap, chunk=chunk, window=0, lam=lam, eps=eps, lambda_init=1.0 - osc)
    cache = NS(pool=case["pool"], block_table=case["bt"], page_size=case["page"])
    out = torch.full((q.shape[0], heads * Dv + 8), 7.0, device="cuda", dtype=torch.bfloat16)
    assert fast.diff_attention_bf16(ctx, q, out[:, 8:], cache, part)
    assert (out[:, :8] == 7.0).all()
    return out[:, 8:].cpu().double()


@gpu
@pytest.mark.parametrize("heads,kvh,D,Dv,chunk,page", [(6, 3, 16, 24, 37, 8), (2, 2, 8, 16, 11, 16), (4, 1, 40, 72, 0, 24),
                                                         (3, 1, 128, 128, 50, 16), (4, 2, 64, 128, 100, 16), (2, 1, 20, 36, 64, 16)])
@pytest.mark.parametrize("single_tokens", ["head rows", "tiles"])
def test_tensor_core_differential_attention_against_the_plain_formula(heads, kvh, D, Dv, chunk, page, single_tokens, monkeypatch):
    """``single_tokens``: which kernel takes the requests that bring one token: the one whose product rows are the heads
    of a KV head, or (that one switched off) the tile kernel like any portion."""
    from airun_b200.kernels import fast
    if single_tokens == "tiles":
        monkeypatch.setattr(fast, "DISABLED", set(fast.DISABLED) | {"diff_group"})
    lens, new = [150, 9, 77, 1, 64], [150, 1, 5, 1, 64]     # whole prompts (three and one tile), single tokens, a portion
    scale, cap, lam, eps, osc = D ** -0.5, 6.0, 0.45, 1e-5, 0.7
    case = paged_attention_case(lens, new, heads, kvh, D, Dv, chunk, page, torch.bfloat16, seed=heads + D)
    got = tensor_core_attention(case, lens, new, heads, kvh, D, Dv, scale, cap, lam, chunk, eps, osc)
    assert int(case["err"].item()) == 0
    rows, spans = case["last"][0], case["last"][1]
    at = 0
    for r in rows:
        a, b = spans[r]
        want = plain_attention_rows(case, r, heads, kvh, D, Dv, scale, cap, lam, chunk, eps, osc, rnd=P.to_bf16_and_back)[a:b]
        err = (got[at:at + b - a] - want).abs()
        assert float(err.max()) < 4e-2 and float(err.mean()) < 4e-3, f"request {r}: {float(err.max())}, {float(err.mean())}"
        at += b - a


@gpu
@pytest.mark.parametrize("where", ["inside", "outside", "far"])
def test_one_dominant_key_at_a_chunk_edge(where):
    """A query whose score with ONE key stands out: the first key of its chunk (seen), the last key of the chunk
    before (not seen), or the first key of a long chunk hundreds of keys back (seen)."""
    from airun_b200.kernels import ops
    heads, kvh, D, Dv, page = 2, 1, 16, 24, 16
    chunk, n = (32, 70) if where != "far" else (512, 500)
    target = {"inside": 64, "outside": 63, "far": 0}[where]
    qw = heads * 2 * D

    def spike(proj, n_):
        proj[n_ - 1, :qw] = 0.0
        proj[n_ - 1, 0:D] = 3.0                         # map 1 of head 0 of the last token
        proj[:, qw:qw + 2 * D] *= 0.05
        proj[target, qw:qw + D] = 3.0                   # map-1 key of the target

    for dtype in (torch.float32, torch.bfloat16):
        case = paged_attention_case([n], [1], heads, kvh, D, Dv, chunk, page, dtype, seed=9, spike=spike, bias=0.0)
        rows, spans, q, pos, req = case["last"]
        out = torch.empty(1, heads * Dv, device="cuda", dtype=dtype)
        # lambda 0: the output of head 0 is its map 1 alone, normed
        if dtype == torch.float32:
            ops.diff_attention(q, out, case["pool"], case["bt"], pos, req, 1, page, heads, kvh, D, Dv, 1.0, 0.0, chunk, 0, 0.0,
                               1e-6, 1.0, case["err"])
        else:
            out = tensor_core_attention(case, [n], [1], heads, kvh, D, Dv, 1.0, 0.0, 0.0, chunk, 1e-6, 1.0).to(dtype).cuda()
        rnd = None if dtype == torch.float32 else P.to_bf16_and_back
        want = plain_attention_rows(case, 0, heads, kvh, D, Dv, 1.0, 0.0, 0.0, chunk, 1e-6, 1.0, rnd)[-1:]
        tol = 1e-4 if dtype == torch.float32 else 3e-2
        assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol), (where, dtype)
        v_target = P.plain_rms_unit(case["reqs"][0][target, qw + 2 * D:qw + 2 * D + Dv].double(), 1e-6)
        close = torch.allclose(out[0, :Dv].cpu().double(), v_target, atol=5e-2)
        assert close == (where != "outside"), (where, dtype)      # the seen target IS the output; the unseen one is not


# ----------------------------------------------------------------------------- whole models through the step function
SEQ = {"s1": [83, 40, 9, 121], "s2": [150, 31, 70, 2]}


@gpu
@pytest.mark.parametrize("name", ["s1", "s2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_residuals(folders, name, dtype):
    folder, cfg, W, page = folders[name]
    eng = engine(folder, dtype, page)
    seqs = [random_tokens(n, cfg["vocab"], 40 + i) for i, n in enumerate(SEQ[name])]
    if dtype == "float32":
        seen = {}
        eng.model.layer_hook = lambda ci, x: seen.__setitem__(ci, x.cpu().double())
        got = run_schedule(eng, seqs[:1], [[(0, len(seqs[0]))]])
        eng.model.layer_hook = None
        res = []
        P.plain_forward(cfg, W, seqs[0], residuals=res)
        assert len(seen) == len(res) == len(P.plain_order(cfg))
        for ci, want in enumerate(res):
            assert torch.allclose(seen[ci][:len(seqs[0])], want, atol=2e-4 * float(want.abs().max())), f"residual after entry {ci}"
        compare(got[0], cfg, W, seqs[0], dtype, f"{name} whole 0")
    got = run_schedule(eng, seqs, [[(i, len(s))] for i, s in enumerate(seqs)])
    for i, s in enumerate(seqs):
        compare(got[i], cfg, W, s, dtype, f"{name} whole {i}")


@gpu
@pytest.mark.parametrize("name", ["s1", "s2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_then_token_by_token_and_from_the_first_token(folders, name, dtype):
    folder, cfg, W, page = folders[name]
    eng = engine(folder, dtype, page)
    s = random_tokens(97, cfg["vocab"], 5)
    got = run_schedule(eng, [s], [[(0, 50)]] + [[(0, 1)]] * 47)            # passes chunk edges while decoding
    compare(got[0], cfg, W, s, dtype, f"{name} prefill+decode")
    got = run_schedule(eng, [s[:45]], [[(0, 1)]] * 45)                    # every token alone, the first too
    compare(got[0], cfg, W, s[:45], dtype, f"{name} decode only")


@gpu
@pytest.mark.parametrize("name", ["s1", "s2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(folders, name, dtype):
    folder, cfg, W, page = folders[name]
    eng = engine(folder, dtype, page)
    s = random_tokens(140, cfg["vocab"], 6)
    for sizes in ([2, 3, 2, 5, 17, 2, 36, 11, 2, 1, 37, 22], [64, 2, 64, 10], [7] * 20):
        assert sum(sizes) == 140
        got = run_schedule(eng, [s], [[(0, n)] for n in sizes])
        compare(got[0], cfg, W, s, dtype, f"{name} portions {sizes[:4]}")


@gpu
@pytest.mark.parametrize("name", ["s1", "s2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_with_slots_and_pages_used_again(folders, name, dtype):
    """Six requests through four slots and a pool that cannot hold them all at once: portions beside single
    tokens, requests that sit a step out; every request's logits against the plain implementation AND, in
    float32, within rounding of the same request run alone."""
    folder, cfg, W, page = folders[name]
    lens = [60, 33, 90, 17, 45, 71]
    seqs = [random_tokens(n, cfg["vocab"], 70 + i) for i, n in enumerate(lens)]
    rng = random.Random(3)
    eng = engine(folder, dtype, page, tokens=256 + 64, batch=128, reqs=4)
    at, live, waiting, steps = {}, [], list(range(len(seqs))), []
    while waiting or live:
        while waiting and len(live) < 4 and sum((len(seqs[i]) + 63) // 64 * 64 for i in live + [waiting[0]]) <= 320:
            live.append(waiting.pop(0)); at[live[-1]] = 0
        step = []
        for i in list(live):
            if len(live) > 1 and rng.random() < 0.25:
                continue
            left = len(seqs[i]) - at[i]
            n = 1 if left <= 6 else min(left - 6, rng.choice([2, 3, 8, 19, 30]))
            step.append((i, n)); at[i] += n
            if at[i] == len(seqs[i]):
                live.remove(i)
        if step:
            steps.append(step)
    got = run_schedule(eng, seqs, steps)
    assert max(len(s) for s in steps) >= 3
    alone = engine(folder, dtype, page) if dtype == "float32" else None
    for i, s in enumerate(seqs):
        compare(got[i], cfg, W, s, dtype, f"{name} mixed {i}")
        if alone is not None:
            one = run_schedule(alone, [s], [[(0, len(s))]])[0]
            assert np.abs(one - got[i]).max() <= 2e-4 * np.abs(one).max()


# ----------------------------------------------------------------------------- other orders of layers
def order_cases():
    g = lambda ff=None: P.gla_layer(2, 8, 24, tau=4.0, ff=ff)
    a = lambda ff=None: P.attention_layer(3, 1, 8, 12, chunk=13, softcap=9.0, diff=0.4, ff=ff)
    return {
        "only linear attention, everything looped": P.make_config(96, 48, [g(40), g()], loop=(0, 2, 3), scale=0.7),
        "only attention, no feed-forward anywhere": P.make_config(96, 48, [a(), a()], scale=1.3),
        "loop at the end, once": P.make_config(96, 50, [a(32), g(32), a()], loop=(1, 3, 1)),
        "a loop that runs no layer": P.make_config(96, 48, [g(24), a(24)], loop=(1, 1, 4)),
        "one layer run five times": P.make_config(64, 40, [g(16)], loop=(0, 1, 5), eps=1e-3),
    }


@gpu
@pytest.mark.parametrize("name", list(order_cases()))
def test_other_orders_of_layers(name, tmp_path):
    cfg = order_cases()[name]
    W = P.random_weights(cfg, seed=3, rank=4)
    stored = dict(W)
    if "loop.step" not in stored and cfg.get("loop"):
        stored["loop.step"] = torch.ones(cfg["loop"]["times"], cfg["width"], dtype=torch.bfloat16)     # a file may still hold it
    folder = P.write_folder(str(tmp_path / "m"), cfg, stored)
    seqs = [random_tokens(n, cfg["vocab"], 7 + n) for n in (45, 8)]
    for dtype in ("float32", "bfloat16"):
        eng = engine(folder, dtype, 8, tokens=192, batch=64)
        got = run_schedule(eng, seqs, [[(0, 30), (1, 2)], [(0, 1), (1, 5)], [(0, 13), (1, 1)], [(0, 1)]])
        for i, sq in enumerate(seqs):
            compare(got[i], cfg, W, sq, dtype, f"{name}, request {i}")


@gpu
def test_long_decoding_across_many_chunks(folders):
    folder, cfg, W, page = folders["s1"]
    eng = engine(folder, "float32", page, tokens=512)
    s = random_tokens(330, cfg["vocab"], 8)
    got = run_schedule(eng, [s], [[(0, 10)]] + [[(0, 1)]] * 320)
    compare(got[0], cfg, W, s, "float32", "long decode")


@gpu
def test_greedy_generation_through_the_entry_point(folders):
    import airun_b200
    folder, cfg, W, page = folders["s2"]
    eng = engine(folder, "float32", page, tokens=512, batch=64, reqs=4)
    prompts = [random_tokens(n, cfg["vocab"], 90 + n) for n in (70, 5, 31)]
    reqs = [eng.add_request(p, airun_b200.SamplingParams.greedy(), max_new_tokens=12) for p in prompts]
    while any(r.finished is None for r in reqs):
        eng.run_step()
    for p, r in zip(prompts, reqs):
        assert r.output == P.plain_greedy(cfg, W, p, 12)
    one = eng.generate(prompts[1], airun_b200.SamplingParams.greedy(), max_new_tokens=12)
    assert one.token_ids == P.plain_greedy(cfg, W, prompts[1], 12)


@gpu
def test_replay_tool_runs_a_vedizen_folder(folders, tmp_path):
    folder, cfg, W, page = folders["s1"]
    seqs = [random_tokens(n, cfg["vocab"], 20 + n) for n in (50, 23)]
    rp = Replay(folder, "float32", str(tmp_path), max_tokens=128, page_size=page)
    a = rp.step([dict(id="a", tokens=seqs[0][:30], want=[0, 29])])
    b = rp.step([dict(id="a", tokens=seqs[0][30:], want=[19]), dict(id="b", tokens=seqs[1], want=[22])], end=["a", "b"])
    assert rp.close() == 0
    wa, wb = P.plain_forward(cfg, W, seqs[0]).numpy(), P.plain_forward(cfg, W, seqs[1]).numpy()
    assert_close(np.concatenate([a, b]), np.stack([wa[0], wa[29], wa[49], wb[22]]).astype(np.float32), "float32", "replay")
