"""The Pogarax decoder in the engine against the plain implementation (tests/plain_pogarax.py): each mechanism's
kernels alone, then whole models of several small shapes through the step function, the scheduler and the replay
tool: whole prompts, token-by-token decoding, portions down to two tokens, unequal batches, slots and pages used
again, window edges, far keys, sinks, the first tokens and long decoding."""
from __future__ import annotations

import math
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_pogarax as P
from helpers import Replay, assert_close, bf16_noise, random_tokens

F64 = torch.float64


# ----------------------------------------------------------------------------- small shapes
def shape_p1() -> dict:
    """Odd sizes everywhere (a width no tensor-core product takes): fewer q/k heads than state heads, routers that
    choose two and three experts, a layer without a feed-forward, a layer that reads another layer's cached rows
    through a LONGER window than the owner's, one attention without any window or frequency scaling."""
    return P.make_config(vocab=150, width=100, eps=3e-5, mult=0.6, layers=[
        P.latent_layer(3, 8, 12, 10, 20, 24, window=13, scale=0.3, base=1000.0, scaling=(4.0, 64, 8.0, 2.0), mlp=P.dense(72)),
        P.delta_layer(4, 2, 12, 20, conv=3, mlp=P.moe(24, 5, 2)),
        P.latent_layer(2, 16, 12, 6, 12, 24, window=29, scale=0.25, base=1000.0, scaling=(4.0, 64, 8.0, 2.0), kv_from=0),
        P.wkv_layer(3, 10, mlp=P.moe(16, 3, 3)),
        P.delta_layer(2, 2, 40, 7, conv=2),
        P.latent_layer(1, 4, 6, 8, 8, 16, mlp=P.dense(40))])


def shape_p2() -> dict:
    """Sizes the tensor-core products take in bfloat16, one q/k head for four state heads, a reader with a SHORTER
    window than the owner of its rows, a router that chooses one expert."""
    return P.make_config(vocab=192, width=128, mult=0.8, layers=[
        P.wkv_layer(2, 32, mlp=P.dense(160)),
        P.latent_layer(4, 32, 16, 32, 64, 64, window=24, scaling=(2.0, 32, 16.0, 1.0), base=50000.0, mlp=P.moe(32, 8, 1)),
        P.delta_layer(4, 1, 16, 32, conv=4, mlp=P.moe(48, 4, 2)),
        P.latent_layer(2, 16, 16, 48, 32, 64, window=8, scaling=(2.0, 32, 16.0, 1.0), base=50000.0, kv_from=1, mlp=P.dense(96))])


SHAPES = {"p1": (shape_p1, 8, (6, 5, 4)), "p2": (shape_p2, 16, (16, 8, 8))}     # name -> (config, page size, ranks)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (make, page, ranks) in SHAPES.items():
        cfg = make()
        W = P.random_weights(cfg, seed=len(name) * 5 + ord(name[-1]), ranks=ranks)
        out[name] = (P.write_folder(str(tmp_path_factory.mktemp(name)), cfg, W), cfg, W, page)
        every = P.all_experts(cfg)
        out[name + " all experts"] = (P.write_folder(str(tmp_path_factory.mktemp(name + "_all")), every, W), every, W, page)
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


def compare(got, cfg, W, seq, dtype, what):
    exact = P.plain_forward(cfg, W, seq).numpy()
    if dtype == "float32":
        return assert_close(got, exact.astype(np.float32), dtype, what)
    rounded = P.plain_forward(cfg, W, seq, rnd=P.to_bf16_and_back).numpy()
    assert_close(got, rounded.astype(np.float32), dtype, what, bf16_noise(rounded, exact))


def pick(folders, name, dtype):
    """Which experts a token goes to is a comparison of scores, and about one token in thirty has two scores so close
    that bfloat16 rounding of the router's input decides otherwise: a different, equally valid computation from there
    on.  So the bfloat16 runs use the same weights with routers that choose ALL experts (the scores still weigh them,
    and sorting, segments and sums run as always); the choice itself is tested in float32 and on the kernel alone."""
    return folders[name if dtype == "float32" else name + " all experts"]


# ----------------------------------------------------------------------------- without a GPU
def test_config_reads_sizes_ranks_sharing_and_windows():
    from airun_b200.config import PogaraxConfig, architecture_name, lookup_architecture
    d = shape_p1()
    assert architecture_name(d) == "Pogarax" and lookup_architecture("Pogarax")[0] is PogaraxConfig
    c = PogaraxConfig.from_dict(d)
    assert (c.vocab_size, c.hidden_size, c.norm_eps, c.residual_mult) == (150, 100, 3e-5, 0.6)
    assert [(o.layer, o.cache_from) for o in c.execution_order()] == [(0, None), (1, None), (2, 0), (3, None), (4, None), (5, None)]
    c2 = c.with_tensor_shapes(P.tensor_shapes(d, (6, 5, 4)))
    assert c2.ranks == ((), (6, 5), (), (4,), (6, 5), ())
    specs = c2.layer_specs()
    assert [s.mixer for s in specs] == ["latent_attention", "gated_delta_rule", "latent_attention", "time_mix",
                                        "gated_delta_rule", "latent_attention"]
    assert [s.feed_forward for s in specs] == ["swiglu", "routed_experts", "", "routed_experts", "", "swiglu"]
    assert all(s.arrangement == "post_norm" and s.arrangement_args == dict(residual_mult=0.6) for s in specs)
    assert (specs[1].mixer_args["decay_rank"], specs[1].mixer_args["gate_rank"], specs[3].mixer_args["decay_rank"]) == (6, 5, 4)
    # both layers on layer 0's rows keep them as long as the longer window needs; each masks with its own
    assert (specs[0].mixer_args["window"], specs[0].mixer_args["cache_window"]) == (13, 29)
    assert (specs[2].mixer_args["window"], specs[2].mixer_args["cache_window"], specs[2].mixer_args["owns_cache"]) == (29, 29, False)
    assert (specs[5].mixer_args["window"], specs[5].mixer_args["cache_window"]) == (0, 0)
    assert specs[5].mixer_args["position_args"]["scaling"] is None
    assert specs[1].ffn_args["top"] == 2 and specs[3].ffn_args["num_experts"] == 3
    assert PogaraxConfig.from_dict(c2.to_dict()).to_dict() == c2.to_dict()


def test_config_lists_every_problem():
    from airun_b200.config import ConfigError, PogaraxConfig
    d = shape_p1()
    d["layers"][1]["mixer"]["kv_heads"] = 3
    d["layers"][2]["mixer"]["kv_from"] = 1
    d["layers"][3]["mlp"]["router"]["top"] = 9
    d["layers"][4]["type"] = "other"
    d["norm"]["eps"] = 0
    with pytest.raises(ConfigError) as e:
        PogaraxConfig.from_dict(d)
    for text in ("multiple of kv_heads", "kv_from", "top exceeds", "layers[4]", "norm.eps"):
        assert text in str(e.value)
    d = shape_p2()
    d["layers"][3]["mixer"]["kv_rank"] = 32
    with pytest.raises(ConfigError, match="must be equal"):
        PogaraxConfig.from_dict(d)


def test_declared_tensors_are_the_files_tensors():
    from airun_b200.config import PogaraxConfig
    from airun_b200.engine.model import DecoderModel
    for make, _, ranks in SHAPES.values():
        cfg = make()
        shapes = P.tensor_shapes(cfg, ranks)
        c = PogaraxConfig.from_dict(cfg).with_tensor_shapes(shapes)
        specs = {s.name: tuple(s.shape) for s in DecoderModel(c, torch.float32, "cpu").weight_specs()}
        assert specs == {n: tuple(s) for n, s in shapes.items()}


def test_cache_groups_share_rows_and_keep_flat_state():
    from airun_b200.cache.manager import CacheManager
    from airun_b200.config import PogaraxConfig
    from airun_b200.engine.model import DecoderModel
    from airun_b200.parts.base import PagedKVSpec, StateSpec
    cfg = shape_p1()
    m = DecoderModel(PogaraxConfig.from_dict(cfg).with_tensor_shapes(P.tensor_shapes(cfg)), torch.float32, "cpu")
    specs, src = m.cache_specs()
    assert specs[0] == specs[2] == PagedKVSpec(1, 36, 29, values=False) and specs[0].elements_per_token() == 36
    assert specs[5] == PagedKVSpec(1, 22, 0, values=False) and src == [None, None, 0, None, None, None]
    assert specs[1] == StateSpec((4 * 12 * 20 + 2 * (2 * 24 + 80),), torch.float32)       # matrices + two rows of conv inputs
    assert specs[3] == StateSpec((3 * 10 * 10 + 100,), torch.float32)                     # matrices + the last token's x
    assert specs[4] == StateSpec((2 * 40 * 7 + 1 * (160 + 14),), torch.float32)
    mgr = CacheManager(specs, src, page_size=8, num_pages=16, max_requests=4)
    assert [b.kind for b in mgr.bindings] == ["paged", "state", "paged", "state", "state", "paged"]
    assert mgr.bindings[2].shared and mgr.bindings[2].gid == mgr.bindings[0].gid and len(mgr.paged) == 2


def test_scaled_frequencies_of_the_position_part_are_the_plain_ones():
    from airun_b200.parts.rope import RotaryScaledInterleaved
    for dims, base, sc in ((12, 1000.0, (4.0, 64, 8.0, 2.0)), (32, 50000.0, (2.0, 32, 16.0, 1.0)), (6, 10000.0, None), (64, 1e6, (8.0, 4096, 32.0, 1.0))):
        scaling = None if sc is None else dict(factor=sc[0], original=sc[1], fast=sc[2], slow=sc[3])
        part = RotaryScaledInterleaved(rotary_dim=dims, theta=base, scaling=scaling, device="cpu")
        pos = torch.tensor([0, 1, 7, 300])
        cos, sin = P.plain_rotary_tables(pos, dims, base, scaling)
        ang = pos.double().unsqueeze(-1) * part.inv_freq.double()
        assert torch.allclose(torch.cos(ang) * part.mult, cos, atol=1e-4) and torch.allclose(torch.sin(ang) * part.mult, sin, atol=1e-4)
        if sc is not None:
            assert part.mult == pytest.approx(0.1 * math.log(sc[0]) + 1.0)
            plain = base ** (-2.0 * torch.arange(dims // 2, dtype=F64) / dims)
            ratio = part.inv_freq.double() / plain
            assert ratio[0] == pytest.approx(1.0, abs=1e-6) and ratio.min() >= 1.0 / sc[0] - 1e-6      # fast pairs untouched


def test_plain_recurrences_carry_their_state():
    g = torch.Generator().manual_seed(3)
    T, Hh, D, Dv = 23, 2, 5, 3
    q, k = torch.randn(T, Hh, D, generator=g, dtype=F64), torch.randn(T, Hh, D, generator=g, dtype=F64)
    v, a = torch.randn(T, Hh, Dv, generator=g, dtype=F64), torch.rand(T, Hh, D, generator=g, dtype=F64) * 0.6 + 0.4
    beta = torch.rand(T, Hh, generator=g, dtype=F64)
    o, S = P.plain_delta_recurrence(q, k, v, a, beta)
    o1, S1 = P.plain_delta_recurrence(q[:9], k[:9], v[:9], a[:9], beta[:9])
    o2, S2 = P.plain_delta_recurrence(q[9:], k[9:], v[9:], a[9:], beta[9:], state=S1)
    assert torch.allclose(torch.cat([o1, o2]), o, atol=1e-12) and torch.allclose(S2, S, atol=1e-12)
    # beta 1, no decay, unit keys: the state then returns exactly the value last written along a key
    kk = torch.nn.functional.normalize(k, dim=-1)
    o3, _ = P.plain_delta_recurrence(kk, kk, v, torch.ones_like(a), torch.ones_like(beta))
    assert torch.allclose(o3, v, atol=1e-10)
    u = torch.randn(Hh, D, generator=g, dtype=F64)
    vv = torch.randn(T, Hh, D, generator=g, dtype=F64)
    o, S = P.plain_wkv_recurrence(q, k, vv, a, u)
    oa, Sa = P.plain_wkv_recurrence(q[:4], k[:4], vv[:4], a[:4], u)
    ob, Sb = P.plain_wkv_recurrence(q[4:], k[4:], vv[4:], a[4:], u, state=Sa)
    assert torch.allclose(torch.cat([oa, ob]), o, atol=1e-12) and torch.allclose(Sb, S, atol=1e-12)
    assert torch.allclose(o[0], (q[0] * u * k[0]).sum(-1, keepdim=True) * vv[0], atol=1e-12)     # the first token sees only its bonus


def test_plain_window_sink_and_both_forms_of_the_latent_attention():
    vis = P.plain_window(5, 3, first=4)
    assert vis.int().tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [1, 1, 1, 0, 0], [0, 1, 1, 1, 0], [0, 0, 1, 1, 1]]
    assert P.plain_window(4, 0).int().tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [1, 1, 1, 1]]
    s = torch.tensor([[0.3, -1.0, 2.0]], dtype=F64)
    p = P.plain_sink_softmax(s, 1.5)
    assert float(p.sum()) == pytest.approx(float(torch.exp(s).sum() / (torch.exp(s).sum() + math.exp(1.5))))
    cfg = shape_p1()
    W = {n: t.double() for n, t in P.random_weights(cfg, 9).items()}
    h = torch.randn(31, 100, generator=torch.Generator().manual_seed(1), dtype=F64)
    pos = torch.arange(31)
    m = cfg["layers"][0]["mixer"]
    c, kr = P.plain_latent_kv(h, W, "l0.mix", m, 1e-5, pos)
    a = P.plain_latent_attention(h, W, "l0.mix", m, 1e-5, c, kr, pos, in_latent_space=False)
    b = P.plain_latent_attention(h, W, "l0.mix", m, 1e-5, c, kr, pos, in_latent_space=True)
    assert torch.allclose(a, b, atol=1e-10)


# ----------------------------------------------------------------------------- kernels alone
gpu = pytest.mark.gpu


def dev(t, dtype=torch.float32):
    return t.to("cuda", dtype).contiguous()


def batch_ctx(spans, slots=None):
    """The device arrays of a step whose request r brings rows spans[r] = (first position, end)."""
    lens = [b - a for a, b in spans]
    cu = torch.tensor(np.cumsum([0] + lens), dtype=torch.int32, device="cuda")
    req = torch.cat([torch.full((n,), r) for r, n in enumerate(lens)]).to("cuda", torch.int32)
    pos = torch.cat([torch.arange(a, b) for a, b in spans]).to("cuda", torch.int32)
    sl = torch.tensor(slots if slots is not None else list(range(len(spans))), dtype=torch.int32, device="cuda")
    return SimpleNamespace(req_of_token=req, cu_tokens=cu, positions=pos, state_slots=sl, num_reqs=len(spans),
                           err=torch.zeros(1, dtype=torch.int32, device="cuda"))


@gpu
def test_norm_on_the_output_adds_to_the_stream_and_leaves_a_copy():
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for T, n in ((7, 70), (3, 2500)):
        x, y, w = torch.randn(T, n, generator=g) * 3, torch.randn(T, n, generator=g) * 5, torch.randn(n, generator=g)
        xd, cast = dev(x), torch.empty(T, n, device="cuda", dtype=torch.bfloat16)
        ops.postnorm_add(xd, dev(y), dev(w), 1e-5, 0.7, cast=cast)
        want = x.double() + 0.7 * P.plain_rmsnorm(y.double(), w.double(), 1e-5)
        assert torch.allclose(xd.cpu().double(), want, atol=1e-5)
        assert torch.equal(cast.cpu(), xd.cpu().to(torch.bfloat16))
        xd2 = dev(x)
        ops.postnorm_add(xd2, dev(y), dev(w), 1e-5, 0.7)
        assert torch.equal(xd2, xd)


@gpu
@pytest.mark.parametrize("mode", ["exp_softplus", "sigmoid", "exp_neg_exp"])
def test_second_halves_of_the_low_rank_pairs(mode):
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    T, rank, groups, D = 11, 7, 3, 20
    n = groups * D
    low, w2, b, a_log = torch.randn(T, rank + 2, generator=g), torch.randn(n, rank, generator=g), torch.randn(n, generator=g), torch.randn(groups, generator=g)
    out = torch.empty(T, n, device="cuda")
    ctx = batch_ctx([(0, T)])
    lowd = dev(low)[:, 1:1 + rank]                                       # a column slice, as the mixers pass it
    z = low[:, 1:1 + rank].double()
    if mode == "exp_softplus":
        ops.lowrank_act(lowd, dev(w2), dev(b), out, ctx.req_of_token, ops.LOWRANK_EXP_SOFTPLUS, group_param=dev(a_log), group=D)
        want = P.plain_delta_decay(z, torch.eye(rank, dtype=F64), w2.double(), b.double(), a_log.double(), groups, D).reshape(T, n)
    elif mode == "sigmoid":
        ops.lowrank_act(lowd, dev(w2), None, out, ctx.req_of_token, ops.LOWRANK_SIGMOID)
        want = torch.sigmoid(z @ w2.double().T)
    else:
        ops.lowrank_act(lowd, dev(w2), dev(b), out, ctx.req_of_token, ops.LOWRANK_EXP_NEG_EXP, in_tanh=True)
        want = torch.exp(-torch.exp(torch.tanh(z) @ w2.double().T + b.double()))
    assert torch.allclose(out.cpu().double(), want, atol=2e-6, rtol=2e-5)


@gpu
@pytest.mark.parametrize("heads,kvh,D,Dv,taps", [(4, 2, 12, 20, 3), (2, 2, 130, 33, 4), (1, 1, 8, 8, 1), (4, 1, 64, 96, 2), (3, 3, 32, 64, 6)])
def test_delta_rule_kernels_carry_state_across_steps_and_requests(heads, kvh, D, Dv, taps):
    """Three requests of unequal length in one batch, each cut into steps at other places (also portions shorter than
    the convolution), slots out of order; the convolution's tail and the matrices against the plain implementation."""
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(heads * 100 + D)
    lens, cuts, slots = [13, 1, 37], [[2, 3, 5], [0, 0, 0], [1, 35, 36]], [2, 0, 3]
    kd, vd = kvh * D, heads * Dv
    C = 2 * kd + vd
    data = [dict(x=torch.randn(n, C, generator=g), beta=torch.randn(n, heads, generator=g),
                 decay=torch.rand(n, heads * D, generator=g) * 0.5 + 0.5) for n in lens]
    wconv = torch.randn(C, taps, generator=g) * 0.6
    nstate = heads * D * Dv + (taps - 1) * C
    state = torch.zeros(4, nstate, device="cuda")
    got = [[] for _ in lens]
    for part in range(4):
        spans = [((c[part - 1] if part else 0), (c[part] if part < 3 else n)) for n, c in zip(lens, cuts)]
        rows = [i for i, (a, b) in enumerate(spans) if b > a]
        ctx = batch_ctx([spans[i] for i in rows], [slots[i] for i in rows])
        cat = lambda key: torch.cat([data[i][key][spans[i][0]:spans[i][1]] for i in rows])
        proj = dev(torch.cat([cat("x"), cat("beta")], dim=1))
        decay = dev(cat("decay"))
        T = proj.shape[0]
        conv = torch.empty(T, C, device="cuda")
        ops.short_conv(proj[:, :C], dev(wconv), state, heads * D * Dv, ctx, conv, 2 * kvh, kvh, D, 1e-6, D ** -0.5)
        o = torch.empty(T, vd, device="cuda")
        ops.recurrent_state(ops.RECURRENCE_DELTA, conv[:, :kd], conv[:, kd:2 * kd], conv[:, 2 * kd:], decay, state, ctx, o, heads,
                            heads // kvh, D, Dv, beta=proj[:, C:], tail_src=proj[:, :C], tail_off=heads * D * Dv, tail_rows=taps - 1)
        assert int(ctx.err.item()) == 0
        for j, i in enumerate(rows):
            got[i].append(o[ctx.cu_tokens[j]:ctx.cu_tokens[j + 1]].cpu())
    rep = heads // kvh
    for i, n in enumerate(lens):
        x = data[i]["x"].double()
        y = P.plain_silu(P.plain_short_conv(x, wconv.double()))
        q = (P.plain_unit(y[:, :kd].view(n, kvh, D)) * D ** -0.5).repeat_interleave(rep, dim=1)
        k = P.plain_unit(y[:, kd:2 * kd].view(n, kvh, D)).repeat_interleave(rep, dim=1)
        o, S = P.plain_delta_recurrence(q, k, y[:, 2 * kd:].view(n, heads, Dv), data[i]["decay"].double().view(n, heads, D),
                                        torch.sigmoid(data[i]["beta"].double()))
        assert torch.allclose(torch.cat(got[i]).double(), o.reshape(n, vd), atol=2e-4, rtol=2e-4), f"request {i}"
        assert torch.allclose(state[slots[i], :heads * D * Dv].cpu().double(), S.reshape(-1), atol=2e-4, rtol=2e-4)
        if taps > 1:
            tail = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x])[-(taps - 1):]
            assert torch.equal(state[slots[i], heads * D * Dv:].cpu().double(), tail.reshape(-1)), f"conv tail of request {i}"
    assert (state[1] == 0).all()                                   # a slot nobody used stays as it was


@gpu
@pytest.mark.parametrize("heads,D", [(3, 10), (2, 32), (1, 130), (2, 64)])
def test_time_mix_kernels_carry_state_across_steps_and_requests(heads, D):
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(heads * 10 + D)
    lens, cuts, slots, Wd = [9, 2, 30], [4, 1, 29], [1, 3, 0], 24
    hd = heads * D
    data = [dict(r=torch.randn(n, hd, generator=g), k=torch.randn(n, hd, generator=g) * 0.5, v=torch.randn(n, hd, generator=g),
                 w=torch.rand(n, hd, generator=g) * 0.6 + 0.4, x=torch.randn(n, Wd, generator=g)) for n in lens]
    bonus, mu = torch.randn(heads, D, generator=g), torch.rand(5, Wd, generator=g)
    state = torch.zeros(4, heads * D * D + Wd, device="cuda")
    got, mixes = [[] for _ in lens], [[] for _ in lens]
    for part in (0, 1):
        spans = [(0, c) if part == 0 else (c, n) for n, c in zip(lens, cuts)]
        ctx = batch_ctx(spans, slots)
        cat = lambda key: dev(torch.cat([data[i][key][a:b] for i, (a, b) in enumerate(spans)]))
        x = cat("x")
        T = x.shape[0]
        mix = torch.empty(5, T, Wd, device="cuda")
        ops.token_shift(x, dev(mu), state, heads * D * D, ctx, mix)
        o = torch.empty(T, hd, device="cuda")
        ops.recurrent_state(ops.RECURRENCE_WKV, cat("r"), cat("k"), cat("v"), cat("w"), state, ctx, o, heads, 1, D, D, bonus=dev(bonus),
                            tail_src=x, tail_off=heads * D * D, tail_rows=1)
        assert int(ctx.err.item()) == 0
        for i in range(len(lens)):
            got[i].append(o[ctx.cu_tokens[i]:ctx.cu_tokens[i + 1]].cpu())
            mixes[i].append(mix[:, ctx.cu_tokens[i]:ctx.cu_tokens[i + 1]].cpu())
    for i, n in enumerate(lens):
        d = {k_: t.double() for k_, t in data[i].items()}
        sh = lambda t: t.view(n, heads, D)
        o, S = P.plain_wkv_recurrence(sh(d["r"]), sh(d["k"]), sh(d["v"]), sh(d["w"]), bonus.double())
        assert torch.allclose(torch.cat(got[i]).double(), o.reshape(n, hd), atol=2e-4, rtol=2e-4), f"request {i}"
        assert torch.allclose(state[slots[i], :heads * D * D].cpu().double(), S.reshape(-1), atol=2e-4, rtol=2e-4)
        assert torch.equal(state[slots[i], heads * D * D:].cpu(), data[i]["x"][-1])
        prev = torch.cat([torch.zeros(1, Wd, dtype=F64), d["x"][:-1]])
        want = d["x"] + (prev - d["x"]) * mu.double().unsqueeze(1)
        assert torch.allclose(torch.cat(mixes[i], dim=1).double(), want, atol=1e-6)
    assert (state[2] == 0).all()


@gpu
def test_delta_rule_remembers_a_token_from_far_back():
    """Decays a hair below one and later tokens that write along other keys: what token 0 wrote along its key is
    still read 600 single-token steps on."""
    from airun_b200.kernels import ops
    heads, D, Dv, n = 1, 16, 32, 600
    q, k, v = torch.zeros(n, D), torch.zeros(n, D), torch.zeros(n, Dv)
    k[0, 3], v[0] = 1.0, torch.arange(Dv) - 10.0
    q[:, 3] = 1.0
    k[1:, 5], v[1:, 0] = 1.0, 1.0
    state = torch.zeros(1, heads * D * Dv, device="cuda")
    beta = torch.full((n, 1), 30.0)                                 # sigmoid -> 1
    o = torch.empty(1, Dv, device="cuda")
    ctx = batch_ctx([(0, 1)])
    qd, kd_, vd, bd, dd = dev(q), dev(k), dev(v), dev(beta), dev(torch.full((n, D), 0.9995))
    for t in range(n):
        ops.recurrent_state(ops.RECURRENCE_DELTA, qd[t:t + 1], kd_[t:t + 1], vd[t:t + 1], dd[t:t + 1], state, ctx, o, heads, 1, D, Dv,
                            beta=bd[t:t + 1])
    assert torch.allclose(o[0].cpu().double(), 0.9995 ** (n - 1) * v[0].double(), rtol=1e-3, atol=1e-3)


def latent_case(seq_lens, new_lens, H, R, rd, page, dtype, seed, spike=None):
    """Cached rows written through the prepare kernel (pages handed out in a scrambled order) for the first len - new
    tokens of every request, then the last ``new`` tokens of each as one batch.  No rotation, unit norm weights."""
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    reqs = []
    for n in seq_lens:
        rows, ql = torch.randn(n, 1 + R + rd, generator=g), torch.randn(n, H * (R + rd), generator=g)
        if spike is not None:
            spike(rows, ql, n)
        reqs.append((rows, ql))
    blocks = [(n + page - 1) // page for n in seq_lens]
    num_pages = sum(blocks) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    bt = torch.full((len(seq_lens), max(blocks)), -1, dtype=torch.int32)
    for r, nb in enumerate(blocks):
        for b in range(nb):
            bt[r, b] = perm.pop()
    cache = SimpleNamespace(pool=torch.zeros(num_pages, page * (R + rd), device="cuda", dtype=dtype), block_table=bt.cuda(), page_size=page)
    ones = torch.ones(max(R, 1), device="cuda")
    last = None
    for phase in (0, 1):
        spans = [(0, n - m) if phase == 0 else (n - m, n) for n, m in zip(seq_lens, new_lens)]
        ctx = batch_ctx(spans)
        proj = dev(torch.cat([reqs[r][0][a:b] for r, (a, b) in enumerate(spans)]))
        if proj.shape[0] == 0:
            continue
        cq = torch.empty(proj.shape[0], 1, device="cuda", dtype=dtype)
        ops.latent_prepare(proj, ones[:1], ones[:R], 1e-6, cq, R, rd, 0, None, 1.0, cache, ctx, True)
        assert int(ctx.err.item()) == 0
        last = (spans, ctx)
    return reqs, cache, last


def plain_latent_rows(rows, ql, H, R, rd, scale, window, sink, rnd=None):
    """The kernel's sum for every token of one request, from the equations: rows [n, 1 + R + rd] as projected."""
    rr = (lambda t: t) if rnd is None else rnd
    n = rows.shape[0]
    c = rr(P.plain_rms_unit(rows[:, 1:1 + R].double(), 1e-6))
    key = torch.cat([c, rr(rows[:, 1 + R:].double())], dim=1)
    vis = P.plain_window(n, window)
    out = torch.zeros(n, H, R, dtype=F64)
    q = rr(ql.double()).view(n, H, R + rd)
    for h in range(H):
        s = (q[:, h] @ key.T * scale).masked_fill(~vis, -math.inf)
        out[:, h] = P.plain_sink_softmax(s, float(sink[h])) @ c
    return out.reshape(n, H * R)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,rd,page,window", [(3, 24, 12, 8, 13), (2, 64, 16, 16, 0), (1, 130, 6, 24, 40), (4, 16, 0, 8, 5)])
def test_latent_attention_over_scrambled_pages(H, R, rd, page, window, dtype):
    from airun_b200.kernels import ops
    seq_lens, new_lens = [70, 9, 33], [1, 9, 20]
    reqs, cache, (spans, ctx) = latent_case(seq_lens, new_lens, H, R, rd, page, dtype, seed=H * 7 + R)
    sink = torch.tensor([0.5, -1.0, 2.0, 0.0][:H])
    ql = dev(torch.cat([reqs[r][1][a:b] for r, (a, b) in enumerate(spans)]), dtype)
    out = torch.empty(ql.shape[0], H * R, device="cuda", dtype=dtype)
    ops.latent_attention(ql, out, cache, ctx, H, R, rd, 0.2, window, dev(sink))
    assert int(ctx.err.item()) == 0
    rnd = None if dtype == torch.float32 else P.to_bf16_and_back
    want = torch.cat([plain_latent_rows(*reqs[r], H, R, rd, 0.2, window, sink, rnd)[a:b] for r, (a, b) in enumerate(spans)])
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)


@gpu
@pytest.mark.parametrize("where", ["inside", "outside", "far", "first"])
@pytest.mark.parametrize("new", [1, 12])
def test_one_dominant_key_at_the_windows_edge_and_far_back(where, new):
    """One cached row is made to dominate the last query's scores (a query along it, scaled up): just inside the
    window it IS the output, one position further back it must not be seen at all; with no window a key 900
    positions back and the sequence's very first token are still found.  Decoded alone and as the last row of a portion."""
    from airun_b200.kernels import ops
    H, R, rd, page = 2, 32, 8, 16
    window = 37 if where in ("inside", "outside") else 0
    n = 1000 if where in ("far", "first") else 120
    target = {"inside": n - window, "outside": n - window - 1, "far": n - 1 - 900, "first": 0}[where]

    def spike(rows, ql, n_):
        c = P.plain_rms_unit(rows[target, 1:1 + R].double(), 1e-6)
        ql[n_ - 1].view(H, R + rd)[:, :R] = 6.0 * c.float()
        ql[n_ - 1].view(H, R + rd)[:, R:] = 0.0
    reqs, cache, (spans, ctx) = latent_case([n], [new], H, R, rd, page, torch.float32, seed=11, spike=spike)
    sink = torch.tensor([-30.0, -30.0])
    out = torch.empty(new, H * R, device="cuda")
    ops.latent_attention(dev(reqs[0][1][n - new:]), out, cache, ctx, H, R, rd, 1.0, window, dev(sink))
    want = plain_latent_rows(*reqs[0], H, R, rd, 1.0, window, sink)[n - new:]
    assert torch.allclose(out.cpu().double(), want, atol=1e-4, rtol=1e-4)
    c_target = P.plain_rms_unit(reqs[0][0][target, 1:1 + R].double(), 1e-6)
    seen = torch.allclose(out[-1, :R].cpu().double(), c_target, atol=5e-2)
    assert seen == (where != "outside")


@gpu
def test_a_sink_takes_its_share_and_nothing_else():
    """With one visible key (the first token of a sequence) the output is the cached latent times
    exp(s) / (exp(s) + exp(sink)); a very negative sink leaves a plain softmax."""
    from airun_b200.kernels import ops
    H, R, rd = 3, 16, 4
    reqs, cache, (spans, ctx) = latent_case([1], [1], H, R, rd, 8, torch.float32, seed=2)
    rows, ql = reqs[0]
    sink = torch.tensor([0.7, -40.0, 3.0])
    out = torch.empty(1, H * R, device="cuda")
    ops.latent_attention(dev(ql), out, cache, ctx, H, R, rd, 0.5, 0, dev(sink))
    c = P.plain_rms_unit(rows[0, 1:1 + R].double(), 1e-6)
    key = torch.cat([c, rows[0, 1 + R:].double()])
    for h in range(H):
        s = 0.5 * float(ql[0].double().view(H, R + rd)[h] @ key)
        share = math.exp(s) / (math.exp(s) + math.exp(float(sink[h])))
        assert torch.allclose(out[0, h * R:(h + 1) * R].cpu().double(), share * c, atol=1e-5)
    assert torch.allclose(out[0, R:2 * R].cpu().double(), c, atol=1e-5)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_of_queries_and_cached_keys(dtype):
    from airun_b200.kernels import ops
    from airun_b200.parts.rope import RotaryScaledInterleaved
    H, D, R, rd, page = 2, 6, 10, 8, 8
    part = RotaryScaledInterleaved(rotary_dim=rd, theta=100.0, scaling=dict(factor=4.0, original=16, fast=4.0, slow=1.0), device="cuda")
    g = torch.Generator().manual_seed(4)
    spans = [(5, 14), (0, 3)]
    ctx = batch_ctx(spans)
    T = 12
    proj, q = torch.randn(T, 7 + R + rd, generator=g), torch.randn(T, H * (D + rd), generator=g)
    wq, wkv = torch.randn(7, generator=g), torch.randn(R, generator=g)
    cache = SimpleNamespace(pool=torch.zeros(5, page * (R + rd), device="cuda", dtype=dtype),
                            block_table=torch.tensor([[3, 1], [4, -1]], dtype=torch.int32, device="cuda"), page_size=page)
    cq = torch.empty(T, 7, device="cuda", dtype=dtype)
    ops.latent_prepare(dev(proj), dev(wq), dev(wkv), 1e-5, cq, R, rd, rd, part.inv_freq, part.mult, cache, ctx, True)
    qn, qlat = torch.empty(T, H * D, device="cuda", dtype=dtype), torch.zeros(T, H * (R + rd), device="cuda", dtype=dtype)
    ops.latent_query(dev(q), qn, qlat, H, D, R, rd, rd, part.inv_freq, part.mult, ctx)
    assert int(ctx.err.item()) == 0
    pos = ctx.positions.cpu()
    cos, sin = P.plain_rotary_tables(pos, rd, 100.0, dict(factor=4.0, original=16, fast=4.0, slow=1.0))
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(cq.cpu().double(), P.plain_rmsnorm(proj[:, :7].double(), wq.double(), 1e-5), atol=tol, rtol=tol)
    want_c = P.plain_rmsnorm(proj[:, 7:7 + R].double(), wkv.double(), 1e-5)
    want_kr = P.plain_rotate_pairs(proj[:, 7 + R:].double(), cos, sin, rd)
    pages = cache.pool.view(5, page, R + rd).cpu().double()
    for t in range(T):
        r, p = int(ctx.req_of_token[t]), int(pos[t])
        row = pages[int(cache.block_table[r, p // page]), p % page]
        assert torch.allclose(row, torch.cat([want_c[t], want_kr[t]]), atol=tol, rtol=tol), f"cached row of token {t}"
    q3 = q.double().view(T, H, D + rd)
    assert torch.allclose(qn.cpu().double().view(T, H, D), q3[..., :D], atol=tol, rtol=tol)
    want_qr = P.plain_rotate_pairs(q3[..., D:], cos, sin, rd)
    assert torch.allclose(qlat.cpu().double().view(T, H, R + rd)[..., R:], want_qr, atol=tol, rtol=tol)
    assert (qlat.view(T, H, R + rd)[..., :R] == 0).all()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_products_per_head_and_per_segment(dtype):
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(6)
    T, B, K, N = 37, 3, 20, 70
    a, w = torch.randn(T, B * K + 4, generator=g), torch.randn(B, N, K, generator=g)
    ad, out = dev(a, dtype), torch.full((T, B * (N + 5)), 7.0, device="cuda", dtype=dtype)
    ops.gemm_simt_batched(ad[:, 4:].unflatten(1, (B, K)), dev(w, dtype),
                          out.unflatten(1, (B, N + 5))[:, :, :N])
    rd_ = (lambda t: t.to(dtype).double())
    want = torch.einsum("tbk,bnk->tbn", rd_(a[:, 4:]).view(T, B, K), rd_(w))
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.view(T, B, N + 5)[:, :, :N].cpu().double(), want, atol=tol, rtol=tol)
    assert (out.view(T, B, N + 5)[:, :, N:] == 7.0).all()
    E, M = 5, 150
    seg = torch.tensor([0, 70, 70, 71, 140, 143], dtype=torch.int32, device="cuda")       # an empty segment, rows left over
    x, we = torch.randn(M, K, generator=g), torch.randn(E, N, K, generator=g)
    out = torch.full((M, N), 7.0, device="cuda")
    ops.gemm_simt_grouped(dev(x, dtype), dev(we, dtype), out, seg)
    for e in range(E):
        lo, hi = int(seg[e]), int(seg[e + 1])
        assert torch.allclose(out[lo:hi].cpu().double(), rd_(x[lo:hi]) @ rd_(we[e]).T, atol=tol, rtol=tol)
    assert (out[143:] == 7.0).all()


@gpu
@pytest.mark.parametrize("top,E,scores", [(1, 5, "sigmoid"), (2, 12, "sigmoid"), (3, 3, "sigmoid"), (2, 7, "softmax")])
def test_router_sorts_rows_by_expert_and_brings_them_back(top, E, scores):
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(top * 10 + E)
    T, Wd = 41, 36
    h, wr = torch.randn(T, Wd, generator=g), torch.randn(E, Wd, generator=g) * 0.5
    req = torch.zeros(T, dtype=torch.int32)
    req[[5, 40]] = -1                                                # padding rows are routed nowhere
    ids, rank, row_of = (torch.full((T, top), -7, dtype=torch.int32, device="cuda") for _ in range(3))
    wts = torch.zeros(T, top, device="cuda")
    counts, seg = torch.zeros(E, dtype=torch.int32, device="cuda"), torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    logits = torch.empty(T, E, device="cuda")
    ops.gemm_simt(dev(h), dev(wr), logits)
    ops.moe_route(logits, top, scores == "softmax", False, req.cuda(), ids, wts, rank, counts, seg)
    z = h.double() @ wr.double().T
    s = torch.sigmoid(z) if scores == "sigmoid" else torch.softmax(z, dim=-1)
    val, idx = torch.topk(s, top, dim=-1)
    live = req >= 0
    assert torch.equal(ids.cpu()[live].long(), idx[live]) and (ids.cpu()[~live] == -1).all()
    assert torch.allclose(wts.cpu()[live].double(), val[live], atol=1e-6)
    assert torch.equal(counts.cpu().long(), torch.bincount(idx[live].reshape(-1), minlength=E))
    assert torch.equal(seg.cpu().long(), torch.cat([torch.zeros(1, dtype=torch.long), torch.cumsum(counts.cpu().long(), 0)]))
    xs = torch.zeros(T * top, Wd, device="cuda")
    ops.moe_scatter(dev(h), top, ids, wts, rank, seg, True, xs, row_of)
    rows = row_of.cpu().long()[live].reshape(-1)
    assert sorted(rows.tolist()) == list(range(int(live.sum()) * top))              # every row of the segments is used once
    for t in torch.nonzero(live).reshape(-1).tolist():
        for j in range(top):
            r = int(row_of[t, j])
            assert int(seg[idx[t, j]]) <= r < int(seg[idx[t, j] + 1])
            assert torch.allclose(xs[r].cpu().double(), val[t, j] * h[t].double(), atol=1e-5)
    ys = torch.randn(T * top, Wd, generator=g)
    out = torch.empty(T, Wd, device="cuda")
    ops.moe_combine(dev(ys), top, ids, wts, row_of, False, out)
    for t in range(T):
        want = sum(ys[int(row_of[t, j])].double() for j in range(top)) if live[t] else torch.zeros(Wd, dtype=F64)
        assert torch.allclose(out[t].cpu().double(), want, atol=1e-5)


# ----------------------------------------------------------------------------- whole models through the step function
SEQ = {"p1": [83, 40, 9, 121], "p2": [150, 31, 70, 2]}


@gpu
@pytest.mark.parametrize("name", ["p1", "p2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_residuals(folders, name, dtype):
    folder, cfg, W, page = pick(folders, name, dtype)
    eng = engine(folder, dtype, page)
    seqs = [random_tokens(n, cfg["vocab"], 40 + i) for i, n in enumerate(SEQ[name])]
    if dtype == "float32":
        seen = {}
        eng.model.layer_hook = lambda ci, x: seen.__setitem__(ci, x.cpu().double())
        got = run_schedule(eng, seqs[:1], [[(0, len(seqs[0]))]])
        eng.model.layer_hook = None
        res = []
        P.plain_forward(cfg, W, seqs[0], residuals=res)
        assert len(seen) == len(res) == len(cfg["layers"])
        for ci, want in enumerate(res):
            assert torch.allclose(seen[ci][:len(seqs[0])], want, atol=2e-4 * float(want.abs().max())), f"residual after layer {ci}"
        compare(got[0], cfg, W, seqs[0], dtype, f"{name} whole 0")
    got = run_schedule(eng, seqs, [[(i, len(s))] for i, s in enumerate(seqs)])
    for i, s in enumerate(seqs):
        compare(got[i], cfg, W, s, dtype, f"{name} whole {i}")


@gpu
@pytest.mark.parametrize("name", ["p1", "p2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_then_token_by_token_and_from_the_first_token(folders, name, dtype):
    folder, cfg, W, page = pick(folders, name, dtype)
    eng = engine(folder, dtype, page)
    s = random_tokens(97, cfg["vocab"], 5)
    got = run_schedule(eng, [s], [[(0, 50)]] + [[(0, 1)]] * 47)            # every window passes over decoded tokens
    compare(got[0], cfg, W, s, dtype, f"{name} prefill+decode")
    got = run_schedule(eng, [s[:45]], [[(0, 1)]] * 45)                    # every token alone, the first too
    compare(got[0], cfg, W, s[:45], dtype, f"{name} decode only")


@gpu
@pytest.mark.parametrize("name", ["p1", "p2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(folders, name, dtype):
    folder, cfg, W, page = pick(folders, name, dtype)
    eng = engine(folder, dtype, page)
    s = random_tokens(140, cfg["vocab"], 6)
    for sizes in ([2, 3, 2, 5, 17, 2, 36, 11, 2, 1, 37, 22], [64, 2, 64, 10], [7] * 20):
        assert sum(sizes) == 140
        got = run_schedule(eng, [s], [[(0, n)] for n in sizes])
        compare(got[0], cfg, W, s, dtype, f"{name} portions {sizes[:4]}")


@gpu
@pytest.mark.parametrize("name", ["p1", "p2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_with_slots_and_pages_used_again(folders, name, dtype):
    """Six requests through four slots and a pool that cannot hold them all at once: portions beside single
    tokens, requests that sit a step out; every request's logits against the plain implementation AND, in
    float32, within rounding of the same request run alone."""
    folder, cfg, W, page = pick(folders, name, dtype)
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
    return {
        "only the delta rule, no feed-forward anywhere": P.make_config(96, 48, [P.delta_layer(2, 1, 8, 24, 2), P.delta_layer(3, 3, 8, 8, 5)], mult=1.0),
        "only attention, every layer on the first layer's rows": P.make_config(96, 48, [
            P.latent_layer(3, 8, 4, 12, 16, 16, window=9, mlp=P.dense(32)), P.latent_layer(2, 4, 4, 8, 8, 16, window=9, kv_from=0),
            P.latent_layer(1, 8, 4, 8, 8, 16, kv_from=0, mlp=P.moe(8, 2, 1))]),          # the last one sees everything
        "only the time mix": P.make_config(64, 40, [P.wkv_layer(1, 8, mlp=P.moe(8, 4, 4)), P.wkv_layer(5, 4)], eps=1e-3),
        "a reader right after its owner, then a second owner": P.make_config(96, 56, [
            P.latent_layer(2, 8, 8, 8, 8, 8, window=6), P.latent_layer(2, 8, 8, 8, 8, 8, window=6, kv_from=0, mlp=P.dense(24)),
            P.wkv_layer(2, 12), P.latent_layer(4, 4, 2, 4, 12, 8, window=3, scaling=(8.0, 16, 4.0, 1.0), mlp=P.dense(16))]),
    }


@gpu
@pytest.mark.parametrize("name", list(order_cases()))
def test_other_orders_of_layers(name, tmp_path):
    cfg = order_cases()[name]
    W = P.random_weights(cfg, seed=3, ranks=(4, 3, 2))
    folder = P.write_folder(str(tmp_path / "m"), cfg, W)
    seqs = [random_tokens(n, cfg["vocab"], 7 + n) for n in (45, 8)]
    for dtype in ("float32", "bfloat16"):
        if dtype == "bfloat16":
            cfg = P.all_experts(cfg)
            folder = P.write_folder(str(tmp_path / "all"), cfg, W)
        eng = engine(folder, dtype, 8, tokens=192, batch=64)
        got = run_schedule(eng, seqs, [[(0, 30), (1, 2)], [(0, 1), (1, 5)], [(0, 13), (1, 1)], [(0, 1)]])
        for i, sq in enumerate(seqs):
            compare(got[i], cfg, W, sq, dtype, f"{name}, request {i}")


@gpu
def test_long_decoding_past_every_window(folders):
    folder, cfg, W, page = folders["p1"]
    eng = engine(folder, "float32", page, tokens=512)
    s = random_tokens(330, cfg["vocab"], 8)
    got = run_schedule(eng, [s], [[(0, 10)]] + [[(0, 1)]] * 320)
    compare(got[0], cfg, W, s, "float32", "long decode")


@gpu
def test_greedy_generation_through_the_entry_point(folders):
    import airun_b200
    folder, cfg, W, page = folders["p2"]
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
def test_replay_tool_runs_a_pogarax_folder(folders, tmp_path):
    folder, cfg, W, page = folders["p1"]
    seqs = [random_tokens(n, cfg["vocab"], 20 + n) for n in (50, 23)]
    rp = Replay(folder, "float32", str(tmp_path), max_tokens=128, page_size=page)
    a = rp.step([dict(id="a", tokens=seqs[0][:30], want=[0, 29])])
    b = rp.step([dict(id="a", tokens=seqs[0][30:], want=[19]), dict(id="b", tokens=seqs[1], want=[22])], end=["a", "b"])
    assert rp.close() == 0
    wa, wb = P.plain_forward(cfg, W, seqs[0]).numpy(), P.plain_forward(cfg, W, seqs[1]).numpy()
    assert_close(np.concatenate([a, b]), np.stack([wa[0], wa[29], wa[49], wb[22]]).astype(np.float32), "float32", "replay")


@gpu
@pytest.mark.parametrize("M,E,N,K", [(300, 5, 96, 64), (37, 12, 512, 128), (1500, 3, 288, 200), (64, 64, 64, 256)])
def test_tensor_core_product_per_segment(M, E, N, K):
    """The grouped tcgen05 product against float64: segments of every size (empty ones, one row, several tiles),
    rows left over behind the last segment, with the plain result and with the gated unit in its epilogue."""
    from airun_b200.kernels import fast
    g = torch.Generator().manual_seed(M + E)
    cuts = sorted(int(c) for c in torch.randint(0, M - 3, (E - 1,), generator=g))
    seg_host = [0] + cuts + [M - 3]
    if E >= 3:
        seg_host[2] = seg_host[1]                                     # an empty segment
    seg_host = sorted(seg_host)
    seg = torch.tensor(seg_host, dtype=torch.int32, device="cuda")
    x, w = torch.randn(M, K, generator=g), torch.randn(E, N, K, generator=g) / math.sqrt(K)
    ctx = SimpleNamespace(err=torch.zeros(1, dtype=torch.int32, device="cuda"))
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    out = torch.full((M, N), 7.0, device="cuda")
    assert fast.grouped_linear_bf16(ctx, xd, wd, out, seg)
    act = torch.full((M, N // 2), 7.0, device="cuda", dtype=torch.bfloat16)
    assert fast.grouped_linear_bf16(ctx, xd, wd, act, seg, swiglu_group=16)
    assert int(ctx.err.item()) == 0
    xr, wr = xd.cpu().double(), wd.cpu().double()
    for e in range(E):
        lo, hi = seg_host[e], seg_host[e + 1]
        want = xr[lo:hi] @ wr[e].T
        assert torch.allclose(out[lo:hi].cpu().double(), want, atol=2e-3, rtol=2e-3), f"segment {e}"
        gu = want.view(hi - lo, N // 32, 2, 16)
        unit = (P.plain_silu(gu[:, :, 0]) * gu[:, :, 1]).reshape(hi - lo, N // 2)
        assert torch.allclose(act[lo:hi].cpu().double(), unit, atol=2e-2, rtol=2e-2), f"gated unit of segment {e}"
    assert (out[M - 3:] == 7.0).all() and (act[M - 3:] == 7.0).all()


@gpu
@pytest.mark.parametrize("single", [False, True])
@pytest.mark.parametrize("H,R,rd,page,window", [(3, 24, 16, 8, 13), (16, 64, 16, 16, 0), (5, 264, 8, 24, 40), (40, 32, 0, 8, 70), (16, 512, 64, 16, 100)])
def test_tensor_core_latent_attention(H, R, rd, page, window, single):
    """The mma kernel in both of its forms (several tokens a CTA; one token a CTA with the keys split over the warps)
    against the equations, over scrambled pages: head counts below and above a row tile, more than 256 output
    columns, windows that end inside a key tile, requests of one token beside portions."""
    from airun_b200.kernels import fast
    seq_lens, new_lens = [150, 9, 77, 1], [1, 9, 30, 1] if not single else [1, 1, 1, 1]
    reqs, cache, (spans, ctx) = latent_case(seq_lens, new_lens, H, R, rd, page, torch.bfloat16, seed=H + R)
    ctx.decode_only = single
    sink = torch.randn(H, generator=torch.Generator().manual_seed(1))
    ql = dev(torch.cat([reqs[r][1][a:b] for r, (a, b) in enumerate(spans)]), torch.bfloat16)
    out = torch.zeros(ql.shape[0], H * R, device="cuda", dtype=torch.bfloat16)
    part = SimpleNamespace(nh=H, R=R, rd=rd, scale=0.2, window=window, sink=dev(sink))
    assert fast.latent_attention_bf16(ctx, ql, out, cache, part)
    assert int(ctx.err.item()) == 0
    want = torch.cat([plain_latent_rows(*reqs[r], H, R, rd, 0.2, window, sink, P.to_bf16_and_back)[a:b] for r, (a, b) in enumerate(spans)])
    assert torch.allclose(out.cpu().double(), want, atol=3e-2, rtol=3e-2)


@gpu
def test_router_tells_apart_scores_that_saturate():
    """Logits of 17 and more all have the float32 sigmoid 1.0: the experts are still chosen in the order of the logits,
    as the exact scores order them."""
    from airun_b200.kernels import ops
    z = torch.tensor([[17.5, -2.0, 21.0, 19.0, 3.0], [30.0, 30.5, -1.0, 29.0, 40.0]])
    T, E, top = z.shape[0], z.shape[1], 3
    ids, rank = (torch.zeros(T, top, dtype=torch.int32, device="cuda") for _ in range(2))
    wts = torch.zeros(T, top, device="cuda")
    counts, seg = torch.zeros(E, dtype=torch.int32, device="cuda"), torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    ops.moe_route(dev(z), top, False, False, torch.zeros(T, dtype=torch.int32, device="cuda"), ids, wts, rank, counts, seg)
    assert ids.cpu().tolist() == [[2, 3, 0], [4, 1, 0]]
    assert torch.allclose(wts.cpu().double(), torch.sigmoid(z.double()).gather(1, ids.cpu().long()), atol=1e-6)
