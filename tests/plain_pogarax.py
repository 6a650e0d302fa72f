"""A plain, slow implementation of the Pogarax decoder for the tests: whole sequences, no cache, torch on the
CPU in float64 unless told otherwise, one function per mechanism.  It shares no code with the package.

Notation: T tokens, width W; a linear weight is [out, in] and applied as x @ w.T.  ``rnd`` (optional) rounds a
tensor where the bfloat16 engine stores one in bfloat16 (the input of the products); it is the identity for the
exact result.

A layer adds the NORMED output of each sub-layer to the residual stream, x += m * rmsnorm(sub(x)) * w, and the
sub-layers read x itself.  Mixers: a gated delta rule with short convolutions (``channel_delta``), a latent
attention with a sliding window, a rotated key part shared by the heads and a sink in the softmax
(``latent_attention``), and a time mix with a matrix state per head (``wkv``).  Feed-forwards: SwiGLU, or a
mixture of SwiGLU experts routed by sigmoid scores that scale the expert's input.
"""
from __future__ import annotations

import json
import math
import os
from typing import Callable, Dict, List, Optional

import torch

Rounding = Optional[Callable[[torch.Tensor], torch.Tensor]]


def _r(rnd: Rounding, t: torch.Tensor) -> torch.Tensor:
    return t if rnd is None else rnd(t)


def to_bf16_and_back(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


# ----------------------------------------------------------------------------- small pieces
def plain_rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def plain_rmsnorm(x, w, eps: float):
    return plain_rms_unit(x, eps) * w


def plain_silu(z):
    return z * torch.sigmoid(z)


def plain_swiglu(h, w_gate, w_up, w_down, rnd: Rounding = None):
    a = plain_silu(h @ w_gate.T) * (h @ w_up.T)
    return _r(rnd, a) @ w_down.T


# ----------------------------------------------------------------------------- routed experts
def plain_router(h, w_router, top: int):
    """(ids [T, top], weights [T, top]): the ``top`` largest sigmoid scores of every token, as they are."""
    s = torch.sigmoid(h @ w_router.T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val


def plain_moe(h, W: Dict[str, torch.Tensor], p: str, experts: int, top: int, rnd: Rounding = None):
    """out[t] = sum over the chosen experts e of expert_e(score_e * h[t])."""
    idx, val = plain_router(h, W[p + ".router"], top)
    out = torch.zeros(h.shape[0], W[p + ".e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            xin = _r(rnd, (val[t, j] * h[t]).unsqueeze(0))
            out[t] += plain_swiglu(xin, W[f"{p}.e{e}.gate"], W[f"{p}.e{e}.up"], W[f"{p}.e{e}.down"], rnd)[0]
    return out


# ----------------------------------------------------------------------------- gated delta rule
def plain_short_conv(x: torch.Tensor, w: torch.Tensor, before: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], w [C, taps]: y[t, c] = sum_j w[c, j] * x[t - (taps - 1) + j, c], the last tap on the token
    itself; ``before`` [taps - 1, C] holds the inputs ahead of the first row (zeros at the start)."""
    taps = w.shape[1]
    pad = torch.zeros(taps - 1, x.shape[1], dtype=x.dtype) if before is None else before
    xp = torch.cat([pad, x], dim=0)
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + xp[j:j + x.shape[0]] * w[:, j]
    return y


def plain_unit(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def plain_delta_decay(h, w_a1, w_a2, dt_bias, a_log, heads: int, D: int):
    """[T, heads, D] in (0, 1): exp(-exp(A_log[head]) * softplus(low-rank projection + bias))."""
    z = (h @ w_a1.T) @ w_a2.T + dt_bias
    sp = torch.nn.functional.softplus(z).view(-1, heads, D)
    return torch.exp(-torch.exp(a_log).view(1, heads, 1) * sp)


def plain_delta_recurrence(q, k, v, g, beta, state=None):
    """q, k, g: [T, heads, D]; v: [T, heads, Dv]; beta [T, heads].  Token by token per head: the rows of S
    shrink by g; the value the state already predicts for k is taken off v and the rest, times beta, is
    written along k; the read-out with q sees that write."""
    T, Hh, D = q.shape
    Dv = v.shape[-1]
    S = torch.zeros(Hh, D, Dv, dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros(T, Hh, Dv, dtype=q.dtype)
    for t in range(T):
        S = g[t].unsqueeze(-1) * S
        pred = (S * k[t].unsqueeze(-1)).sum(dim=1)                   # S^T k  [heads, Dv]
        u = beta[t].unsqueeze(-1) * (v[t] - pred)
        S = S + k[t].unsqueeze(-1) * u.unsqueeze(-2)
        o[t] = (S * q[t].unsqueeze(-1)).sum(dim=1)
    return o, S


def plain_channel_delta(h, W, p: str, m: dict, eps: float, rnd: Rounding = None):
    T = h.shape[0]
    heads, kvh, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rep = heads // kvh
    q = plain_silu(plain_short_conv(h @ W[p + ".q"].T, W[p + ".q.conv"])).view(T, kvh, D)
    k = plain_silu(plain_short_conv(h @ W[p + ".k"].T, W[p + ".k.conv"])).view(T, kvh, D)
    v = plain_silu(plain_short_conv(h @ W[p + ".v"].T, W[p + ".v.conv"])).view(T, heads, Dv)
    q = (plain_unit(q) * D ** -0.5).repeat_interleave(rep, dim=1)
    k = plain_unit(k).repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ W[p + ".b"].T)
    g = plain_delta_decay(h, W[p + ".a1"], W[p + ".a2"], W[p + ".dt_bias"], W[p + ".A_log"], heads, D)
    o, _ = plain_delta_recurrence(q, k, v, g, beta)
    gate = torch.sigmoid((h @ W[p + ".g1"].T) @ W[p + ".g2"].T).view(T, heads, Dv)
    y = plain_rms_unit(o, eps) * W[p + ".norm"] * gate
    return _r(rnd, y.reshape(T, heads * Dv)) @ W[p + ".o"].T


# ----------------------------------------------------------------------------- latent attention
def plain_rotary_tables(positions: torch.Tensor, dims: int, base: float, scaling: Optional[dict], dtype=torch.float64):
    """(cos, sin) [T, dims / 2].  With ``scaling`` (factor, original, fast, slow) the slow pairs turn ``factor``
    times slower, the fast ones keep their speed, a linear ramp in between, and both tables are stretched by
    0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    if scaling:
        fac = float(scaling["factor"])

        def at(turns):
            return dims * math.log(scaling["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

        lo = max(math.floor(at(scaling["fast"])), 0)
        hi = min(math.ceil(at(scaling["slow"])), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / fac * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(fac) + 1.0
    ang = positions.to(torch.float64).unsqueeze(-1) * f
    return (torch.cos(ang) * mult).to(dtype), (torch.sin(ang) * mult).to(dtype)


def plain_rotate_pairs(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dims: int) -> torch.Tensor:
    """x [T, ..., n]: neighbours (2i, 2i + 1) of the first ``dims`` entries turn by the angle of pair i."""
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = cos.view(shape), sin.view(shape)
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def plain_window(T: int, size: int, first: int = 0) -> torch.Tensor:
    """[T, T] mask: query i sees key j iff 0 <= i - j < size (size 0: every earlier key)."""
    pos = torch.arange(first, first + T)
    d = pos[:, None] - pos[None, :]
    return (d >= 0) & ((d < size) if size > 0 else torch.ones_like(d, dtype=torch.bool))


def plain_sink_softmax(s: torch.Tensor, sink: float) -> torch.Tensor:
    """Softmax along the last axis whose denominator holds one more term exp(sink) that has no value."""
    m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=sink)
    e = torch.exp(s - m)
    return e / (e.sum(dim=-1, keepdim=True) + math.exp(sink) * torch.exp(-m))


def plain_latent_kv(h, W, p: str, m: dict, eps: float, positions, rnd: Rounding = None):
    """What a layer with its own down-projection caches: (latent [T, kv_rank], rotated key part [T, rot_dim])."""
    R, rd = m["kv_rank"], m["rot_dim"]
    d = h @ W[p + ".dkv"].T
    c = plain_rmsnorm(d[:, :R], W[p + ".dkv.norm"], eps)
    rot = m.get("rot") or {}
    dims = rot.get("dims", rd)
    cos, sin = plain_rotary_tables(positions, dims, rot.get("base", 10000.0), rot.get("scaling"), h.dtype)
    kr = plain_rotate_pairs(d[:, R:R + rd], cos, sin, dims)
    return _r(rnd, c), _r(rnd, kr)


def plain_latent_attention(h, W, p: str, m: dict, eps: float, c, kr, positions, rnd: Rounding = None,
                           in_latent_space: Optional[bool] = None):
    """``in_latent_space`` (the default when ``rnd`` is given): the same sums associated the other way, with the
    query's unrotated part carried through Wuk^T and Wuv applied to the weighted sum of latents, which is where the
    bfloat16 engine rounds."""
    if in_latent_space is None:
        in_latent_space = rnd is not None
    T = h.shape[0]
    H, D, rd, Dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = _r(rnd, plain_rmsnorm(h @ W[p + ".dq"].T, W[p + ".dq.norm"], eps))
    q = (cq @ W[p + ".uq"].T).view(T, H, D + rd)
    rot = m.get("rot") or {}
    dims = rot.get("dims", rd)
    cos, sin = plain_rotary_tables(positions, dims, rot.get("base", 10000.0), rot.get("scaling"), h.dtype)
    qn, qr = q[..., :D], plain_rotate_pairs(q[..., D:], cos, sin, dims)
    kn = (c @ W[p + ".uk"].T).view(T, H, D)
    v = (c @ W[p + ".uv"].T).view(T, H, Dv)
    vis = plain_window(T, (m.get("mask") or {}).get("size", 0))
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    wuk, wuv = W[p + ".uk"].view(H, D, -1), W[p + ".uv"].view(H, Dv, -1)
    for hd in range(H):
        if in_latent_space:
            qa = _r(rnd, _r(rnd, qn[:, hd]) @ wuk[hd])                        # [T, R]
            s = (qa @ c.T + _r(rnd, qr[:, hd]) @ kr.T) * m["scale"]
        else:
            s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * m["scale"]
        s = s.masked_fill(~vis, -math.inf)
        pr = plain_sink_softmax(s, float(W[p + ".sink"][hd]))
        out[:, hd] = _r(rnd, pr @ c) @ wuv[hd].T if in_latent_space else pr @ v[:, hd]
    return _r(rnd, out.reshape(T, H * Dv)) @ W[p + ".o"].T


# ----------------------------------------------------------------------------- wkv
def plain_wkv_recurrence(r, k, v, w, u, state=None):
    """r, k, v, w: [T, heads, D]; u [heads, D].  o_t reads the state BEFORE the token plus the token's own outer
    product weighted by u; then the rows of the state shrink by w_t and the outer product is added."""
    T, Hh, D = r.shape
    S = torch.zeros(Hh, D, D, dtype=r.dtype) if state is None else state.clone()
    o = torch.zeros(T, Hh, D, dtype=r.dtype)
    for t in range(T):
        kv = k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = ((S + u.unsqueeze(-1) * kv) * r[t].unsqueeze(-1)).sum(dim=1)
        S = w[t].unsqueeze(-1) * S + kv
    return o, S


def plain_wkv(h, W, p: str, m: dict, eps: float, rnd: Rounding = None):
    T = h.shape[0]
    heads, D = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, h.shape[1], dtype=h.dtype), h[:-1]], dim=0)
    mix = {s: _r(rnd, h + (prev - h) * W[f"{p}.mu.{s}"]) for s in "rkvgw"}
    r = (mix["r"] @ W[p + ".r"].T).view(T, heads, D)
    k = (mix["k"] @ W[p + ".k"].T).view(T, heads, D)
    v = (mix["v"] @ W[p + ".v"].T).view(T, heads, D)
    gate = plain_silu(mix["g"] @ W[p + ".g"].T)
    w = torch.exp(-torch.exp(torch.tanh(mix["w"] @ W[p + ".w1"].T) @ W[p + ".w2"].T + W[p + ".w0"])).view(T, heads, D)
    o, _ = plain_wkv_recurrence(r, k, v, w, W[p + ".u"])
    y = plain_rms_unit(o, eps).reshape(T, heads * D) * W[p + ".norm"] * gate
    return _r(rnd, y) @ W[p + ".o"].T


# ----------------------------------------------------------------------------- the model
def plain_forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, rnd: Rounding = None,
                  residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence.  ``residuals`` collects the stream after every layer."""
    W = {n: t.to(dtype) for n, t in W.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    T = len(tokens)
    pos = torch.arange(T)
    x = W["embed"][torch.tensor(tokens)]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = _r(rnd, x)
        if layer["type"] == "channel_delta":
            y = plain_channel_delta(h, W, p + ".mix", m, eps, rnd)
        elif layer["type"] == "latent_attention":
            if "kv_from" in m:
                c, kr = latents[m["kv_from"]]
            else:
                c, kr = latents[i] = plain_latent_kv(h, W, p + ".mix", m, eps, pos, rnd)
            y = plain_latent_attention(h, W, p + ".mix", m, eps, c, kr, pos, rnd)
        else:
            y = plain_wkv(x, W, p + ".mix", m, eps, rnd)
        x = x + mult * plain_rmsnorm(y, W[p + ".norm1"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = _r(rnd, x)
            if mlp["kind"] == "dense":
                y = plain_swiglu(h, W[p + ".mlp.gate"], W[p + ".mlp.up"], W[p + ".mlp.down"], rnd)
            else:
                y = plain_moe(h, W, p + ".mlp", mlp["router"]["experts"], mlp["router"]["top"], rnd)
            x = x + mult * plain_rmsnorm(y, W[p + ".norm2"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return _r(rnd, plain_rmsnorm(x, W["final.norm"], eps)) @ W["head"].T


def plain_greedy(cfg, W, prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(plain_forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]


# ----------------------------------------------------------------------------- configurations and weights
def dense(ff: int) -> dict:
    return dict(kind="dense", ff=ff)


def moe(ff: int, experts: int, top: int) -> dict:
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def delta_layer(heads, kv_heads, dim, vdim, conv, mlp=None) -> dict:
    return dict(type="channel_delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv), mlp=mlp)


def latent_layer(heads, dim, rot_dim, vdim, q_rank, kv_rank, window=None, scale=None, base=10000.0, scaling=None,
                 kv_from=None, mlp=None) -> dict:
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank,
             scale=scale if scale is not None else (dim + rot_dim) ** -0.5, rot=dict(dims=rot_dim, base=base))
    if scaling is not None:
        m["rot"]["scaling"] = dict(factor=scaling[0], original=scaling[1], fast=scaling[2], slow=scaling[3])
    if window is not None:
        m["mask"] = dict(size=window)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m, mlp=mlp)


def wkv_layer(heads, dim, mlp=None) -> dict:
    return dict(type="wkv", mixer=dict(heads=heads, dim=dim), mlp=mlp)


def all_experts(cfg: dict) -> dict:
    """The same model with every router choosing ALL its experts (the scores still weigh them): a choice that no
    rounding can change, for comparisons in reduced precision."""
    out = json.loads(json.dumps(cfg))
    for l in out["layers"]:
        if l.get("mlp") and l["mlp"]["kind"] == "moe":
            l["mlp"]["router"]["top"] = l["mlp"]["router"]["experts"]
    return out


def make_config(vocab, width, layers, eps=1e-5, mult=0.7) -> dict:
    return dict(architecture="Pogarax", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, layers=layers)


def tensor_shapes(cfg: dict, ranks=(6, 5, 4)) -> Dict[str, tuple]:
    """name -> shape of every tensor of a model; ``ranks``: of the delta rule's decay pair and gate pair, and of the
    time mix's decay pair."""
    Wd, shapes = cfg["width"], {}
    shapes["embed"] = (cfg["vocab"], Wd)
    shapes["head"] = (cfg["vocab"], Wd)
    shapes["final.norm"] = (Wd,)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}", l["mixer"]
        shapes[p + ".norm1"] = (Wd,)
        x = p + ".mix."
        if l["type"] == "channel_delta":
            kd, vd, hd = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m["heads"] * m["dim"]
            shapes.update({x + "q": (kd, Wd), x + "k": (kd, Wd), x + "v": (vd, Wd), x + "q.conv": (kd, m["conv"]),
                           x + "k.conv": (kd, m["conv"]), x + "v.conv": (vd, m["conv"]), x + "b": (m["heads"], Wd),
                           x + "A_log": (m["heads"],), x + "norm": (m["vdim"],), x + "a1": (ranks[0], Wd), x + "a2": (hd, ranks[0]),
                           x + "dt_bias": (hd,), x + "g1": (ranks[1], Wd), x + "g2": (vd, ranks[1]), x + "o": (Wd, vd)})
        elif l["type"] == "latent_attention":
            H, D, rd, Dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            shapes.update({x + "dq": (m["q_rank"], Wd), x + "dq.norm": (m["q_rank"],), x + "uq": (H * (D + rd), m["q_rank"]),
                           x + "uk": (H * D, R), x + "uv": (H * Dv, R), x + "sink": (H,), x + "o": (Wd, H * Dv)})
            if "kv_from" not in m:
                shapes.update({x + "dkv": (R + rd, Wd), x + "dkv.norm": (R,)})
        else:
            hd = m["heads"] * m["dim"]
            shapes.update({x + f"mu.{s}": (Wd,) for s in "rkvgw"})
            shapes.update({x + s: (hd, Wd) for s in "rkvg"})
            shapes.update({x + "w1": (ranks[2], Wd), x + "w2": (hd, ranks[2]), x + "w0": (hd,), x + "u": (m["heads"], m["dim"]),
                           x + "norm": (hd,), x + "o": (Wd, hd)})
        mlp = l.get("mlp")
        if mlp:
            shapes[p + ".norm2"] = (Wd,)
            if mlp["kind"] == "dense":
                shapes.update({p + ".mlp.gate": (mlp["ff"], Wd), p + ".mlp.up": (mlp["ff"], Wd), p + ".mlp.down": (Wd, mlp["ff"])})
            else:
                ff = mlp["expert"]["ff"]
                shapes[p + ".mlp.router"] = (mlp["router"]["experts"], Wd)
                for e in range(mlp["router"]["experts"]):
                    shapes.update({f"{p}.mlp.e{e}.gate": (ff, Wd), f"{p}.mlp.e{e}.up": (ff, Wd), f"{p}.mlp.e{e}.down": (Wd, ff)})
    return shapes


def random_weights(cfg: dict, seed: int, ranks=(6, 5, 4), gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """Weights large enough that every mechanism moves the logits: matrices N(0, gain^2 / fan_in), norm weights
    near 1, decays spread between slow and fast, sinks, bonuses and blends of a visible size; all rounded to
    bfloat16, the file's type."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg, ranks).items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith(".conv"):
            t = 0.6 * torch.randn(shape, generator=g)
        elif ".mu." in name:
            t = torch.rand(shape, generator=g)
        elif len(shape) == 2 and leaf != "u":
            std = 1.0 if name == "embed" else gain / math.sqrt(shape[1])
            if leaf in ("a2", "g2", "w2", "router"):
                std *= 2.0
            t = torch.randn(shape, generator=g) * std
        elif leaf.startswith("norm") or name == "final.norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "A_log":
            t = torch.randn(shape, generator=g) - 1.0
        elif leaf == "w0":
            t = torch.randn(shape, generator=g) - 2.0
        elif leaf == "sink":
            t = torch.randn(shape, generator=g) + 0.5
        else:                                               # dt_bias, u
            t = 0.5 * torch.randn(shape, generator=g)
        W[name] = t.to(torch.bfloat16)
    return W


def write_folder(folder: str, cfg: dict, W: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({n: t.contiguous() for n, t in W.items()}, os.path.join(folder, "model.safetensors"))
    return folder
