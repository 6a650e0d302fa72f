"""A plain, slow implementation of the Vedizen decoder for the tests: whole sequences, no cache, torch on
the CPU in float64 unless told otherwise, one function per mechanism.  It shares no code with the package.

Notation: T tokens, width W; a linear weight is [out, in] and applied as x @ w.T.  ``rnd`` (optional) rounds
a tensor where the bfloat16 engine stores one in bfloat16 (the normed input of a layer, q, keys, values and
the activations in front of the output products); it is the identity for the exact result.
"""
from __future__ import annotations

import json
import math
import os
from typing import Callable, Dict, List, Optional

import torch

Round = Optional[Callable[[torch.Tensor], torch.Tensor]]


def _r(rnd: Round, t: torch.Tensor) -> torch.Tensor:
    return t if rnd is None else rnd(t)


def to_bf16_and_back(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


# ----------------------------------------------------------------------------- mechanisms
def plain_dyt(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    """Dynamic Tanh: squash each element, then scale and shift per channel."""
    return torch.tanh(alpha * x) * weight + bias


def plain_rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def plain_clamped_glu(h, w_gate, w_up, w_down, limit: float, slope: float = 1.702, rnd: Round = None):
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, min=-limit, max=limit)
    a = g * torch.sigmoid(slope * g) * (u + 1.0)
    return _r(rnd, a) @ w_down.T


def plain_gla_decay(h, w_a1, w_a2, b_a2, tau: float) -> torch.Tensor:
    """Per-channel decay in (0, 1): the tau-th root of a sigmoid of a low-rank projection."""
    z = (h @ w_a1.T) @ w_a2.T + b_a2
    return torch.exp(torch.nn.functional.logsigmoid(z) / tau)


def plain_gla_recurrence(q, k, v, decay, state=None):
    """q, k, decay: [T, heads, D]; v: [T, heads, Dv].  Returns (o [T, heads, Dv], final state [heads, D, Dv]).
    Token by token: every row d of the state shrinks by decay[d], the outer product of key and value is
    added, and the output reads the new state with the query."""
    T, Hh, D = q.shape
    Dv = v.shape[-1]
    S = torch.zeros(Hh, D, Dv, dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros(T, Hh, Dv, dtype=q.dtype)
    for t in range(T):
        S = decay[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = (S * q[t].unsqueeze(-1)).sum(dim=1)
    return o, S


def plain_gla_closed_form(q, k, v, decay):
    """The same outputs without a state: o_t = sum over s <= t of (q_t * prod_{s < r <= t} decay_r) . k_s times v_s."""
    T, Hh, D = q.shape
    logc = torch.cumsum(torch.log(decay), dim=0)                  # [T, heads, D]
    o = torch.zeros(T, Hh, v.shape[-1], dtype=q.dtype)
    for t in range(T):
        w = torch.exp(logc[t].unsqueeze(0) - logc[: t + 1])       # [t+1, heads, D]
        score = (q[t].unsqueeze(0) * w * k[: t + 1]).sum(-1)      # [t+1, heads]
        o[t] = (score.unsqueeze(-1) * v[: t + 1]).sum(0)
    return o


def plain_gla(h, W: Dict[str, torch.Tensor], p: str, heads: int, D: int, Dv: int, tau: float, eps: float, rnd: Round = None):
    T = h.shape[0]
    q = (h @ W[p + ".q"].T).view(T, heads, D) * D ** -0.5
    k = (h @ W[p + ".k"].T).view(T, heads, D)
    v = (h @ W[p + ".v"].T).view(T, heads, Dv)
    a = plain_gla_decay(h, W[p + ".a1"], W[p + ".a2"], W[p + ".a2.b"], tau).view(T, heads, D)
    o, _ = plain_gla_recurrence(q, k, v, a)
    o = plain_rms_unit(o, eps) * W[p + ".norm"]
    g = h @ W[p + ".g"].T
    y = o.reshape(T, heads * Dv) * (g * torch.sigmoid(g))
    return _r(rnd, y) @ W[p + ".o"].T


def plain_visible(T: int, chunk: int, first: int = 0) -> torch.Tensor:
    """[T, T] mask: query i (at position first + i) sees key j iff j <= i and both lie in the same block of
    ``chunk`` positions counted from position 0 (chunk 0: plain causal)."""
    pos = torch.arange(first, first + T)
    vis = pos[None, :] <= pos[:, None]
    if chunk > 0:
        vis = vis & ((pos[None, :] // chunk) == (pos[:, None] // chunk))
    return vis


def plain_diff_lambda(W, p: str, init: float) -> float:
    f = lambda n: float((W[p + ".lq" + n].double() * W[p + ".lk" + n].double()).sum())
    return math.exp(f("1")) - math.exp(f("2")) + init


def plain_diff_attention(h, W, p: str, heads: int, kv_heads: int, D: int, Dv: int, scale: float, cap: float,
                         init: float, chunk: int, eps: float, rnd: Round = None):
    T = h.shape[0]
    q = _r(rnd, h @ W[p + ".q"].T + W[p + ".q.b"]).view(T, heads, 2, D)
    k = _r(rnd, h @ W[p + ".k"].T + W[p + ".k.b"]).view(T, kv_heads, 2, D)
    v = _r(rnd, h @ W[p + ".v"].T + W[p + ".v.b"]).view(T, kv_heads, Dv)
    lam = plain_diff_lambda(W, p, init)
    vis = plain_visible(T, chunk)
    out = torch.zeros(T, heads, Dv, dtype=h.dtype)
    for hd in range(heads):
        g = hd // (heads // kv_heads)
        maps = []
        for m in range(2):
            s = (q[:, hd, m] @ k[:, g, m].T) * scale
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            s = s.masked_fill(~vis, -math.inf)
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        out[:, hd] = plain_rms_unit(maps[0] - lam * maps[1], eps) * (1.0 - init)
    return _r(rnd, out.reshape(T, heads * Dv)) @ W[p + ".o"].T


# ----------------------------------------------------------------------------- the model
def plain_order(cfg: dict):
    """[(layer, pass or None)]: the pass number stands at the first layer of each pass of the loop."""
    L = len(cfg["layers"])
    loop = cfg.get("loop") or dict(start=0, stop=0, times=1)
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], L)]


def plain_forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, rnd: Round = None,
                  residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence."""
    W = {n: t.to(dtype) for n, t in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, step in plain_order(cfg):
        if step is not None:
            x = x + W["loop.step"][step]
        layer, p = cfg["layers"][i], f"l{i}"
        m = layer["mixer"]
        h = _r(rnd, plain_dyt(x, W[p + ".norm1"], W[p + ".norm1.b"], W[p + ".norm1.alpha"]))
        if layer["type"] == "gla":
            y = plain_gla(h, W, p + ".mix", m["heads"], m["dim"], m["vdim"], m["tau"], eps, rnd)
        else:
            y = plain_diff_attention(h, W, p + ".mix", m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"],
                                     m["softcap"], m["diff"], m["mask"]["size"], eps, rnd)
        if layer.get("mlp"):
            y = y + plain_clamped_glu(h, W[p + ".mlp.gate"], W[p + ".mlp.up"], W[p + ".mlp.down"], layer["mlp"]["limit"], rnd=rnd)
        x = x + y
        if residuals is not None:
            residuals.append(x.clone())
    h = _r(rnd, plain_dyt(x, W["final.norm"], W["final.norm.b"], W["final.norm.alpha"]))
    return h @ W["head"].T


def plain_greedy(cfg, W, prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(plain_forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]


# ----------------------------------------------------------------------------- configurations and weights
def gla_layer(heads, dim, vdim, tau, ff=None, limit=1.5):
    return dict(type="gla", mixer=dict(heads=heads, dim=dim, vdim=vdim, tau=tau),
                mlp=None if ff is None else dict(kind="dense", ff=ff, limit=limit))


def attention_layer(heads, kv_heads, dim, vdim, chunk, scale=None, softcap=20.0, diff=0.3, ff=None, limit=1.5):
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale or dim ** -0.5,
                                             softcap=softcap, diff=diff, mask=dict(size=chunk)),
                mlp=None if ff is None else dict(kind="dense", ff=ff, limit=limit))


def make_config(vocab, width, layers, loop=None, scale=1.0, eps=1e-5) -> dict:
    cfg = dict(architecture="Vedizen", vocab=vocab, width=width, embedding=dict(scale=scale), norm=dict(eps=eps), layers=layers)
    if loop is not None:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


def tensor_shapes(cfg: dict, rank: int = 8) -> Dict[str, tuple]:
    Wd, shapes = cfg["width"], {}
    shapes["embed"] = (cfg["vocab"], Wd)
    shapes["head"] = (cfg["vocab"], Wd)
    loop = cfg.get("loop")
    if loop and loop["times"] > 0 and loop["stop"] > loop["start"]:
        shapes["loop.step"] = (loop["times"], Wd)

    def norm(n):
        shapes[n], shapes[n + ".b"], shapes[n + ".alpha"] = (Wd,), (Wd,), ()

    norm("final.norm")
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}", l["mixer"]
        norm(p + ".norm1")
        if l["type"] == "gla":
            kd, vd = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            shapes.update({p + ".mix.q": (kd, Wd), p + ".mix.k": (kd, Wd), p + ".mix.v": (vd, Wd), p + ".mix.g": (vd, Wd),
                           p + ".mix.o": (Wd, vd), p + ".mix.norm": (m["vdim"],), p + ".mix.a1": (rank, Wd),
                           p + ".mix.a2": (kd, rank), p + ".mix.a2.b": (kd,)})
        else:
            qw, kw, vw = m["heads"] * 2 * m["dim"], m["kv_heads"] * 2 * m["dim"], m["kv_heads"] * m["vdim"]
            shapes.update({p + ".mix.q": (qw, Wd), p + ".mix.q.b": (qw,), p + ".mix.k": (kw, Wd), p + ".mix.k.b": (kw,),
                           p + ".mix.v": (vw, Wd), p + ".mix.v.b": (vw,), p + ".mix.o": (Wd, m["heads"] * m["vdim"])})
            for n in ("lq1", "lk1", "lq2", "lk2"):
                shapes[f"{p}.mix.{n}"] = (m["dim"],)
        if l.get("mlp"):
            shapes.update({p + ".mlp.gate": (l["mlp"]["ff"], Wd), p + ".mlp.up": (l["mlp"]["ff"], Wd),
                           p + ".mlp.down": (Wd, l["mlp"]["ff"])})
    return shapes


def random_weights(cfg: dict, seed: int, rank: int = 8, gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """Weights large enough that every mechanism moves the logits: matrices N(0, gain^2 / fan_in), norm weights near
    1, biases and offsets of a visible size; all rounded to bfloat16, the file's type."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg, rank).items():
        if len(shape) == 2:
            std = gain / math.sqrt(shape[1]) if name != "embed" else 1.0
            t = torch.randn(shape, generator=g) * std
        elif name.endswith(".alpha"):
            t = torch.tensor(0.6) + 0.2 * torch.rand((), generator=g)
        elif name.endswith("norm1") or name.endswith("final.norm") or name.endswith(".mix.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif ".mix.l" in name:
            t = 0.3 * torch.randn(shape, generator=g)
        else:
            t = 0.3 * torch.randn(shape, generator=g)
        W[name] = t.to(torch.bfloat16)
    return W


def write_folder(folder: str, cfg: dict, W: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({n: t.contiguous() for n, t in W.items()}, os.path.join(folder, "model.safetensors"))
    return folder
