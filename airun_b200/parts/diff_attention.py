"""Differential attention over paged keys and values.

Every query head has two query vectors of size D and every KV head two key vectors (laid out head by
head as [map 1, map 2]) and one value vector of size Dv; query head h reads KV head h / (heads / kv_heads).
Each map is a softmax attention of its own over the same values:

    q = Wq h + bq,  k = Wk h + bk,  v = Wv h + bv          (no position encoding)
    s_m = scale * q_m . k_m;  with a soft cap c:  s_m <- c * tanh(s_m / c)
    a_m = softmax over the visible keys (s_m) V
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init      (one number for the layer)
    o = a_1 - lambda * a_2;   o <- o / rms(o) * (1 - lambda_init)   per head, without a weight
    out = Wo concat_heads(o)

Key j is visible to position i iff j <= i and, with ``chunk`` C > 0, both lie in the same block of C
positions counted from the start of the sequence (and, with ``window`` w > 0, i - j < w).  The three
input projections run as one product; keys and values go into pages whose key rows have 2*D elements
and value rows Dv (``PagedKVSpec.value_dim``).  The part has the split form (parts/base.py).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Mixer, PagedKVSpec, register_part
from .linear import linear


class DifferentialAttention(Mixer):
    device_driven = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                 scale: float, lambda_init: float, norm_eps: float, soft_cap: float = 0.0, chunk: int = 0, window: int = 0,
                 bias: bool = True, dtype: torch.dtype = torch.bfloat16, device=None,
                 names: Optional[Dict[str, str]] = None):
        self.prefix, self.H = prefix, int(hidden_size)
        self.nh, self.nkv, self.D, self.Dv = int(num_heads), int(num_kv_heads), int(head_dim), int(value_dim)
        if min(self.nh, self.nkv, self.D, self.Dv) <= 0:
            raise ValueError("head counts and sizes must be positive")
        if self.nh % self.nkv:
            raise ValueError(f"heads ({num_heads}) must be a multiple of kv_heads ({num_kv_heads})")
        if self.D > 256 or self.Dv > 256:
            raise ValueError("head sizes above 256 are beyond the attention kernels")
        self.scale, self.cap = float(scale), float(soft_cap or 0.0)
        self.lambda_init, self.eps = float(lambda_init), float(norm_eps)
        self.chunk, self.window, self.bias = int(chunk or 0), int(window or 0), bool(bias)
        self.dtype, self.device = dtype, device
        n = dict(q="q", k="k", v="v", o="o", q_bias="q.b", k_bias="k.b", v_bias="v.b",
                 lq1="lq1", lk1="lk1", lq2="lq2", lk2="lk2")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_in = self.w_q = self.w_out = self.q_b = self.k_b = self.v_b = None
        self.lam = self.lambda_init
        self.core_width = self.nh * self.Dv

    # ---- weights ----
    def weight_specs(self) -> List[WeightSpec]:
        nm, H, qw, kw, vw = self.names, self.H, self.nh * 2 * self.D, self.nkv * 2 * self.D, self.nkv * self.Dv
        specs = [WeightSpec(nm["q"], (qw, H)), WeightSpec(nm["k"], (kw, H)), WeightSpec(nm["v"], (vw, H)),
                 WeightSpec(nm["o"], (H, self.nh * self.Dv))]
        if self.bias:
            specs += [WeightSpec(nm["q_bias"], (qw,), storage="float32"), WeightSpec(nm["k_bias"], (kw,), storage="float32"),
                      WeightSpec(nm["v_bias"], (vw,), storage="float32")]
        specs += [WeightSpec(nm[k], (self.D,), storage="float32") for k in ("lq1", "lk1", "lq2", "lk2")]
        return specs

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm = self.names
        self.w_in = torch.cat([tensors.pop(nm["q"]), tensors.pop(nm["k"]), tensors.pop(nm["v"])], dim=0).contiguous()
        self.w_q = self.w_in[: self.nh * 2 * self.D]
        self.w_out = tensors.pop(nm["o"])
        if self.bias:
            self.q_b, self.k_b, self.v_b = tensors[nm["q_bias"]], tensors[nm["k_bias"]], tensors[nm["v_bias"]]
        # lambda is a constant of the layer once the weights are known: float32 products summed in double
        l = [tensors[nm[k]].detach().to("cpu", torch.float32) for k in ("lq1", "lk1", "lq2", "lk2")]
        s1 = float((l[0] * l[1]).double().sum())
        s2 = float((l[2] * l[3]).double().sum())
        self.lam = math.exp(s1) - math.exp(s2) + self.lambda_init

    def adopt_w_out(self, view: torch.Tensor) -> None:
        self.w_out = view

    # ---- cache ----
    def cache_spec(self):
        return PagedKVSpec(self.nkv, 2 * self.D, self.window, value_dim=self.Dv if self.Dv != 2 * self.D else 0)

    # ---- compute ----
    def forward_core(self, ctx, h: torch.Tensor, act: torch.Tensor, cache) -> None:
        T, ws = h.shape[0], ctx.ws
        owns = not cache.shared
        qw, kd = self.nh * 2 * self.D, 2 * self.D
        width = qw + (self.nkv * (kd + self.Dv) if owns else 0)
        proj = ws.alloc((T, width), torch.float32)
        linear(ctx, h, self.w_in if owns else self.w_q, proj)
        q = ws.alloc((T, qw), self.dtype)
        ops.qkv_bias_store(proj, self.q_b, self.k_b, self.v_b, q, cache.pool, cache.block_table, ctx.positions,
                           ctx.req_of_token, ctx.num_reqs, cache.page_size, qw, self.nkv, kd, self.Dv, ctx.err, store=owns)
        self.attend(ctx, q, act, cache)

    def attend(self, ctx, q: torch.Tensor, out: torch.Tensor, cache) -> None:
        if q.dtype == torch.bfloat16:
            from ..kernels import fast
            if fast.diff_attention_bf16(ctx, q, out, cache, self):
                return
        ops.diff_attention(q, out, cache.pool, cache.block_table, ctx.positions, ctx.req_of_token, ctx.num_reqs,
                           cache.page_size, self.nh, self.nkv, self.D, self.Dv, self.scale, self.cap, self.chunk,
                           self.window, self.lam, self.eps, 1.0 - self.lambda_init, ctx.err)

    def forward(self, ctx, h, cache, sink=None):
        T = h.shape[0]
        act = ctx.ws.alloc((T, self.core_width), self.dtype)
        self.forward_core(ctx, h, act, cache)
        delta = ctx.ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_out, delta)
        return delta


register_part("mixer", "differential_attention", DifferentialAttention)
