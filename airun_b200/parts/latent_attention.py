"""Attention over a cached latent: a token caches one short row that all heads share.

With h the mixer's input, H heads of D unrotated and rd rotated query/key dimensions, value size Dv, latent size R:

    cq = rmsnorm(Wdq h) * w_dq,        q_h = Wuq cq                    head by head [D unrotated | rd rotated]
    [d | kr] = Wdkv h,                 c = rmsnorm(d) * w_dkv          c (R) and the rotated kr (rd) are cached
    k_h(j) = (Wuk_h c_j, kr_j),        v_h(j) = Wuv_h c_j
    s = scale * (q_h . k_h(j)),  key j visible iff 0 <= i - j < window  (window 0: every j <= i)
    p = exp(s) / (sum_visible exp(s) + exp(sink_h)),    o_h = sum_j p_j v_h(j),    out = Wo concat_heads(o)

The up-projections never touch the cache: the unrotated query is carried into the latent space,
qa_h = Wuk_h^T qn_h, so that s = scale * (qa_h . c_j + qr_h . kr_j), the weighted sum is taken over the cached c_j
and Wuv_h is applied to it afterwards.  The position encoding (a registered ``position`` part with the
interleaved pairing) turns the first ``rot_dims`` of the rd rotated dimensions of q and kr.  A layer that reads
another layer's cache (``cache.shared``) has no Wdkv: it attends over the owner's rows with its own Wuk, Wuv,
queries, window and sinks; ``cache_window`` is the longest window of all layers on one cache (0: unbounded) and
tells the cache manager how long rows have to be kept.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Mixer, PagedKVSpec, make_part, register_part
from .linear import linear


class LatentAttention(Mixer):
    device_driven = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int,
                 q_rank: int, kv_rank: int, scale: float, norm_eps: float, window: int = 0, cache_window: Optional[int] = None,
                 sink: bool = True, owns_cache: bool = True, position: str = "rotary_scaled_interleaved",
                 position_args: Optional[dict] = None, dtype: torch.dtype = torch.bfloat16, device=None,
                 names: Optional[Dict[str, str]] = None):
        self.prefix, self.H = prefix, int(hidden_size)
        self.nh, self.D, self.rd, self.Dv = int(num_heads), int(head_dim), int(rot_dim), int(value_dim)
        self.q_rank, self.R = int(q_rank), int(kv_rank)
        if min(self.nh, self.D, self.Dv, self.q_rank, self.R) <= 0 or self.rd < 0:
            raise ValueError("heads, head sizes and ranks must be positive")
        if self.R + self.rd > 640:
            raise ValueError(f"a cached row of {self.R + self.rd} elements is above the attention kernel's limit of 640")
        self.scale, self.eps = float(scale), float(norm_eps)
        self.window = int(window or 0)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        self.has_sink, self.owns = bool(sink), bool(owns_cache)
        self.dtype, self.device = dtype, device
        self.pos = make_part("position", position, prefix=prefix, dtype=dtype, device=device, **(position_args or {}))
        kind, self.rot_dims, self.inv_freq = self.pos.fused()
        if kind not in (ops.ROPE_NONE, ops.ROPE_INTERLEAVED):
            raise ValueError("the latent attention rotates neighbouring dimensions (the interleaved pairing) or nothing")
        if self.rot_dims > self.rd:
            raise ValueError(f"{self.rot_dims} rotated dimensions do not fit a rotated part of {self.rd}")
        self.rot_mult = float(getattr(self.pos, "mult", 1.0))
        n = dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", sink="sink", o="o")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_in = self.w_dq = self.w_uq = self.w_ukT = self.w_uv = self.w_out = None
        self.dq_norm = self.dkv_norm = self.sink = None

    # ---- weights ----
    def weight_specs(self) -> List[WeightSpec]:
        nm, H, nh = self.names, self.H, self.nh
        specs = [WeightSpec(nm["dq"], (self.q_rank, H)), WeightSpec(nm["dq_norm"], (self.q_rank,), storage="float32", init="norm"),
                 WeightSpec(nm["uq"], (nh * (self.D + self.rd), self.q_rank)),
                 WeightSpec(nm["uk"], (nh * self.D, self.R)), WeightSpec(nm["uv"], (nh * self.Dv, self.R)),
                 WeightSpec(nm["o"], (H, nh * self.Dv))]
        if self.owns:
            specs += [WeightSpec(nm["dkv"], (self.R + self.rd, H)),
                      WeightSpec(nm["dkv_norm"], (self.R,), storage="float32", init="norm")]
        if self.has_sink:
            specs.append(WeightSpec(nm["sink"], (nh,), storage="float32"))
        return specs

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm = self.names
        if self.owns:
            self.w_in = torch.cat([tensors.pop(nm["dq"]), tensors.pop(nm["dkv"])], dim=0).contiguous()
            self.w_dq = self.w_in[: self.q_rank]
            self.dkv_norm = tensors[nm["dkv_norm"]]
        else:
            self.w_dq = tensors.pop(nm["dq"])
        self.dq_norm = tensors[nm["dq_norm"]]
        self.w_uq = tensors.pop(nm["uq"])
        # Wuk per head, transposed: [H, R, D], so that qa_h = Wuk_h^T qn_h is a product over rows of length D
        self.w_ukT = tensors.pop(nm["uk"]).view(self.nh, self.D, self.R).transpose(1, 2).contiguous()
        self.w_uv = tensors.pop(nm["uv"]).view(self.nh, self.Dv, self.R).contiguous()
        self.w_out = tensors.pop(nm["o"])
        self.sink = tensors[nm["sink"]] if self.has_sink else None

    # ---- cache ----
    def cache_spec(self):
        return PagedKVSpec(1, self.R + self.rd, self.cache_window, values=False)

    # ---- compute ----
    def forward(self, ctx, h: torch.Tensor, cache, sink=None):
        T, ws, nh, R, rd = h.shape[0], ctx.ws, self.nh, self.R, self.rd
        store = self.owns and not cache.shared
        proj = ws.alloc((T, self.q_rank + ((R + rd) if store else 0)), torch.float32)
        linear(ctx, h, self.w_in if store else self.w_dq, proj)
        cq = ws.alloc((T, self.q_rank), self.dtype)
        ops.latent_prepare(proj, self.dq_norm, self.dkv_norm, self.eps, cq, R, rd, self.rot_dims, self.inv_freq, self.rot_mult,
                           cache, ctx, store)
        q = ws.alloc((T, nh * (self.D + rd)), torch.float32)
        linear(ctx, cq, self.w_uq, q)
        qn = ws.alloc((T, nh * self.D), self.dtype)
        qlat = ws.alloc((T, nh * (R + rd)), self.dtype)
        ops.latent_query(q, qn, qlat, nh, self.D, R, rd, self.rot_dims, self.inv_freq, self.rot_mult, ctx)
        head_linear(ctx, qn.view(T, nh, self.D), self.w_ukT, qlat.view(T, nh, R + rd)[:, :, :R])
        olat = ws.alloc((T, nh * R), self.dtype)
        self.attend(ctx, qlat, olat, cache)
        attn = ws.alloc((T, nh * self.Dv), self.dtype)
        head_linear(ctx, olat.view(T, nh, R), self.w_uv, attn.view(T, nh, self.Dv))
        delta = ws.alloc((T, self.H), torch.float32)
        linear(ctx, attn, self.w_out, delta)
        return delta

    def attend(self, ctx, qlat: torch.Tensor, out: torch.Tensor, cache) -> None:
        if qlat.dtype == torch.bfloat16:
            from ..kernels import fast
            if fast.latent_attention_bf16(ctx, qlat, out, cache, self):
                return
        ops.latent_attention(qlat, out, cache, ctx, self.nh, self.R, self.rd, self.scale, self.window, self.sink)


def head_linear(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[:, h, :] = x[:, h, :] @ w[h]^T for every head: x [T, heads, K], w [heads, N, K], out [T, heads, N]
    (x and out may be column slices of wider rows).  Prompt portions in bfloat16 run head by head on the tensor
    cores where the slices are aligned for them; everything else is one launch of the plain batched product."""
    T, heads, K = x.shape
    if (x.dtype == torch.bfloat16 and T > HEAD_LOOP_MIN_TOKENS and K % 8 == 0 and x.stride(0) % 8 == 0
            and (x.stride(1) * 2) % 16 == 0 and x.data_ptr() % 16 == 0):
        from ..kernels import fast
        if all(fast.linear_bf16(ctx, x[:, h], w[h], out[:, h]) for h in range(heads)):
            return
    ops.gemm_simt_batched(x, w, out)


HEAD_LOOP_MIN_TOKENS = 128


register_part("mixer", "latent_attention", LatentAttention)
