"""Time mix with a matrix state per head and a bonus for the current token.

With x the mixer's input and x' the input of the token before (zero for a request's first token), each of the five
projections reads its own blend x + (x' - x) * mu_s:

    r, k, v = Wr m_r, Wk m_k, Wv m_v       (heads x D each),   gate = silu(Wg m_g)
    w = exp(-exp(Ww2 tanh(Ww1 m_w) + w0))   a decay per head and key channel
    o_t = (S + diag(u) k_t v_t^T)^T r_t,    then  S <- diag(w_t) S + k_t v_t^T      (per head; S starts at zero)
    out = Wo ( concat_heads(o / rms(o)) * w_norm * gate )

The blends are formed from the float32 input (``input_float32``), the decay, the recurrence, the norm and the gate
are float32.  A request's matrices and its last token's x live side by side in its slot of the state tensor.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Mixer, StateSpec, register_part
from .linear import linear

MIXES = ("r", "k", "v", "g", "w")


class TimeMix(Mixer):
    device_driven = True
    input_float32 = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, decay_rank: int, norm_eps: float,
                 dtype: torch.dtype = torch.bfloat16, device=None, names: Optional[Dict[str, str]] = None):
        self.prefix, self.H = prefix, int(hidden_size)
        self.nh, self.D, self.rank = int(num_heads), int(head_dim), int(decay_rank)
        if min(self.nh, self.D, self.rank) <= 0:
            raise ValueError("heads, head size and decay rank must be positive")
        if self.D > 256:
            raise ValueError(f"{self.D} channels a head are above the recurrence kernel's limit of 256")
        self.eps = float(norm_eps)
        self.dtype, self.device = dtype, device
        n = dict(r="r", k="k", v="v", g="g", o="o", decay_in="w1", decay_out="w2", decay_bias="w0", bonus="u", norm="norm")
        n.update({f"mu_{s}": f"mu.{s}" for s in MIXES})
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.hd = self.nh * self.D
        self.state_matrix = self.nh * self.D * self.D
        self.mu = self.w_r = self.w_k = self.w_v = self.w_g = self.w_w1 = self.w_w2 = self.w0 = self.bonus = None
        self.norm_w = self.w_out = None

    def weight_specs(self) -> List[WeightSpec]:
        nm, H, hd = self.names, self.H, self.hd
        return ([WeightSpec(nm[f"mu_{s}"], (H,), storage="float32") for s in MIXES] +
                [WeightSpec(nm[s], (hd, H)) for s in ("r", "k", "v", "g")] +
                [WeightSpec(nm["decay_in"], (self.rank, H)), WeightSpec(nm["decay_out"], (hd, self.rank)),
                 WeightSpec(nm["decay_bias"], (hd,), storage="float32"),
                 WeightSpec(nm["bonus"], (self.nh, self.D), storage="float32"),
                 WeightSpec(nm["norm"], (hd,), storage="float32", init="norm"), WeightSpec(nm["o"], (H, hd))])

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm = self.names
        self.mu = torch.stack([tensors.pop(nm[f"mu_{s}"]) for s in MIXES], dim=0).contiguous()
        self.w_r, self.w_k, self.w_v, self.w_g = (tensors.pop(nm[s]) for s in ("r", "k", "v", "g"))
        self.w_w1, self.w_w2, self.w_out = tensors.pop(nm["decay_in"]), tensors.pop(nm["decay_out"]), tensors.pop(nm["o"])
        self.w0, self.bonus, self.norm_w = tensors[nm["decay_bias"]], tensors[nm["bonus"]], tensors[nm["norm"]]

    def cache_spec(self):
        return StateSpec((self.state_matrix + self.H,), torch.float32)

    def forward(self, ctx, x: torch.Tensor, cache, sink=None):
        T, ws, hd = x.shape[0], ctx.ws, self.hd
        mixes = ws.alloc((len(MIXES), T, self.H), self.dtype)
        ops.token_shift(x, self.mu, cache.state, self.state_matrix, ctx, mixes)
        r, k, v, g = (ws.alloc((T, hd), torch.float32) for _ in range(4))
        for i, (out, w) in enumerate(((r, self.w_r), (k, self.w_k), (v, self.w_v), (g, self.w_g))):
            linear(ctx, mixes[i], w, out)
        low = ws.alloc((T, self.rank), torch.float32)
        linear(ctx, mixes[4], self.w_w1, low)
        decay = ws.alloc((T, hd), torch.float32)
        ops.lowrank_act(low, self.w_w2, self.w0, decay, ctx.req_of_token, ops.LOWRANK_EXP_NEG_EXP, in_tanh=True)
        o = ws.alloc((T, hd), torch.float32)
        ops.recurrent_state(ops.RECURRENCE_WKV, r, k, v, decay, cache.state, ctx, o, self.nh, 1, self.D, self.D,
                            bonus=self.bonus, tail_src=x, tail_off=self.state_matrix, tail_rows=1)
        act = ws.alloc((T, hd), self.dtype)
        ops.gla_out_gate(o, g, self.norm_w, self.eps, act, self.nh, self.D, ctx.req_of_token, gate_act=ops.GATE_SILU,
                         weight_per_head=True)
        delta = ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_out, delta)
        return delta


register_part("mixer", "time_mix", TimeMix)
