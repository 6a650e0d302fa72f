"""Gated delta rule: a recurrent mixer whose state is a matrix per head that is corrected, not only added to.

With h the mixer's input, per head of D key channels and Dv value channels (q and k have ``num_kv_heads`` heads,
head i of the state reads q/k head i // (heads / kv_heads)):

    q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h))      a causal convolution over time per channel
    q <- q / |q| * D^-1/2,  k <- k / |k|                               per head, |x| = sqrt(sum x^2 + 1e-6)
    beta = sigmoid(Wb h)                                               one number per head
    g = exp(-exp(A_log[head]) * softplus(Wa2 (Wa1 h) + dt_bias))       a decay per head and key channel
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q  (token by token; S starts at zero)
    out = Wo concat_heads( o / rms(o) * w_norm * sigmoid(Wg2 (Wg1 h)) )

The state, the decays, beta, the unit vectors, the norm and the gate are float32.  The matrix state of a request
and the last ``taps - 1`` inputs of the convolution live side by side in its slot of the cache manager's state
tensor (one flat float32 row), so prompts cut anywhere, single tokens and whole prompts run the same recurrence.
The six input projections run as one product over [Wq; Wk; Wv; Wb; Wa1; Wg1].
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Mixer, StateSpec, register_part
from .linear import linear


class GatedDeltaRule(Mixer):
    device_driven = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 conv_taps: int, decay_rank: int, gate_rank: int, norm_eps: float, unit_eps: float = 1e-6,
                 q_scale: Optional[float] = None, dtype: torch.dtype = torch.bfloat16, device=None,
                 names: Optional[Dict[str, str]] = None):
        self.prefix, self.H = prefix, int(hidden_size)
        self.nh, self.nkv, self.D, self.Dv = int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
        self.taps, self.rank_a, self.rank_g = int(conv_taps), int(decay_rank), int(gate_rank)
        if min(self.nh, self.nkv, self.D, self.Dv, self.taps, self.rank_a, self.rank_g) <= 0:
            raise ValueError("heads, sizes, taps and ranks must be positive")
        if self.nh % self.nkv:
            raise ValueError(f"heads ({num_heads}) must be a multiple of kv_heads ({num_kv_heads})")
        if self.D > 256:
            raise ValueError(f"{self.D} key channels a head are above the recurrence kernel's limit of 256")
        self.eps, self.unit_eps = float(norm_eps), float(unit_eps)
        self.q_scale = float(q_scale) if q_scale is not None else self.D ** -0.5
        self.dtype, self.device = dtype, device
        n = dict(q="q", k="k", v="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", beta="b", a_log="A_log", norm="norm",
                 decay_in="a1", decay_out="a2", decay_bias="dt_bias", gate_in="g1", gate_out="g2", o="o")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.kd, self.vd = self.nkv * self.D, self.nh * self.Dv
        self.C = 2 * self.kd + self.vd                       # channels that pass the convolution
        self.state_matrix = self.nh * self.D * self.Dv       # the flat state: the matrices, then the convolution's tail
        self.w_in = self.w_out = self.conv_w = self.w_a2 = self.w_g2 = self.dt_bias = self.a_log = self.norm_w = None

    # ---- weights ----
    def weight_specs(self) -> List[WeightSpec]:
        nm, H = self.names, self.H
        return [WeightSpec(nm["q"], (self.kd, H)), WeightSpec(nm["k"], (self.kd, H)), WeightSpec(nm["v"], (self.vd, H)),
                WeightSpec(nm["q_conv"], (self.kd, self.taps), storage="float32"),
                WeightSpec(nm["k_conv"], (self.kd, self.taps), storage="float32"),
                WeightSpec(nm["v_conv"], (self.vd, self.taps), storage="float32"),
                WeightSpec(nm["beta"], (self.nh, H)), WeightSpec(nm["a_log"], (self.nh,), storage="float32"),
                WeightSpec(nm["norm"], (self.Dv,), storage="float32", init="norm"),
                WeightSpec(nm["decay_in"], (self.rank_a, H)), WeightSpec(nm["decay_out"], (self.nh * self.D, self.rank_a)),
                WeightSpec(nm["decay_bias"], (self.nh * self.D,), storage="float32"),
                WeightSpec(nm["gate_in"], (self.rank_g, H)), WeightSpec(nm["gate_out"], (self.vd, self.rank_g)),
                WeightSpec(nm["o"], (H, self.vd))]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm = self.names
        self.w_in = torch.cat([tensors.pop(nm[k]) for k in ("q", "k", "v", "beta", "decay_in", "gate_in")], dim=0).contiguous()
        self.conv_w = torch.cat([tensors.pop(nm[k]) for k in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.w_a2, self.w_g2, self.w_out = tensors.pop(nm["decay_out"]), tensors.pop(nm["gate_out"]), tensors.pop(nm["o"])
        self.dt_bias, self.a_log, self.norm_w = tensors[nm["decay_bias"]], tensors[nm["a_log"]], tensors[nm["norm"]]

    # ---- cache ----
    def cache_spec(self):
        return StateSpec((self.state_matrix + (self.taps - 1) * self.C,), torch.float32)

    # ---- compute ----
    def forward(self, ctx, h: torch.Tensor, cache, sink=None):
        T, ws, C, nh = h.shape[0], ctx.ws, self.C, self.nh
        proj = ws.alloc((T, C + nh + self.rank_a + self.rank_g), torch.float32)
        linear(ctx, h, self.w_in, proj)
        qkv, beta = proj[:, :C], proj[:, C:C + nh]
        low_a, low_g = proj[:, C + nh:C + nh + self.rank_a], proj[:, C + nh + self.rank_a:]
        conv = ws.alloc((T, C), torch.float32)
        ops.short_conv(qkv, self.conv_w, cache.state, self.state_matrix, ctx, conv, n_unit_heads=2 * self.nkv,
                       q_heads=self.nkv, unit_dim=self.D, unit_eps=self.unit_eps, q_scale=self.q_scale)
        decay = ws.alloc((T, nh * self.D), torch.float32)
        ops.lowrank_act(low_a, self.w_a2, self.dt_bias, decay, ctx.req_of_token, ops.LOWRANK_EXP_SOFTPLUS,
                        group_param=self.a_log, group=self.D)
        gate = ws.alloc((T, self.vd), torch.float32)
        ops.lowrank_act(low_g, self.w_g2, None, gate, ctx.req_of_token, ops.LOWRANK_SIGMOID)
        o = ws.alloc((T, self.vd), torch.float32)
        ops.recurrent_state(ops.RECURRENCE_DELTA, conv[:, :self.kd], conv[:, self.kd:2 * self.kd], conv[:, 2 * self.kd:], decay,
                            cache.state, ctx, o, nh, nh // self.nkv, self.D, self.Dv, beta=beta, tail_src=qkv,
                            tail_off=self.state_matrix, tail_rows=self.taps - 1)
        act = ws.alloc((T, self.vd), self.dtype)
        ops.gla_out_gate(o, gate, self.norm_w, self.eps, act, nh, self.Dv, ctx.req_of_token, gate_act=ops.GATE_AS_IS)
        delta = ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_out, delta)
        return delta


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
