"""Configuration of the Pogarax decoder, read from its config.json keys.

A Pogarax model is a stack of layers whose norms sit on the sub-layers' OUTPUTS (x += m * rmsnorm(mixer(x)), then
x += m * rmsnorm(ffn(x)); the sub-layers read x itself), each with its own kind of mixer and feed-forward:

``architecture``        "Pogarax"
``vocab``, ``width``    vocabulary and residual width
``norm.eps``            eps of every root mean square
``residual_mult``       m, the factor on what a sub-layer adds to the residual stream
``layers``              one entry per layer: ``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp``
                        ({"kind": "dense", "ff"}, {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}},
                        or null for none)

Mixer keys.  "channel_delta" (gated delta rule with short convolutions): ``heads``, ``kv_heads``, ``dim``, ``vdim``,
``conv`` (taps).  "latent_attention": ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``q_rank``, ``kv_rank``, ``scale``,
``mask.size`` (sliding window; absent: none), ``rot`` {``dims``, ``base``, ``scaling`` {factor, original, fast, slow}} and
optionally ``kv_from``: the layer whose cached rows this layer attends over instead of caching its own.  "wkv" (time
mix): ``heads``, ``dim``.  The ranks of the low-rank pairs (the delta rule's decay and gate, the time mix's decay) are in
no key and are taken from the tensors ``l<i>.mix.{a1,g1,w1}``.

Tensor names: ``embed``, ``head``, ``final.norm`` and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.router`` with ``l<i>.mlp.e<j>.{gate,up,down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, LayerCall, LayerSpec, ModelConfig

MIXERS = ("channel_delta", "latent_attention", "wkv")
RANK_TENSORS = {"channel_delta": ("a1", "g1"), "wkv": ("w1",), "latent_attention": ()}


@dataclass(frozen=True)
class PogaraxConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    norm_eps: float
    residual_mult: float
    layers: Tuple[Dict[str, Any], ...]
    ranks: Tuple[Tuple[int, ...], ...] = ()      # per layer, the rows of its RANK_TENSORS; 0: not known (the default)
    architecture: str = "Pogarax"
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 1 << 20       # the cache alone bounds a request

    DEFAULT_RANK = 16

    # ---- reading ----
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PogaraxConfig":
        problems: List[str] = []

        def integer(where, key: str, what: str, default=None, least: int = 1) -> int:
            v = where.get(key, default) if isinstance(where, dict) else default
            if isinstance(v, bool) or not isinstance(v, int):
                problems.append(f"{what} must be an integer, found {v!r}")
                return least
            if v < least:
                problems.append(f"{what} must be at least {least}, found {v}")
                return least
            return v

        def number(where, key: str, what: str, default=None, positive: bool = False) -> float:
            v = where.get(key, default) if isinstance(where, dict) else default
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                problems.append(f"{what} must be a number, found {v!r}")
                return 1.0
            if positive and not v > 0:
                problems.append(f"{what} must be positive, found {v}")
                return 1.0
            return float(v)

        V = integer(d, "vocab", "vocab")
        H = integer(d, "width", "width")
        eps = number(d.get("norm") or {}, "eps", "norm.eps", positive=True)
        mult = number(d, "residual_mult", "residual_mult", 1.0)
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json cannot be used: 'layers' must be a non-empty list")
        layers: List[Dict[str, Any]] = []
        for i, l in enumerate(raw):
            w = f"layers[{i}]"
            if not isinstance(l, dict) or l.get("type") not in MIXERS or not isinstance(l.get("mixer"), dict):
                problems.append(f"{w} needs a 'type' out of {list(MIXERS)} and a 'mixer' object")
                layers.append(dict(type=None, mixer={}, mlp=None))
                continue
            m, kind = l["mixer"], l["type"]
            mixer: Dict[str, Any] = dict(heads=integer(m, "heads", f"{w}.mixer.heads"), dim=integer(m, "dim", f"{w}.mixer.dim"))
            if kind == "channel_delta":
                mixer["kv_heads"] = integer(m, "kv_heads", f"{w}.mixer.kv_heads", mixer["heads"])
                if mixer["heads"] % mixer["kv_heads"]:
                    problems.append(f"{w}.mixer.heads ({mixer['heads']}) must be a multiple of kv_heads ({mixer['kv_heads']})")
                mixer["vdim"] = integer(m, "vdim", f"{w}.mixer.vdim")
                mixer["conv"] = integer(m, "conv", f"{w}.mixer.conv")
            elif kind == "latent_attention":
                mixer["vdim"] = integer(m, "vdim", f"{w}.mixer.vdim")
                mixer["rot_dim"] = integer(m, "rot_dim", f"{w}.mixer.rot_dim", least=0)
                mixer["q_rank"] = integer(m, "q_rank", f"{w}.mixer.q_rank")
                mixer["kv_rank"] = integer(m, "kv_rank", f"{w}.mixer.kv_rank")
                mixer["scale"] = number(m, "scale", f"{w}.mixer.scale")
                if isinstance(m.get("mask"), dict):
                    mixer["mask"] = dict(size=integer(m["mask"], "size", f"{w}.mixer.mask.size"))
                rot = m.get("rot")
                if isinstance(rot, dict):
                    r: Dict[str, Any] = dict(dims=integer(rot, "dims", f"{w}.mixer.rot.dims", mixer["rot_dim"], least=0),
                                             base=number(rot, "base", f"{w}.mixer.rot.base", 10000.0, positive=True))
                    if r["dims"] % 2 or r["dims"] > mixer["rot_dim"]:
                        problems.append(f"{w}.mixer.rot.dims must be even and at most rot_dim, found {r['dims']}")
                    sc = rot.get("scaling")
                    if isinstance(sc, dict):
                        r["scaling"] = {k: number(sc, k, f"{w}.mixer.rot.scaling.{k}", positive=True)
                                        for k in ("factor", "original", "fast", "slow")}
                    mixer["rot"] = r
                elif mixer["rot_dim"] > 0:
                    problems.append(f"{w}.mixer.rot is missing although rot_dim is {mixer['rot_dim']}")
                if "kv_from" in m:
                    mixer["kv_from"] = integer(m, "kv_from", f"{w}.mixer.kv_from", least=0)
            mlp = l.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    problems.append(f"{w}.mlp must be null or an object of kind 'dense' or 'moe'")
                    mlp = None
                elif mlp["kind"] == "dense":
                    mlp = dict(kind="dense", ff=integer(mlp, "ff", f"{w}.mlp.ff"))
                else:
                    router = mlp.get("router") or {}
                    mlp = dict(kind="moe", expert=dict(ff=integer(mlp.get("expert") or {}, "ff", f"{w}.mlp.expert.ff")),
                               router=dict(experts=integer(router, "experts", f"{w}.mlp.router.experts"),
                                           top=integer(router, "top", f"{w}.mlp.router.top")))
                    if mlp["router"]["top"] > mlp["router"]["experts"]:
                        problems.append(f"{w}.mlp.router.top exceeds the number of experts")
            layers.append(dict(type=kind, mixer=mixer, mlp=mlp))
        for i, l in enumerate(layers):
            j = l["mixer"].get("kv_from")
            if j is None:
                continue
            src = layers[j] if j < i else None
            if src is None or src["type"] != "latent_attention" or "kv_from" in src["mixer"]:
                problems.append(f"layers[{i}].mixer.kv_from must name an earlier latent_attention layer with a cache of its own")
            elif any(src["mixer"].get(k) != l["mixer"].get(k) for k in ("kv_rank", "rot_dim", "rot")):
                problems.append(f"layers[{i}] reads the cache of layer {j}: their kv_rank, rot_dim and rot must be equal")
        if problems:
            raise ConfigError("config.json cannot be used: " + "; ".join(problems))
        return cls(vocab_size=V, hidden_size=H, norm_eps=eps, residual_mult=mult, layers=tuple(layers),
                   architecture=str(d.get("architecture", "Pogarax")))

    def to_dict(self) -> Dict[str, Any]:
        def copy(v):
            return {k: copy(x) for k, x in v.items()} if isinstance(v, dict) else v
        return {"architecture": self.architecture,
                "layers": [dict(type=l["type"], mixer=copy(l["mixer"]), mlp=copy(l["mlp"])) for l in self.layers],
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                "vocab": self.vocab_size, "width": self.hidden_size}

    # ---- sizes that only the weights give ----
    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "PogaraxConfig":
        """The configuration completed by the ranks of the low-rank pairs (rows of ``l<i>.mix.a1``, ``.g1``, ``.w1``)."""
        ranks = []
        for i, l in enumerate(self.layers):
            old = self.ranks[i] if i < len(self.ranks) else ()
            row = []
            for j, name in enumerate(RANK_TENSORS[l["type"]]):
                shape = shapes.get(f"l{i}.mix.{name}")
                row.append(int(shape[0]) if shape else (old[j] if j < len(old) else 0))
            ranks.append(tuple(row))
        return PogaraxConfig(**{**self.__dict__, "ranks": tuple(ranks)})

    def rank(self, layer: int, which: int) -> int:
        row = self.ranks[layer] if layer < len(self.ranks) else ()
        return (row[which] if which < len(row) else 0) or self.DEFAULT_RANK

    # ---- what the model is made of ----
    def tensor_names(self) -> Dict[str, str]:
        return dict(embed="embed", layer="l{i}", mixer="mix", ffn="mlp", norm1="norm1", norm2="norm2",
                    final_norm="final.norm", head="head")

    def final_norm(self) -> Tuple[str, dict]:
        return "rmsnorm", dict(size=self.hidden_size, eps=self.norm_eps, weight_name="")

    def cache_window(self, owner: int) -> int:
        """How long the rows layer ``owner`` caches must be kept: the longest window of the layers that attend over
        them (0: for ever, as soon as one of them has no window)."""
        sizes = [(l["mixer"].get("mask") or {}).get("size", 0) for i, l in enumerate(self.layers)
                 if l["type"] == "latent_attention" and (i == owner or l["mixer"].get("kv_from") == owner)]
        return 0 if any(s == 0 for s in sizes) else max(sizes)

    def layer_specs(self) -> List[LayerSpec]:
        H, specs = self.hidden_size, []
        for i, l in enumerate(self.layers):
            m = l["mixer"]
            if l["type"] == "channel_delta":
                mixer, args = "gated_delta_rule", dict(
                    hidden_size=H, num_heads=m["heads"], num_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
                    conv_taps=m["conv"], decay_rank=self.rank(i, 0), gate_rank=self.rank(i, 1), norm_eps=self.norm_eps)
            elif l["type"] == "latent_attention":
                rot = m.get("rot") or {}
                owner = m.get("kv_from", i)
                mixer, args = "latent_attention", dict(
                    hidden_size=H, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], value_dim=m["vdim"],
                    q_rank=m["q_rank"], kv_rank=m["kv_rank"], scale=m["scale"], norm_eps=self.norm_eps,
                    window=(m.get("mask") or {}).get("size", 0), cache_window=self.cache_window(owner), sink=True,
                    owns_cache="kv_from" not in m,
                    position="rotary_scaled_interleaved" if rot.get("dims", 0) > 0 else "none",
                    position_args=dict(rotary_dim=rot["dims"], theta=rot["base"], scaling=rot.get("scaling"))
                    if rot.get("dims", 0) > 0 else {})
            else:
                mixer, args = "time_mix", dict(hidden_size=H, num_heads=m["heads"], head_dim=m["dim"],
                                               decay_rank=self.rank(i, 0), norm_eps=self.norm_eps)
            mlp = l["mlp"]
            names = dict(gate="gate", up="up", down="down")
            if not mlp:
                ffn, fargs = "", {}
            elif mlp["kind"] == "dense":
                ffn, fargs = "swiglu", dict(hidden_size=H, intermediate_size=mlp["ff"], names=names)
            else:
                ffn, fargs = "routed_experts", dict(hidden_size=H, intermediate_size=mlp["expert"]["ff"],
                                                    num_experts=mlp["router"]["experts"], top=mlp["router"]["top"],
                                                    scores="sigmoid", renormalize=False, weight_on="input")
            specs.append(LayerSpec(mixer=mixer, mixer_args=args, feed_forward=ffn, ffn_args=fargs, norm="rmsnorm",
                                   norm_args=dict(size=H, eps=self.norm_eps, weight_name=""), arrangement="post_norm",
                                   arrangement_args=dict(residual_mult=self.residual_mult)))
        return specs

    def execution_order(self) -> List[LayerCall]:
        return [LayerCall(i, cache_from=l["mixer"].get("kv_from")) for i, l in enumerate(self.layers)]

    def summary(self) -> str:
        kinds = "".join({"channel_delta": "d", "latent_attention": "a", "wkv": "w"}[l["type"]] for l in self.layers)
        moe = sum(1 for l in self.layers if l["mlp"] and l["mlp"]["kind"] == "moe")
        return (f"{self.architecture}: {len(self.layers)} post-norm layers ({kinds}: d gated delta rule, a latent attention, "
                f"w time mix), {moe} with routed experts, width {self.hidden_size}, vocab {self.vocab_size}")
