"""Configuration of the Vedizen decoder, read from its config.json keys.

A Vedizen model is a stack of parallel layers (one Dynamic Tanh norm whose output both the mixer and the
feed-forward read; their sum is added to the residual stream), each with its own kind of mixer:

``architecture``        "Vedizen"
``vocab``, ``width``    vocabulary and residual width
``embedding.scale``     every embedded row is multiplied by it
``norm.eps``            eps of the root mean squares inside the mixers (the layer norm itself uses none)
``layers``              one entry per layer: ``type`` ("gla" or "attention"), ``mixer`` (its sizes and
                        constants) and ``mlp`` ({"kind": "dense", "ff", "limit"}, or null for none)
``loop``                {"start", "stop", "times"}: layers start .. stop-1 run ``times`` times in a row with
                        the same weights and a cache or state per pass; before the first layer of pass t the
                        row t of the tensor ``loop.step`` is added to the residual stream

Mixer keys.  "gla": ``heads``, ``dim`` (key channels a head), ``vdim`` (value channels a head), ``tau``; the rank
of the decay's low-rank pair is not in config.json and is taken from the tensor ``l<i>.mix.a1``.  "attention"
(differential, chunked): ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``softcap``, ``diff`` and ``mask.size``.

Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``, ``.alpha``), ``loop.step`` and per layer
``l<i>.norm1`` (+ ``.b``, ``.alpha``), ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, LayerCall, LayerSpec, ModelConfig

MIXERS = ("gla", "attention")


@dataclass(frozen=True)
class VedizenConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    decay_ranks: Tuple[int, ...] = ()        # per layer, for "gla" layers; 0: not known (the default rank)
    architecture: str = "Vedizen"
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 1 << 20   # no layer encodes positions; the cache alone bounds a request

    # ---- reading ----
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "VedizenConfig":
        problems: List[str] = []

        def integer(where: Dict[str, Any], key: str, what: str, default=None, least: int = 1) -> int:
            v = where.get(key, default) if isinstance(where, dict) else default
            if isinstance(v, bool) or not isinstance(v, int):
                problems.append(f"{what} must be an integer, found {v!r}")
                return least
            if v < least:
                problems.append(f"{what} must be at least {least}, found {v}")
                return least
            return v

        def number(where: Dict[str, Any], key: str, what: str, default=None, positive: bool = False) -> float:
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
        emb = d.get("embedding") or {}
        scale = number(emb, "scale", "embedding.scale", 1.0)
        eps = number(d.get("norm") or {}, "eps", "norm.eps", positive=True)
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json cannot be used: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw):
            w = f"layers[{i}]"
            if not isinstance(l, dict) or l.get("type") not in MIXERS or not isinstance(l.get("mixer"), dict):
                problems.append(f"{w} needs a 'type' out of {list(MIXERS)} and a 'mixer' object")
                continue
            m, kind = l["mixer"], l["type"]
            mixer: Dict[str, Any] = dict(heads=integer(m, "heads", f"{w}.mixer.heads"), dim=integer(m, "dim", f"{w}.mixer.dim"),
                                         vdim=integer(m, "vdim", f"{w}.mixer.vdim"))
            if kind == "gla":
                mixer["tau"] = number(m, "tau", f"{w}.mixer.tau", positive=True)
            else:
                mixer["kv_heads"] = integer(m, "kv_heads", f"{w}.mixer.kv_heads", mixer["heads"])
                if mixer["heads"] % mixer["kv_heads"]:
                    problems.append(f"{w}.mixer.heads ({mixer['heads']}) must be a multiple of kv_heads ({mixer['kv_heads']})")
                mixer["scale"] = number(m, "scale", f"{w}.mixer.scale", mixer["dim"] ** -0.5)
                mixer["softcap"] = number(m, "softcap", f"{w}.mixer.softcap", 0.0)
                mixer["diff"] = number(m, "diff", f"{w}.mixer.diff")
                mask = m.get("mask") or {}
                mixer["mask"] = dict(size=integer(mask, "size", f"{w}.mixer.mask.size", 0, least=0))
            mlp = l.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                    problems.append(f"{w}.mlp must be null or an object of kind 'dense'")
                    mlp = None
                else:
                    mlp = dict(kind="dense", ff=integer(mlp, "ff", f"{w}.mlp.ff"),
                               limit=number(mlp, "limit", f"{w}.mlp.limit", positive=True))
            layers.append(dict(type=kind, mixer=mixer, mlp=mlp))
        L = len(raw)
        loop = d.get("loop") or {}
        start = integer(loop, "start", "loop.start", 0, least=0)
        stop = integer(loop, "stop", "loop.stop", start, least=0)
        times = integer(loop, "times", "loop.times", 1, least=0)
        if not (0 <= start <= stop <= L):
            problems.append(f"loop must satisfy 0 <= start <= stop <= {L}, found start {start}, stop {stop}")
        if problems:
            raise ConfigError("config.json cannot be used: " + "; ".join(problems))
        return cls(vocab_size=V, hidden_size=H, embedding_scale=scale, norm_eps=eps, layers=tuple(layers),
                   loop_start=start, loop_stop=stop, loop_times=times,
                   architecture=str(d.get("architecture", "Vedizen")))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [dict(type=l["type"], mixer=dict(l["mixer"]), mlp=None if l["mlp"] is None else dict(l["mlp"]))
                       for l in self.layers],
            "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.hidden_size,
        }
        return d

    # ---- sizes that only the weights give ----
    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "VedizenConfig":
        """The configuration completed by what only the tensors' shapes say: the rank of every gated
        linear attention layer's decay pair (rows of ``l<i>.mix.a1``)."""
        ranks = []
        for i, l in enumerate(self.layers):
            shape = shapes.get(f"l{i}.mix.a1")
            ranks.append(int(shape[0]) if l["type"] == "gla" and shape else
                         (self.decay_ranks[i] if i < len(self.decay_ranks) else 0))
        return VedizenConfig(**{**self.__dict__, "decay_ranks": tuple(ranks)})

    DEFAULT_DECAY_RANK = 16

    def decay_rank(self, layer: int) -> int:
        r = self.decay_ranks[layer] if layer < len(self.decay_ranks) else 0
        return r or self.DEFAULT_DECAY_RANK

    # ---- what the model is made of ----
    def tensor_names(self) -> Dict[str, str]:
        return dict(embed="embed", layer="l{i}", mixer="mix", ffn="mlp", norm1="norm1", norm2="norm2",
                    final_norm="final.norm", head="head", order_table="loop.step")

    def embedding(self) -> Tuple[str, dict]:
        return "token_embedding", {"scale": self.embedding_scale}

    def final_norm(self) -> Tuple[str, dict]:
        return "dynamic_tanh", dict(size=self.hidden_size)

    def layer_specs(self) -> List[LayerSpec]:
        H, specs = self.hidden_size, []
        for i, l in enumerate(self.layers):
            m = l["mixer"]
            if l["type"] == "gla":
                mixer, args = "gated_linear_attention", dict(
                    hidden_size=H, num_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
                    decay_rank=self.decay_rank(i), tau=m["tau"], norm_eps=self.norm_eps)
            else:
                mixer, args = "differential_attention", dict(
                    hidden_size=H, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
                    scale=m["scale"], soft_cap=m["softcap"], lambda_init=m["diff"], norm_eps=self.norm_eps,
                    chunk=m["mask"]["size"], bias=True)
            mlp = l["mlp"]
            specs.append(LayerSpec(
                mixer=mixer, mixer_args=args,
                feed_forward="clamped_glu" if mlp else "",
                ffn_args=dict(hidden_size=H, intermediate_size=mlp["ff"], limit=mlp["limit"]) if mlp else {},
                norm="dynamic_tanh", norm_args=dict(size=H), arrangement="parallel"))
        return specs

    def execution_order(self) -> List[LayerCall]:
        """Layers before the loop once, the looped layers ``times`` times (each pass with caches of its own, its
        first entry adding row t of the pass table), then the rest."""
        L = len(self.layers)
        order = [LayerCall(i) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            for i in range(self.loop_start, self.loop_stop):
                order.append(LayerCall(i, add_row=t if i == self.loop_start else None))
        return order + [LayerCall(i) for i in range(self.loop_stop, L)]

    def order_table(self) -> Optional[Tuple[str, int]]:
        """(tensor name, rows) of the table whose rows ``LayerCall.add_row`` names; None when nothing is looped."""
        if self.loop_times <= 0 or self.loop_stop <= self.loop_start:
            return None
        return "loop.step", self.loop_times

    def ignorable_tensors(self) -> List[str]:
        """Tensors a model file may hold although nothing reads them: the pass table of a loop that runs no layer."""
        return [] if self.order_table() else ["loop.step"]

    def summary(self) -> str:
        kinds = "".join("g" if l["type"] == "gla" else "a" for l in self.layers)
        loop = (f", layers {self.loop_start}..{self.loop_stop - 1} x {self.loop_times}"
                if self.order_table() else "")
        return (f"{self.architecture}: {len(self.layers)} parallel layers ({kinds}: g gated linear attention, "
                f"a differential attention), width {self.hidden_size}, vocab {self.vocab_size}{loop}, "
                f"{len(self.execution_order())} layer runs a token")
