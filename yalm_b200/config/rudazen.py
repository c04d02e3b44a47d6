"""Typed configuration of the Rudazen decoder, read from its ``config.json``.

The design: a scaled token embedding; layers that norm AFTER the residual sum,
x <- n(a x + mixer(x)), x <- n(a x + ff(x)), whose sublayers read x itself; two kinds of mixer
in any order -- "attention" (queries and keys normed over the whole projection, neighbouring
pairs rotated on a part of each head, values that are the keys as projected, a sliding window
plus one pooled row per block of positions before it) and "parallel" (a gated sliding-window
attention with YaRN-scaled rotation and a factor per head beside a gated linear recurrence,
each branch normed over the width, half their sum); a SwiGLU feed-forward or none.  Every size
and constant is read from config.json:

    architecture          "Rudazen"
    vocab, width          vocabulary and residual width
    norm.eps              epsilon of every RMS norm
    embedding.scale       x = E[token] * scale
    postln_alpha          the factor a on x in both sums of a layer
    layers[i]             {type: "attention" | "parallel", mixer: {...}, mlp: null | {kind: "dense", ff}}
      attention mixer     {heads, kv_heads, dim, vdim, scale, mask: {size, pool}, rot: {base, dims}}
      parallel mixer      {left: {heads, kv_heads, dim, vdim, scale, mask: {size},
                                  rot: {base, dims, scaling: {factor, original, fast, slow}}},
                           right: {heads, dim, vdim}}

Checkpoint tensors: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``final.norm``, ``head``;
attention: ``l<i>.mix.{q,k,o}``, ``l<i>.mix.{q,k}.norm``; parallel: ``l<i>.mix.left.{q,k,v,g,o,temp}``,
``l<i>.mix.left.{q,k}.norm``, ``l<i>.mix.right.{q,f,v,o,f.b,lower,norm}``, ``l<i>.mix.{left,right}.out``;
feed-forward: ``l<i>.mlp.{gate,up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .llama import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

# Positions are a 32-bit count and the rotation has no largest one; the context used when the
# caller names none is this.
NO_POSITION_LIMIT = 1 << 30
DEFAULT_CONTEXT = 1 << 16

# Constants the design fixes.
BRANCH_SCALE = 0.5             # the parallel mixer is half the sum of its two normed branches


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks {where}{key}")
    return d[key]


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: Optional[Dict[str, float]]          # factor, original, fast, slow

    @staticmethod
    def from_dict(d: Optional[Dict[str, Any]], where: str, head: int) -> Optional["Rotation"]:
        if not d:
            return None
        sc = d.get("scaling")
        if sc:
            sc = {k: float(_need(sc, k, where + "scaling.")) for k in ("factor", "original", "fast", "slow")}
            if not (sc["factor"] > 0 and sc["original"] > 0 and sc["fast"] > 0 and sc["slow"] > 0):
                raise ConfigError(f"{where}scaling: factor, original, fast and slow must be positive")
        r = Rotation(base=float(_need(d, "base", where)), dims=int(_need(d, "dims", where)), scaling=sc or None)
        if r.dims % 2 or not 0 < r.dims <= head or not r.base > 1:
            raise ConfigError(f"{where}: dims={r.dims} must be even and at most the head's {head}; base > 1")
        return r

    def part(self, head: int, layout: str) -> PartSpec:
        return PartSpec("rope_partial", {"head_dim": head, "dims": self.dims, "base": self.base,
                                         "layout": layout, "scaling": self.scaling})


@dataclass(frozen=True)
class AttentionShape:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    pool: Optional[int]
    rot: Optional[Rotation]

    @staticmethod
    def from_dict(d: Dict[str, Any], where: str) -> "AttentionShape":
        mask = d.get("mask") or {}
        dim = int(_need(d, "dim", where))
        m = AttentionShape(
            heads=int(_need(d, "heads", where)), kv_heads=int(_need(d, "kv_heads", where)), dim=dim,
            vdim=int(_need(d, "vdim", where)), scale=float(_need(d, "scale", where)),
            window=None if not mask.get("size") else int(mask["size"]),
            pool=None if not mask.get("pool") else int(mask["pool"]),
            rot=Rotation.from_dict(d.get("rot"), where + "rot.", dim))
        if min(m.heads, m.kv_heads, m.dim, m.vdim) <= 0 or m.heads % m.kv_heads:
            raise ConfigError(f"{where}: heads={m.heads} must be a positive multiple of kv_heads={m.kv_heads}, "
                              f"and dim, vdim positive")
        if not m.scale > 0:
            raise ConfigError(f"{where}scale must be positive, got {m.scale}")
        if (m.window is not None and m.window <= 0) or (m.pool is not None and m.pool <= 0):
            raise ConfigError(f"{where}mask: size and pool must be positive")
        if m.pool and not m.window:
            raise ConfigError(f"{where}mask.pool needs mask.size")
        return m

    def position(self, layout: str) -> PartSpec:
        if self.rot is None:
            return PartSpec("rope_partial", {"head_dim": self.dim, "dims": 0, "base": 2.0, "layout": layout})
        return self.rot.part(self.dim, layout)


@dataclass(frozen=True)
class RecurrenceShape:
    heads: int
    dim: int
    vdim: int

    @staticmethod
    def from_dict(d: Dict[str, Any], where: str) -> "RecurrenceShape":
        r = RecurrenceShape(heads=int(_need(d, "heads", where)), dim=int(_need(d, "dim", where)),
                            vdim=int(_need(d, "vdim", where)))
        if min(r.heads, r.dim, r.vdim) <= 0:
            raise ConfigError(f"{where}: heads, dim and vdim must be positive")
        return r


@dataclass(frozen=True)
class RudazenLayer:
    kind: str                                    # "attention" or "parallel"
    attention: AttentionShape                    # the mixer, or the left branch of "parallel"
    recurrence: Optional[RecurrenceShape]        # the right branch of "parallel"
    ff: Optional[int]


@dataclass(frozen=True)
class RudazenConfig:
    vocab: int
    width: int
    eps: float
    alpha: float
    embedding_scale: float
    layers: List[RudazenLayer]
    raw: Dict[str, Any] = field(default_factory=dict, compare=False)

    architecture = "Rudazen"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RudazenConfig":
        layers = []
        for i, ld in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            kind = _need(ld, "type", where)
            mixer = _need(ld, "mixer", where)
            if kind == "attention":
                att = AttentionShape.from_dict(mixer, where + "mixer.")
                if att.vdim != att.dim:
                    raise ConfigError(f"{where}mixer: the values are the keys, so vdim={att.vdim} must equal dim={att.dim}")
                rec = None
            elif kind == "parallel":
                att = AttentionShape.from_dict(_need(mixer, "left", where + "mixer."), where + "mixer.left.")
                if att.pool:
                    raise ConfigError(f"{where}mixer.left: a pooled mask is not part of this branch")
                rec = RecurrenceShape.from_dict(_need(mixer, "right", where + "mixer."), where + "mixer.right.")
            else:
                raise ConfigError(f"{where}type={kind!r} is not supported ('attention' or 'parallel')")
            mlp = ld.get("mlp")
            if mlp and mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"{where}mlp.kind={mlp.get('kind')!r} is not supported (only 'dense')")
            layers.append(RudazenLayer(kind, att, rec, None if not mlp else int(_need(mlp, "ff", where + "mlp."))))
        if not layers:
            raise ConfigError("config.json lists no layers")
        cfg = cls(vocab=int(_need(d, "vocab", "")), width=int(_need(d, "width", "")),
                  eps=float(_need(_need(d, "norm", ""), "eps", "norm.")),
                  alpha=float(d.get("postln_alpha", 1.0)),
                  embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                  layers=layers, raw=copy.deepcopy(d))
        if cfg.vocab <= 0 or cfg.width <= 0 or not cfg.eps > 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        if any(l.ff is not None and l.ff <= 0 for l in layers):
            raise ConfigError("mlp.ff must be positive")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)

    def ignorable_tensor(self, name: str) -> bool:
        """The second norm of a layer without a feed-forward may be in a checkpoint; it is not read."""
        return any(layer.ff is None and name == f"l{i}.norm2" for i, layer in enumerate(self.layers))

    # ---- the architecture as a list of parts ----------------------------------
    def _attention(self, a: AttentionShape, prefix: str, layout: str, **options) -> PartSpec:
        D = self.width
        params = {"hidden_size": D, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
                  "value_dim": a.vdim, "scale": a.scale, "window": a.window, "pool": a.pool,
                  "qk_norm": {"eps": self.eps}, "exact_softmax": True, "position": a.position(layout),
                  **options}
        keys = ["q", "k", "o", "q.norm", "k.norm"]
        if not options.get("values_from_keys"):
            keys.append("v")
        if options.get("element_gate"):
            keys.append("g")
        if options.get("head_temp"):
            keys.append("temp")
        return PartSpec("gqa_attention", params, {k: f"{prefix}.{k}" for k in keys})

    def to_spec(self) -> ModelSpec:
        D = self.width
        post = lambda name: PartSpec("sum_rmsnorm", {"size": D, "eps": self.eps, "residual_scale": self.alpha},
                                     {"weight": name})
        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}"
            if layer.kind == "attention":
                mixer = self._attention(layer.attention, f"{p}.mix", "neighbours", values_from_keys=True)
            else:
                left = self._attention(layer.attention, "left", "halves", element_gate=True, head_temp=True)
                r = layer.recurrence
                right = PartSpec("gated_linear_recurrence",
                                 {"hidden_size": D, "num_heads": r.heads, "key_dim": r.dim,
                                  "value_dim": r.vdim, "eps": self.eps})
                # the branches' tensors go by "<branch>.<key>" under the mixer's prefix
                left = PartSpec(left.kind, left.params)
                tensors = {}
                for name, keys in (("left", ["q", "k", "v", "o", "g", "temp", "q.norm", "k.norm", "out"]),
                                   ("right", ["q", "f", "v", "o", "f.b", "lower", "norm", "out"])):
                    for k in keys:
                        tensors[f"{name}.{k}"] = f"{p}.mix.{name}.{k}"
                mixer = PartSpec("parallel_branches",
                                 {"hidden_size": D, "eps": self.eps, "scale": BRANCH_SCALE,
                                  "branches": [("left", left), ("right", right)]}, tensors)
            parts = {"mixer": mixer, "mixer_norm": post(f"{p}.norm1")}
            if layer.ff is not None:
                parts["feed_forward"] = PartSpec(
                    "swiglu", {"hidden_size": D, "intermediate_size": layer.ff},
                    {k: f"{p}.mlp.{k}" for k in ("gate", "up", "down")})
                parts["feed_forward_norm"] = post(f"{p}.norm2")
            layers.append(LayerSpec("postnorm", parts))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D,
            max_positions=NO_POSITION_LIMIT, default_context=DEFAULT_CONTEXT,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "size": D,
                                             "scale": self.embedding_scale}, {"weight": "embed"}),
            layers=layers, run_order=[RunEntry(i) for i in range(len(layers))],
            final_norm=PartSpec("rmsnorm", {"size": D, "eps": self.eps}, {"weight": "final.norm"}),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "size": D, "tied": False},
                          {"weight": "head"}),
        )
        spec.validate()
        return spec
