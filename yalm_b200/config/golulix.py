"""Typed configuration of the Golulix decoder, read from its ``config.json``.

The design: a token embedding plus a hashed (previous token, token) table; pre-norm
layers whose norm weights are stored around zero; a mixer of gated, chunk-masked
grouped-query attention without position encoding; a feed-forward of routed experts
with a shared expert, or none; a span of layers that runs several times with the same
weights, the embedding output being added again before each repetition; a soft cap on
the logits.  Every size and constant is read from config.json:

    architecture          "Golulix"
    vocab, width          vocabulary and residual width
    norm.eps              epsilon of every RMS norm
    embedding.bigram      {buckets, mul_prev, mul_cur}: row (prev * mul_prev + tok * mul_cur)
                          mod buckets of the tensor ``bigram``; row ``buckets`` at position 0
    layers[i]             {type: "attention", mixer: {heads, kv_heads, dim, vdim, scale,
                          mask: {size}}, mlp: null | {kind: "moe", expert: {ff, limit},
                          router: {experts, top, groups: {count, keep}}, shared: {ff, limit}}}
    loop                  {start, stop, times}: layers start .. stop - 1 run ``times`` times
    logit_softcap         logits <- cap * tanh(logits / cap)

Checkpoint tensors: ``embed``, ``bigram``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.{q,k,v,g,o}``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{gate,up,down}``,
``l<i>.mlp.shared.{gate,up,down}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .llama import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

# The design has no position encoding, hence no largest position of its own.  A sequence's
# position is a 32-bit count; the context used when the caller names none is this.
NO_POSITION_LIMIT = 1 << 30
DEFAULT_CONTEXT = 1 << 16

# Constants the design fixes.
EXPERT_GATE_SLOPE = 1.702      # y = g * sigmoid(1.702 g) * (u + 1)
EXPERT_UP_SHIFT = 1.0


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks {where}{key}")
    return d[key]


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int                       # per-head query/key size
    vdim: int                      # per-head value size
    scale: float
    mask_size: Optional[int]       # a query sees the keys of its own chunk of this many positions

    @staticmethod
    def from_dict(d: Dict[str, Any], where: str) -> "AttentionMixer":
        mask = d.get("mask")
        m = AttentionMixer(
            heads=int(_need(d, "heads", where)), kv_heads=int(_need(d, "kv_heads", where)),
            dim=int(_need(d, "dim", where)), vdim=int(_need(d, "vdim", where)),
            scale=float(_need(d, "scale", where)),
            mask_size=None if not mask else int(_need(mask, "size", where + "mask.")))
        if min(m.heads, m.kv_heads, m.dim, m.vdim) <= 0 or m.heads % m.kv_heads:
            raise ConfigError(f"{where}: heads={m.heads} must be a positive multiple of kv_heads={m.kv_heads}, "
                              f"and dim, vdim positive")
        if not m.scale > 0:
            raise ConfigError(f"{where}scale must be positive, got {m.scale}")
        if m.mask_size is not None and m.mask_size <= 0:
            raise ConfigError(f"{where}mask.size must be positive, got {m.mask_size}")
        return m


@dataclass(frozen=True)
class ExpertShape:
    ff: int
    limit: float

    @staticmethod
    def from_dict(d: Dict[str, Any], where: str) -> "ExpertShape":
        e = ExpertShape(ff=int(_need(d, "ff", where)), limit=float(_need(d, "limit", where)))
        if e.ff <= 0 or not e.limit > 0:
            raise ConfigError(f"{where}: ff and limit must be positive")
        return e


@dataclass(frozen=True)
class RoutedMlp:
    expert: ExpertShape
    experts: int
    top: int
    group_count: int
    group_keep: int
    shared: Optional[ExpertShape]

    @staticmethod
    def from_dict(d: Dict[str, Any], where: str) -> "RoutedMlp":
        kind = d.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"{where}kind={kind!r} is not supported (only 'moe')")
        r = _need(d, "router", where)
        groups = r.get("groups") or {"count": 1, "keep": 1}
        m = RoutedMlp(expert=ExpertShape.from_dict(_need(d, "expert", where), where + "expert."),
                      experts=int(_need(r, "experts", where + "router.")),
                      top=int(_need(r, "top", where + "router.")),
                      group_count=int(_need(groups, "count", where + "router.groups.")),
                      group_keep=int(_need(groups, "keep", where + "router.groups.")),
                      shared=None if not d.get("shared") else
                      ExpertShape.from_dict(d["shared"], where + "shared."))
        if m.experts <= 0 or m.group_count <= 0 or m.experts % m.group_count:
            raise ConfigError(f"{where}router: {m.experts} experts do not form {m.group_count} equal groups")
        if not 0 < m.group_keep <= m.group_count:
            raise ConfigError(f"{where}router.groups.keep={m.group_keep} of {m.group_count} groups")
        if not 0 < m.top <= m.group_keep * (m.experts // m.group_count):
            raise ConfigError(f"{where}router.top={m.top} exceeds the experts of the kept groups")
        return m


@dataclass(frozen=True)
class GolulixLayer:
    mixer: AttentionMixer
    mlp: Optional[RoutedMlp]


@dataclass(frozen=True)
class GolulixConfig:
    vocab: int
    width: int
    eps: float
    layers: List[GolulixLayer]
    bigram: Optional[Dict[str, int]]             # buckets, mul_prev, mul_cur
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    logit_softcap: Optional[float] = None
    raw: Dict[str, Any] = field(default_factory=dict, compare=False)

    architecture = "Golulix"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GolulixConfig":
        layers = []
        for i, ld in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            kind = _need(ld, "type", where)
            if kind != "attention":
                raise ConfigError(f"{where}type={kind!r} is not supported (only 'attention')")
            layers.append(GolulixLayer(
                mixer=AttentionMixer.from_dict(_need(ld, "mixer", where), where + "mixer."),
                mlp=None if not ld.get("mlp") else RoutedMlp.from_dict(ld["mlp"], where + "mlp.")))
        if not layers:
            raise ConfigError("config.json lists no layers")
        bg = (d.get("embedding") or {}).get("bigram")
        bigram = None
        if bg:
            bigram = {k: int(_need(bg, k, "embedding.bigram.")) for k in ("buckets", "mul_prev", "mul_cur")}
            if bigram["buckets"] <= 0:
                raise ConfigError("embedding.bigram.buckets must be positive")
        loop = d.get("loop") or {}
        start, stop = int(loop.get("start", 0)), int(loop.get("stop", 0))
        times = int(loop.get("times", 1))
        if loop and not (0 <= start <= stop <= len(layers) and times >= 1):
            raise ConfigError(f"loop {loop} does not fit {len(layers)} layers")
        cap = d.get("logit_softcap")
        cfg = cls(vocab=int(_need(d, "vocab", "")), width=int(_need(d, "width", "")),
                  eps=float(_need(_need(d, "norm", ""), "eps", "norm.")), layers=layers, bigram=bigram,
                  loop_start=start, loop_stop=stop, loop_times=times,
                  logit_softcap=None if not cap else float(cap), raw=copy.deepcopy(d))
        if cfg.vocab <= 0 or cfg.width <= 0 or not cfg.eps > 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return copy.deepcopy(self.raw)

    def ignorable_tensor(self, name: str) -> bool:
        """The second norm of a layer without a feed-forward may be in a checkpoint; it is not read."""
        return any(layer.mlp is None and name == f"l{i}.norm2" for i, layer in enumerate(self.layers))

    # ---- the order of layer runs ----------------------------------------------
    def run_order(self) -> List[RunEntry]:
        L = len(self.layers)
        a, b, n = self.loop_start, self.loop_stop, self.loop_times
        if n <= 1 or b <= a:
            return [RunEntry(i) for i in range(L)]
        order = [RunEntry(i) for i in range(a)]
        for rep in range(n):
            order += [RunEntry(i, adds_embedding=(rep > 0 and i == a)) for i in range(a, b)]
        return order + [RunEntry(i) for i in range(b, L)]

    # ---- the architecture as a list of parts ----------------------------------
    def to_spec(self) -> ModelSpec:
        D = self.width
        norm = lambda name: PartSpec("rmsnorm", {"size": D, "eps": self.eps, "unit_offset": True},
                                     {"weight": name})
        layers = []
        for i, layer in enumerate(self.layers):
            m, p = layer.mixer, f"l{i}"
            parts = {
                "mixer_norm": norm(f"{p}.norm1"),
                "mixer": PartSpec("gqa_attention", {
                    "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads,
                    "head_dim": m.dim, "value_dim": m.vdim, "scale": m.scale, "window": None,
                    "chunk": m.mask_size, "head_gate": True,
                    "position": PartSpec("none", {"head_dim": m.dim}),
                }, {k: f"{p}.mix.{k}" for k in ("q", "k", "v", "o", "g")}),
            }
            if layer.mlp is not None:
                f = layer.mlp
                act = {"slope": EXPERT_GATE_SLOPE, "shift": EXPERT_UP_SHIFT}
                tensors = {"router": f"{p}.mlp.router"}
                for j in range(f.experts):
                    for k in ("gate", "up", "down"):
                        tensors[f"{k}.{j}"] = f"{p}.mlp.e{j}.{k}"
                params = {"hidden_size": D, "intermediate_size": f.expert.ff, "limit": f.expert.limit,
                          "experts": f.experts, "top": f.top, "groups": f.group_count,
                          "keep_groups": f.group_keep, "renormalise": False, **act, "shared": None}
                if f.shared is not None:
                    params["shared"] = {"intermediate_size": f.shared.ff, "limit": f.shared.limit, **act}
                    for k in ("gate", "up", "down"):
                        tensors[f"shared.{k}"] = f"{p}.mlp.shared.{k}"
                parts["feed_forward_norm"] = norm(f"{p}.norm2")
                parts["feed_forward"] = PartSpec("routed_experts", params, tensors)
            layers.append(LayerSpec("prenorm", parts))
        if self.bigram:
            embedding = PartSpec("hashed_pair_embedding",
                                 {"vocab_size": self.vocab, "size": D, **self.bigram},
                                 {"weight": "embed", "pair": "bigram"})
        else:
            embedding = PartSpec("embedding", {"vocab_size": self.vocab, "size": D}, {"weight": "embed"})
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D,
            max_positions=NO_POSITION_LIMIT, default_context=DEFAULT_CONTEXT,
            embedding=embedding, layers=layers, run_order=self.run_order(),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "size": D, "tied": False,
                                          "softcap": self.logit_softcap}, {"weight": "head"}),
        )
        spec.validate()
        return spec
