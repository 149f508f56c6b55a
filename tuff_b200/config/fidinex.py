"""`FidinexConfig`: the hyper-parameters of a Fidinex decoder.

config.json of this design is nested: top level `architecture` (a string), `vocab`, `width`, `norm.eps`,
`streams` (how many residual streams the layers keep; absent: one plain residual stream) and `layers`, one
object per layer: `type` (which mixer), `mixer` (its sizes and constants) and `mlp` (the feed-forward, or
null for none).

  type "attention"          mixer {heads, kv_heads, dim, vdim, scale, q_temp {coef, every}, v_mix}
  type "latent_attention"   mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}}
  mlp {"kind": "dense", "ff": F}

Every size and constant is read from there; nothing is fixed in code.  Whether the layers carry the small
weights of several streams is taken from the checkpoint's tensor names (`refine`): a model without them runs
the ordinary pre-norm layer.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Tuple

from .base import ConfigError, KeyReader
from .gimupel import _finite, _sub

ARCHITECTURE = "Fidinex"


@dataclass(frozen=True)
class QueryTemperature:
    coef: float
    every: int


@dataclass(frozen=True)
class SinkAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: QueryTemperature | None
    v_mix: bool


@dataclass(frozen=True)
class LatentAttentionMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class FidinexLayer:
    type: str
    mixer: object
    mlp: DenseMlp | None


@dataclass(frozen=True)
class FidinexConfig:
    vocab: int
    width: int
    norm_eps: float
    streams: int | None                       # None: one plain residual stream
    layers: Tuple[FidinexLayer, ...]
    stream_weights: bool = True               # the checkpoint has in/out/mix per sublayer (see `refine`)
    raw: dict = field(default_factory=dict, compare=False, repr=False)
    architectures: Tuple[str, ...] = (ARCHITECTURE,)
    ignored_keys: Tuple[str, ...] = field(default=(), compare=False)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hyper(self) -> bool:
        return self.streams is not None and self.stream_weights

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "FidinexConfig":
        r = KeyReader(raw, where)
        r.used.update(("architecture", "architectures"))
        V = r.integer("vocab", min_value=1)
        d = r.integer("width", min_value=1)
        eps = _sub(r, "norm").number("eps", positive=True)
        _finite(where, eps=eps)
        streams = r.optional_integer("streams", min_value=1)
        if streams is not None and streams > 8:
            raise ConfigError(f"{where}: key 'streams' = {streams}; at most 8 streams are supported")
        r.used.add("layers")
        if not isinstance(raw.get("layers"), list) or not raw["layers"]:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list of layer objects")
        layers = []
        for i, lraw in enumerate(raw["layers"]):
            lw = f"{where}: layers[{i}]"
            lr = KeyReader(lraw, lw)
            kind = lr.raw.get("type")
            lr.used.add("type")
            mr = _sub(lr, "mixer")
            if kind == "attention":
                mixer = _attention(mr)
            elif kind == "latent_attention":
                mixer = _latent(mr)
            else:
                raise ConfigError(f"{lw}: type = {kind!r}; known types: attention, latent_attention")
            layers.append(FidinexLayer(kind, mixer, _mlp(_sub(lr, "mlp", required=False))))
        shapes = {(l.mixer.kv_heads, l.mixer.vdim) for l in layers if isinstance(l.mixer, SinkAttention) and l.mixer.v_mix}
        if len(shapes) > 1:
            raise ConfigError(f"{where}: layers that mix values across layers must have the same kv_heads and vdim, found {sorted(shapes)}")
        return cls(vocab=V, width=d, norm_eps=eps, streams=streams, layers=tuple(layers), raw=dict(raw),
                   ignored_keys=tuple(r.unused()))

    def refine(self, shapes: dict) -> "FidinexConfig":
        """With the checkpoint's tensor names: whether the layers carry the streams' weights."""
        if self.streams is None:
            return self
        return replace(self, stream_weights="l0.hc1.in" in shapes)

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            m = l.mixer
            if isinstance(m, SinkAttention):
                mixer = dict(heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale, v_mix=m.v_mix)
                if m.q_temp is not None:
                    mixer["q_temp"] = dict(coef=m.q_temp.coef, every=m.q_temp.every)
            else:
                mixer = dict(heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale,
                             rot=dict(base=m.rot_base, dims=m.rot_dims))
            layers.append(dict(type=l.type, mixer=mixer, mlp=None if l.mlp is None else dict(kind="dense", ff=l.mlp.ff)))
        out = dict(architecture=ARCHITECTURE, vocab=self.vocab, width=self.width, norm=dict(eps=self.norm_eps), layers=layers)
        if self.streams is not None:
            out["streams"] = self.streams
        return out

    def describe(self) -> dict:
        return dict(vocab=self.vocab, width=self.width, norm_eps=self.norm_eps, streams=self.streams,
                    n_layers=len(self.layers), layer_types=[l.type for l in self.layers],
                    feed_forwards=["none" if l.mlp is None else f"dense {l.mlp.ff}" for l in self.layers])


def _attention(r: KeyReader) -> SinkAttention:
    H = r.integer("heads", min_value=1)
    G = r.integer("kv_heads", default=H, min_value=1)
    if H % G:
        raise ConfigError(f"{r.where}: heads {H} is not a multiple of kv_heads {G}")
    dim = r.integer("dim", min_value=2)
    if dim % 2:
        raise ConfigError(f"{r.where}: dim {dim} must be even")
    vdim = r.integer("vdim", default=dim, min_value=1)
    scale = r.number("scale", default=1.0 / math.sqrt(dim))
    qt = _sub(r, "q_temp", required=False)
    q_temp = None
    if qt is not None:
        q_temp = QueryTemperature(qt.number("coef"), qt.integer("every", min_value=1))
        _finite(qt.where, coef=q_temp.coef)
    _finite(r.where, scale=scale)
    return SinkAttention(H, G, dim, vdim, scale, q_temp, r.boolean("v_mix", default=False))


def _latent(r: KeyReader) -> LatentAttentionMixer:
    H = r.integer("heads", min_value=1)
    dim = r.integer("dim", min_value=1)
    rd = r.integer("rot_dim", min_value=0)
    vdim = r.integer("vdim", default=dim, min_value=1)
    rank = r.integer("kv_rank", min_value=1)
    scale = r.number("scale", default=1.0 / math.sqrt(dim + rd))
    rot = _sub(r, "rot", required=rd > 0)
    base = rot.number("base", positive=True) if rot is not None else 10000.0
    dims = rot.integer("dims", default=rd, min_value=0) if rot is not None else 0
    if rd % 2 or dims % 2 or dims > rd:
        raise ConfigError(f"{r.where}: rot_dim {rd} and rot.dims {dims} must be even, and rot.dims at most rot_dim")
    _finite(r.where, scale=scale, base=base)
    return LatentAttentionMixer(H, dim, rd, vdim, rank, scale, base, dims)


def _mlp(r: KeyReader | None):
    if r is None:
        return None
    kind = r.raw.get("kind")
    r.used.add("kind")
    if kind == "dense":
        return DenseMlp(r.integer("ff", min_value=1))
    raise ConfigError(f"{r.where}: kind = {kind!r}; known kinds: dense")
