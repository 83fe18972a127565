"""Typed configuration of the Linonex decoder, read from config.json.

A Linonex model adds a learned vector per position to its embeddings and runs pre-norm layers that may differ one
from the next. A layer's mixer is either a matrix memory with exponential gates ("mlstm": a recurrent layer with a
float32 state) or two mixers side by side on the same input ("parallel": on the left attention without a rotation,
with a short convolution on q, k and v, capped scores and keys seen only within the token's chunk of positions; on the
right the gated delta rule with one decay per head), their outputs normed over the width and averaged. Its
feed-forward is gated and dense, or routed experts (softmax over all router outputs, a learned correction of the
choice, weights on the outputs, gated experts, and router outputs that stand for experts returning their input), or
absent. A run of layers may be gone through several times with the same weights, each pass with a cache and state of
its own, the embeddings joining the stream again before every pass but the first. Every size and constant comes from
config.json.
"""
from dataclasses import dataclass
from typing import Optional, Tuple

from .registry import ConfigError
from .specs import (AttentionSpec, ExpertSpec, GatedMLPSpec, HeadDeltaSpec, MatrixMemorySpec, ModelSpec, NormSpec,
                    PositionEmbeddingSpec, RoutedMLPSpec, ScheduleEntry, SideBySideSpec, StreamsBlockSpec)
from .temetar import _float, _int

MEMORY, PARALLEL = "mlstm", "parallel"


@dataclass(frozen=True)
class LinonexMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, where, m):
        return cls(_int(where, m, "heads"), _int(where, m, "dim"), _int(where, m, "vdim"), _float(where, m, "gate_cap"))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class LinonexAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int                  # taps of the convolution on q, k and v; 0: none
    chunk: Optional[int]       # positions of a chunk; None: every earlier key is seen
    softcap: Optional[float]   # None: scores as they are

    @classmethod
    def from_dict(cls, where, m):
        heads, kv_heads = _int(where, m, "heads"), _int(where, m, "kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}heads {heads} do not divide into kv_heads {kv_heads}")
        mask = m.get("mask")
        chunk = None if mask is None else _int(where + "mask.", mask, "size")
        softcap = None if m.get("softcap") is None else _float(where, m, "softcap")
        return cls(heads, kv_heads, _int(where, m, "dim"), _int(where, m, "vdim"), _float(where, m, "scale"),
                   _int(where, m, "conv", 0, 0), chunk, softcap)

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.conv:
            d["conv"] = self.conv
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        return d


@dataclass(frozen=True)
class LinonexDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, where, m):
        heads, kv_heads = _int(where, m, "heads"), _int(where, m, "kv_heads")
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}heads {heads} do not divide into kv_heads {kv_heads}")
        return cls(heads, kv_heads, _int(where, m, "dim"), _int(where, m, "vdim"), _int(where, m, "conv"))

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class LinonexParallel:
    left: LinonexAttention
    right: LinonexDelta

    @classmethod
    def from_dict(cls, where, m):
        if not isinstance(m, dict) or not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
            raise ConfigError(f"config.json: {where[:-1]} must have a left and a right mixer")
        return cls(LinonexAttention.from_dict(where + "left.", m["left"]), LinonexDelta.from_dict(where + "right.", m["right"]))

    def to_dict(self):
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class LinonexDense:
    ff: int

    def to_dict(self):
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class LinonexExperts:
    experts: int    # experts with tensors
    identity: int   # further router outputs: experts that return their input
    top: int
    scale: float
    ff: int

    @classmethod
    def from_dict(cls, where, m):
        router, expert = m.get("router"), m.get("expert")
        experts, top = _int(where + "router.", router, "experts"), _int(where + "router.", router, "top")
        identity = _int(where + "router.", router, "identity", 0, 0)
        if top > experts + identity:
            raise ConfigError(f"config.json: {where}router.top {top} is more than the {experts + identity} router outputs")
        return cls(experts, identity, top, _float(where + "router.", router, "scale", 1.0), _int(where + "expert.", expert, "ff"))

    def to_dict(self):
        return {"kind": "moe", "router": {"experts": self.experts, "identity": self.identity, "top": self.top,
                                          "scale": self.scale}, "expert": {"ff": self.ff}}


@dataclass(frozen=True)
class LinonexLayer:
    type: str       # "mlstm" or "parallel"
    mixer: object   # LinonexMemory or LinonexParallel
    mlp: object     # LinonexDense, LinonexExperts or None (no feed-forward)


@dataclass(frozen=True)
class LinonexLoop:
    start: int
    stop: int
    times: int

    def to_dict(self):
        return {"start": self.start, "stop": self.stop, "times": self.times}


@dataclass(frozen=True)
class LinonexConfig:
    vocab: int
    width: int
    layers: Tuple[LinonexLayer, ...]
    eps: float
    max_positions: int
    loop: Optional[LinonexLoop] = None
    architecture: str = "Linonex"

    @classmethod
    def from_dict(cls, raw):
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        parsed = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind == MEMORY:
                mixer = LinonexMemory.from_dict(where + "mixer.", layer.get("mixer"))
            elif kind == PARALLEL:
                mixer = LinonexParallel.from_dict(where + "mixer.", layer.get("mixer"))
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is neither {MEMORY} nor {PARALLEL}")
            mlp = layer.get("mlp")
            if mlp is not None:
                mlp_kind = mlp.get("kind", "dense") if isinstance(mlp, dict) else None
                if mlp_kind == "dense":
                    mlp = LinonexDense(_int(where + "mlp.", mlp, "ff"))
                elif mlp_kind == "moe":
                    mlp = LinonexExperts.from_dict(where + "mlp.", mlp)
                else:
                    raise ConfigError(f"config.json: {where}mlp.kind {mlp_kind!r} is neither dense nor moe")
            parsed.append(LinonexLayer(kind, mixer, mlp))
        loop = raw.get("loop")
        if loop is not None:
            start, times = _int("loop.", loop, "start", 0), _int("loop.", loop, "times")
            stop = _int("loop.", loop, "stop", 0)
            if not start <= stop <= len(parsed):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(parsed)} layers")
            loop = LinonexLoop(start, stop, times) if stop > start and times != 1 else None
        return cls(vocab=_int("", raw, "vocab"), width=_int("", raw, "width"), layers=tuple(parsed),
                   eps=_float("norm.", raw.get("norm"), "eps"), max_positions=_int("", raw, "max_positions"), loop=loop)

    def to_dict(self):
        """A config.json that from_dict reads back to this object."""
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "max_positions": self.max_positions,
             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                        for l in self.layers]}
        if self.loop is not None:
            d["loop"] = self.loop.to_dict()
        return d

    def run_order(self):
        """[(layer, whether the embeddings join the stream again right before it)] in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(l, False) for l in range(n)]
        a, b, times = self.loop.start, self.loop.stop, self.loop.times
        order = [(l, False) for l in range(a)]
        for k in range(times):
            order += [(l, l == a and k > 0) for l in range(a, b)]
        return order + [(l, False) for l in range(b, n)]

    def to_spec(self):
        norm = NormSpec(self.width, self.eps)
        blocks = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == MEMORY:
                mixer = MatrixMemorySpec(hidden=self.width, n_heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
                                         gate_cap=m.gate_cap, norm_eps=self.eps)
            else:
                a, r = m.left, m.right
                left = AttentionSpec(hidden=self.width, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim,
                                     scale=a.scale, qk_norm_eps=None, position=None, window=None, v_head_dim=a.vdim,
                                     exact_weights=True, conv_taps=a.conv, chunk=a.chunk, softcap=a.softcap)
                right = HeadDeltaSpec(hidden=self.width, n_heads=r.heads, n_kv_heads=r.kv_heads, key_dim=r.dim,
                                      value_dim=r.vdim, conv_taps=r.conv, norm_eps=self.eps)
                mixer = SideBySideSpec(hidden=self.width, left=left, right=right, norm_eps=self.eps, share=0.5)
            if layer.mlp is None:
                ffn = None
            elif isinstance(layer.mlp, LinonexDense):
                ffn = GatedMLPSpec(self.width, layer.mlp.ff, "silu")
            else:
                e = layer.mlp
                ffn = RoutedMLPSpec(hidden=self.width, experts=e.experts, top=e.top, expert=ExpertSpec(e.ff, "silu_gated"),
                                    shared=None, score="softmax_all", weight_on="output", correction=True,
                                    weight_scale=e.scale, identity=e.identity)
            blocks.append(StreamsBlockSpec(mixer_norm=norm, mixer=mixer, ffn_norm=norm if ffn else None, ffn=ffn,
                                           streams=1, branch_scale=1.0, learned=False))
        order = self.run_order()
        schedule = tuple(ScheduleEntry(l, None, again) for l, again in order)
        return ModelSpec(architecture=self.architecture, hidden=self.width, vocab=self.vocab, layers=tuple(blocks),
                         schedule=schedule, final_norm=norm, tied_head=False, max_positions=self.max_positions,
                         frame="positions",
                         frame_spec=PositionEmbeddingSpec(self.max_positions, keep=any(again for _, again in order)))
