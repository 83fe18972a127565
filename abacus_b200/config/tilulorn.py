"""Typed configuration of the Tilulorn decoder, read from config.json.

A Tilulorn model runs pre-norm layers that may differ one from the next. A layer's mixer is latent attention (queries
through a latent of their own, keys and values kept as one low-rank latent row per token with one rotated key part
beside it, half-pair rotation with blended frequencies, a gate per head), or windowed attention (grouped heads whose
values are their keys as projected, q and k normed over their whole rows, interleaved rotation with slowed
frequencies, a sink in the softmax, a gate per head), or "wkv" time mixing (a recurrent layer with a float32 state, a
decay per key channel and token, and the token before as part of the state). Its feed-forward is a set of gated
experts that a table picks by token id, or absent. A run of layers may be gone through several times with the same
weights, each pass with a cache and state of its own, the stream being made anew from itself and the embedding before
every pass. Every size and constant comes from config.json (the inner size of a wkv layer's decay from its tensor).
"""
from dataclasses import dataclass, replace
from typing import Optional, Tuple

from .registry import ConfigError
from .specs import (AttentionSpec, ExpertSpec, LatentAttentionSpec, LoopInputSpec, ModelSpec, NormSpec, RotarySpec,
                    RoutedMLPSpec, ScheduleEntry, StreamsBlockSpec, WkvSpec)
from .temetar import MAX_POSITIONS, _float, _int

LATENT, WINDOWED, WKV = "latent_attention", "attention", "wkv"


@dataclass(frozen=True)
class TilulornRotation:
    base: float
    dims: int
    factor: Optional[float]    # None: frequencies as they are
    original: Optional[int]    # with fast and slow: the frequencies are blended; None: all divided by the factor
    fast: Optional[float]
    slow: Optional[float]

    @classmethod
    def from_dict(cls, where, r, most):
        base, dims = _float(where, r, "base"), _int(where, r, "dims", 2)
        if dims % 2 or dims > most:
            raise ConfigError(f"config.json: {where}dims {dims} must be even and at most {most}")
        scaling = r.get("scaling")
        if scaling is None:
            return cls(base, dims, None, None, None, None)
        w = where + "scaling."
        factor = _float(w, scaling, "factor")
        if "original" not in scaling:
            return cls(base, dims, factor, None, None, None)
        return cls(base, dims, factor, _int(w, scaling, "original"), _float(w, scaling, "fast"), _float(w, scaling, "slow"))

    def to_dict(self):
        d = {"base": self.base, "dims": self.dims}
        if self.factor is not None:
            d["scaling"] = {"factor": self.factor}
            if self.original is not None:
                d["scaling"].update(original=self.original, fast=self.fast, slow=self.slow)
        return d

    def to_spec(self, pairing):
        blend = None if self.original is None else (self.factor, self.original, self.fast, self.slow)
        linear = self.factor if self.factor is not None and self.original is None else 1.0
        return RotarySpec(theta=self.base, rotary_dim=self.dims, pairing=pairing, exact_angles=True, linear_factor=linear,
                          blend=blend)


@dataclass(frozen=True)
class TilulornLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: Optional[TilulornRotation]

    @classmethod
    def from_dict(cls, where, m):
        rot_dim = _int(where, m, "rot_dim", 0)
        rot = m.get("rot")
        if rot is not None:
            if not rot_dim:
                raise ConfigError(f"config.json: {where}rot goes with a rot_dim")
            rot = TilulornRotation.from_dict(where + "rot.", rot, rot_dim)
        return cls(_int(where, m, "heads"), _int(where, m, "dim"), rot_dim, _int(where, m, "vdim"), _int(where, m, "kv_rank"),
                   _int(where, m, "q_rank"), _float(where, m, "scale"), rot)

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "q_rank": self.q_rank, "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class TilulornWindowed:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    window: Optional[int]      # None: every earlier key
    rot: Optional[TilulornRotation]

    @classmethod
    def from_dict(cls, where, m):
        heads, kv = _int(where, m, "heads"), _int(where, m, "kv_heads")
        if heads % kv:
            raise ConfigError(f"config.json: {where}heads {heads} is no multiple of kv_heads {kv}")
        dim = _int(where, m, "dim")
        if m.get("vdim", dim) != dim:
            raise ConfigError(f"config.json: {where}vdim {m.get('vdim')} is not dim {dim}: a value is its key as projected")
        mask, rot = m.get("mask"), m.get("rot")
        window = None if mask is None else _int(where + "mask.", mask, "size")
        rot = None if rot is None else TilulornRotation.from_dict(where + "rot.", rot, dim)
        return cls(heads, kv, dim, _float(where, m, "scale"), window, rot)

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.dim, "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class TilulornWkv:
    heads: int
    dim: int
    decay_rank: int = 0        # the inner size of the decay's two matrices; 0: not yet read from the tensors' shapes

    @classmethod
    def from_dict(cls, where, m):
        return cls(_int(where, m, "heads"), _int(where, m, "dim"), _int(where, m, "decay_rank", 0, 0))

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim}


@dataclass(frozen=True)
class TilulornExperts:
    experts: int
    top: int
    ff: int

    @classmethod
    def from_dict(cls, where, m):
        router, expert = m.get("router"), m.get("expert")
        experts, top = _int(where + "router.", router, "experts"), _int(where + "router.", router, "top")
        if top > experts:
            raise ConfigError(f"config.json: {where}router.top {top} is more than the {experts} experts")
        return cls(experts, top, _int(where + "expert.", expert, "ff"))

    def to_dict(self):
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}


@dataclass(frozen=True)
class TilulornLayer:
    type: str
    mixer: object   # TilulornLatent, TilulornWindowed or TilulornWkv
    mlp: object     # TilulornExperts or None (no feed-forward)


@dataclass(frozen=True)
class TilulornLoop:
    start: int
    stop: int
    times: int

    def to_dict(self):
        return {"start": self.start, "stop": self.stop, "times": self.times}


_MIXERS = {LATENT: TilulornLatent, WINDOWED: TilulornWindowed, WKV: TilulornWkv}


@dataclass(frozen=True)
class TilulornConfig:
    vocab: int
    width: int
    layers: Tuple[TilulornLayer, ...]
    eps: float
    loop: Optional[TilulornLoop] = None
    architecture: str = "Tilulorn"

    @classmethod
    def from_dict(cls, raw):
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        parsed = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is none of {', '.join(_MIXERS)}")
            if not isinstance(layer.get("mixer"), dict):
                raise ConfigError(f"config.json: {where}mixer must give the mixer's sizes")
            mixer = _MIXERS[kind].from_dict(where + "mixer.", layer["mixer"])
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {where}mlp.kind must be moe (experts picked by a table), or mlp null")
                mlp = TilulornExperts.from_dict(where + "mlp.", mlp)
            parsed.append(TilulornLayer(kind, mixer, mlp))
        loop = raw.get("loop")
        if loop is not None:
            start, stop, times = _int("loop.", loop, "start", 0), _int("loop.", loop, "stop", 0), _int("loop.", loop, "times")
            if not start < stop <= len(parsed):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(parsed)} layers")
            loop = TilulornLoop(start, stop, times)
        return cls(vocab=_int("", raw, "vocab"), width=_int("", raw, "width"), layers=tuple(parsed),
                   eps=_float("norm.", raw.get("norm"), "eps"), loop=loop)

    def to_dict(self):
        """A config.json that from_dict reads back to this object (but for what the tensors' shapes give)."""
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                        for l in self.layers]}
        if self.loop is not None:
            d["loop"] = self.loop.to_dict()
        return d

    def with_ranks(self, shapes):
        """The inner size of every wkv layer's decay, from the shape of its first matrix ({tensor name: shape})."""
        layers = []
        for i, layer in enumerate(self.layers):
            if layer.type == WKV and not layer.mixer.decay_rank:
                name = f"l{i}.mix.w1"
                if name not in shapes or len(shapes[name]) != 2:
                    raise ConfigError(f"the model has no matrix {name} to read the decay's inner size from")
                layer = replace(layer, mixer=replace(layer.mixer, decay_rank=int(shapes[name][0])))
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    def run_order(self):
        """[(layer, the number of the pass that starts right before it, or None)] in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(l, None) for l in range(n)]
        a, b, times = self.loop.start, self.loop.stop, self.loop.times
        order = [(l, None) for l in range(a)]
        for t in range(times):
            order += [(l, t if l == a else None) for l in range(a, b)]
        return order + [(l, None) for l in range(b, n)]

    def to_spec(self):
        norm = NormSpec(self.width, self.eps)
        blocks = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == LATENT:
                mixer = LatentAttentionSpec(hidden=self.width, n_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim,
                                            v_head_dim=m.vdim, rank=m.kv_rank, scale=m.scale, norm_eps=self.eps,
                                            position=None if m.rot is None else m.rot.to_spec("half"), sink=False,
                                            q_rank=m.q_rank, head_gate=True)
            elif layer.type == WINDOWED:
                mixer = AttentionSpec(hidden=self.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                                      scale=m.scale, qk_norm_eps=self.eps,
                                      position=None if m.rot is None else m.rot.to_spec("interleaved"), window=m.window,
                                      sink=True, exact_weights=True, norm_over="projection", values="keys", head_gate=True)
            else:
                if not m.decay_rank:
                    raise ConfigError("a wkv layer's decay has an inner size that the tensors' shapes give (with_ranks)")
                mixer = WkvSpec(hidden=self.width, n_heads=m.heads, key_dim=m.dim, decay_rank=m.decay_rank, norm_eps=self.eps)
            ffn = None
            if layer.mlp is not None:
                e = layer.mlp
                ffn = RoutedMLPSpec(hidden=self.width, experts=e.experts, top=e.top, expert=ExpertSpec(e.ff, "silu_gated"),
                                    shared=None, score="table", weight_on="output", vocab=self.vocab)
            blocks.append(StreamsBlockSpec(mixer_norm=norm, mixer=mixer, ffn_norm=norm if ffn else None, ffn=ffn,
                                           streams=1, branch_scale=1.0, learned=False))
        schedule = tuple(ScheduleEntry(l, None, False, t) for l, t in self.run_order())
        return ModelSpec(architecture=self.architecture, hidden=self.width, vocab=self.vocab, layers=tuple(blocks),
                         schedule=schedule, final_norm=norm, tied_head=False, max_positions=MAX_POSITIONS,
                         frame="loop_input", frame_spec=LoopInputSpec(self.loop.times if self.loop is not None else 0))
