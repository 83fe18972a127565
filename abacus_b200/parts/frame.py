"""The frame around the layers: how tokens become the residual stream and how the stream becomes logits.

"plain" is abacus's: x = float(embed[token]) with no scale (src/model.c:290-291); after the last layer
x += y, xn = norm(x) (src/model.c:311-312) and logits = xn . head^T on the wanted rows only
(src/model.c:322-325), the output matrix being the embedding table when the model ties them
(src/model.c:102-103). An architecture that scales its embeddings, caps its logits or norms elsewhere
registers another frame; the model's forward pass does not change.

A frame has
  param_shapes(tied) -> {slot: shape}     slots "embed", "final_norm", and "head" unless tied
  bind(params, ctx)
  embed(batch, ws, status) -> x           float32 [rows, hidden], the residual stream
  logits(x, y, batch, ws) -> float32 [batch.n_logit_rows, vocab]
  step_weights() -> tensors a step reads once whatever its size
"""
import torch

from ..kernels import ops
from .base import FRAMES, NORMS, to_device
from .linear import Linear


@FRAMES.register("plain")
class PlainFrame:
    capturable = True  # launches kernels only

    def __init__(self, spec):
        """spec: the ModelSpec (hidden, vocab, final_norm)."""
        self.hidden, self.vocab = spec.hidden, spec.vocab
        self.final_norm = NORMS.build(spec.final_norm)

    def param_shapes(self, tied):
        shapes = {"embed": (self.vocab, self.hidden), "final_norm": tuple(self.final_norm.param_shapes()["weight"])}
        if not tied:
            shapes["head"] = (self.vocab, self.hidden)
        return shapes

    def bind(self, params, ctx):
        self.ctx = ctx
        self.table = to_device(params["embed"], ctx, ctx.dtype)
        self.tied = "head" not in params
        self.head = Linear(self.table if self.tied else to_device(params["head"], ctx, ctx.dtype))
        self.final_norm.bind({"weight": params["final_norm"]}, ctx)

    def step_weights(self):
        # of the embedding table a step reads only the rows it looks up; the output matrix it reads whole
        return [self.head.weight, *self.final_norm.step_weights()]

    def embed(self, batch, ws, status):
        x = ws.get("x", (batch.n_rows, self.hidden), torch.float32)
        ops.embed(batch.tokens, self.table, x, status)
        return x

    def logits(self, x, y, batch, ws):
        r = batch.n_logit_rows
        out = ws.get("logits", (max(r, 1), self.vocab), torch.float32)[:r]
        if r:
            xn = ws.get("xn_final", (r, self.hidden), self.ctx.dtype)
            self.final_norm.forward(x, y, xn, rows=batch.logit_rows, n_rows=r)
            self.head.forward(xn, out, r)
        return out


@FRAMES.register("scaled_pairs")
class PairsFrame:
    """x = table[token] * scale, plus (with buckets > 0) a row of a second table chosen by the pair (previous token,
    token): row (previous * mul_prev + token * mul_cur) mod buckets, or row `buckets` for a sequence's first token. The
    previous token of a step's first row is part of the sequence's state (an int32 per slot, cache.frame). The stream
    starts as `streams` copies of x, [rows, streams, hidden] (parts/streams.py); at the end the copies are summed,
    normed and multiplied with the output matrix on the wanted rows. config.specs.PairEmbeddingSpec has the constants."""
    capturable = True  # launches kernels only

    def __init__(self, spec):
        self.hidden, self.vocab = spec.hidden, spec.vocab
        self.options = spec.frame_spec
        self.final_norm = NORMS.build(spec.final_norm)

    def param_shapes(self, tied):
        shapes = {"embed": (self.vocab, self.hidden), "final_norm": tuple(self.final_norm.param_shapes()["weight"])}
        if self.options.buckets > 0:
            shapes["pairs"] = (self.options.buckets + 1, self.hidden)
        if not tied:
            shapes["head"] = (self.vocab, self.hidden)
        return shapes

    def cache_need(self):
        from ..cache.need import CacheNeed
        return CacheNeed(states=(("last_token", (), "int32"),)) if self.options.buckets > 0 else None

    def bind(self, params, ctx):
        self.ctx = ctx
        self.table = to_device(params["embed"], ctx, ctx.dtype)
        self.pairs = to_device(params["pairs"], ctx, ctx.dtype) if "pairs" in params else None
        self.tied = "head" not in params
        self.head = Linear(self.table if self.tied else to_device(params["head"], ctx, ctx.dtype))
        self.final_norm.bind({"weight": params["final_norm"]}, ctx)
        self.ones = torch.ones(self.options.streams, dtype=torch.float32, device=ctx.device)

    def step_weights(self):
        return [self.head.weight, *self.final_norm.step_weights()]

    def embed(self, batch, ws, status, cache=None):
        o = self.options
        x = ws.get("x_streams", (batch.n_rows, o.streams, self.hidden), torch.float32)
        remembered = cache.states["last_token"] if self.pairs is not None else None
        ops.embed_pairs(batch, self.table, self.pairs, remembered, x, o.scale, o.buckets, o.mul_prev, o.mul_cur, status)
        if self.pairs is not None:
            ops.remember_tokens(batch, remembered)
        return x

    def logits(self, x, pending, batch, ws):
        from .streams import read_streams
        r = batch.n_logit_rows
        out = ws.get("logits", (max(r, 1), self.vocab), torch.float32)[:r]
        if r:
            xn = ws.get("xn_final", (r, self.hidden), self.ctx.dtype)
            read_streams(x, pending, self.ones, self.final_norm, xn, rows=batch.logit_rows, n_rows=r)
            self.head.forward(xn, out, r)
        return out


@FRAMES.register("positions")
class PositionsFrame:
    """x = table[token] + positions[position]: a learned vector per position, added unscaled (config.specs.
    PositionEmbeddingSpec). The stream is [rows, 1, hidden] (parts/streams.py). With `keep` the frame holds on to x as
    the embedding left it, and rejoin() adds it to the stream again where the schedule says so (a run of layers that
    is gone through more than once). The end is the plain frame's: the pending branch, the last norm, the output
    matrix on the wanted rows."""
    capturable = True  # launches kernels only

    def __init__(self, spec):
        self.hidden, self.vocab = spec.hidden, spec.vocab
        self.options = spec.frame_spec
        self.final_norm = NORMS.build(spec.final_norm)

    def param_shapes(self, tied):
        shapes = {"embed": (self.vocab, self.hidden), "positions": (self.options.max_positions, self.hidden),
                  "final_norm": tuple(self.final_norm.param_shapes()["weight"])}
        if not tied:
            shapes["head"] = (self.vocab, self.hidden)
        return shapes

    def bind(self, params, ctx):
        self.ctx = ctx
        self.table = to_device(params["embed"], ctx, ctx.dtype)
        self.positions = to_device(params["positions"], ctx, ctx.dtype)
        self.tied = "head" not in params
        self.head = Linear(self.table if self.tied else to_device(params["head"], ctx, ctx.dtype))
        self.final_norm.bind({"weight": params["final_norm"]}, ctx)
        self.ones = torch.ones(1, dtype=torch.float32, device=ctx.device)
        self.kept = None

    def step_weights(self):
        return [self.head.weight, *self.final_norm.step_weights()]

    def embed(self, batch, ws, status):
        x = ws.get("x_streams", (batch.n_rows, 1, self.hidden), torch.float32)
        self.kept = ws.get("x_embedded", (batch.n_rows, self.hidden), torch.float32) if self.options.keep else None
        ops.embed_positions(batch, self.table, self.positions, x, self.kept, status)
        return x

    def rejoin(self, x, batch):
        """x += what the embedding left, for every row of the step."""
        if self.kept is None:
            raise ValueError("the schedule joins the embedding again, but the frame does not keep it")
        ops.rejoin(x, self.kept, batch.n_rows)

    def logits(self, x, pending, batch, ws):
        from .streams import read_streams
        r = batch.n_logit_rows
        out = ws.get("logits", (max(r, 1), self.vocab), torch.float32)[:r]
        if r:
            xn = ws.get("xn_final", (r, self.hidden), self.ctx.dtype)
            read_streams(x, pending, self.ones, self.final_norm, xn, rows=batch.logit_rows, n_rows=r)
            self.head.forward(xn, out, r)
        return out


@FRAMES.register("loop_input")
class LoopInputFrame:
    """x = table[token], unscaled; the stream is [rows, 1, hidden] (parts/streams.py). Where the schedule goes through a
    run of layers in passes (config.specs.LoopInputSpec), the frame keeps the embedding x_0 and, right before the entry
    that starts pass t, makes the stream anew from itself and the embedding: x <- Win [x; x_0] + step[t] (the branch
    still pending is written first; the product's operands are of the model's type, its sums and the stream float32).
    The end is the plain frame's: the pending branch, the last norm, the output matrix on the wanted rows."""
    capturable = True  # launches kernels only

    def __init__(self, spec):
        self.hidden, self.vocab = spec.hidden, spec.vocab
        self.options = spec.frame_spec
        self.final_norm = NORMS.build(spec.final_norm)

    def param_shapes(self, tied):
        shapes = {"embed": (self.vocab, self.hidden), "final_norm": tuple(self.final_norm.param_shapes()["weight"])}
        if self.options.passes > 0:
            shapes.update(loop_in=(self.hidden, 2 * self.hidden), loop_step=(self.options.passes, self.hidden))
        if not tied:
            shapes["head"] = (self.vocab, self.hidden)
        return shapes

    def bind(self, params, ctx):
        self.ctx = ctx
        self.table = to_device(params["embed"], ctx, ctx.dtype)
        self.tied = "head" not in params
        self.head = Linear(self.table if self.tied else to_device(params["head"], ctx, ctx.dtype))
        self.final_norm.bind({"weight": params["final_norm"]}, ctx)
        self.ones = torch.ones(1, dtype=torch.float32, device=ctx.device)
        self.loop_in = self.loop_step = self.kept = None
        if self.options.passes > 0:
            self.loop_in = Linear(to_device(params["loop_in"], ctx, ctx.dtype))
            self.loop_step = to_device(params["loop_step"], ctx, torch.float32)

    def step_weights(self):
        return [self.head.weight, *self.final_norm.step_weights(), self.loop_in.weight if self.loop_in else None, self.loop_step]

    def embed(self, batch, ws, status):
        n = batch.n_rows
        x = ws.get("x_streams", (n, 1, self.hidden), torch.float32)
        ops.embed(batch.tokens, self.table, x.view(n, self.hidden), status)
        if self.loop_in is not None:
            self.kept = ws.get("x_embedded", (n, self.hidden), torch.float32)
            ops.embed(batch.tokens, self.table, self.kept, status)
        return x

    def inject(self, x, pending, batch, ws, t):
        """The stream made anew before pass t; returns what is pending afterwards (nothing)."""
        if self.loop_in is None or not 0 <= t < self.options.passes:
            raise ValueError(f"the schedule starts pass {t}, but the frame has {self.options.passes} passes")
        if pending is not None and (pending.mult != 1.0 or x.shape[1] != 1):
            raise ValueError("the stream is made anew from one stream whose branches are added as they are")
        n = batch.n_rows
        beside = ws.get("x_beside", (n, 2 * self.hidden), self.ctx.dtype)
        ops.stream_beside(x, pending.y if pending is not None else None, self.kept, beside, n)
        self.loop_in.forward(beside, x.view(x.shape[0], self.hidden), n)
        ops.add_vector(x, self.loop_step[t], n)
        return None

    def logits(self, x, pending, batch, ws):
        from .streams import read_streams
        r = batch.n_logit_rows
        out = ws.get("logits", (max(r, 1), self.vocab), torch.float32)[:r]
        if r:
            xn = ws.get("xn_final", (r, self.hidden), self.ctx.dtype)
            read_streams(x, pending, self.ones, self.final_norm, xn, rows=batch.logit_rows, n_rows=r)
            self.head.forward(xn, out, r)
        return out
