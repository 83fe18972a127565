"""A recurrent mixer: the gated delta rule with a decay per head and key channel (config.specs.DeltaRuleSpec).

Per head a float32 state S [key, value], zero at a sequence's start and carried from token to token:
    S <- diag(g) S;   e = b (v - S^T k);   S <- S + k e^T;   o = S^T q
The mixer owns everything around it: one stacked product for q, k, v, the write strength b and the inner vectors of
the decay and of the output gate; the short causal convolution and SiLU on q, k and v; the product that widens the two
inner vectors (their matrices on the diagonal of one); the per-head norm of o with its gate; the output product. Its cache is a state per sequence
and entry: S, and the last inputs of the convolution. It keeps no keys, so its cost per token does not grow.

Everything that enters the recurrence is float32 (unit vectors, decays, b, the state); q, k, v and the inner vectors
leave their products in the model's storage type.
"""
import torch

from ..cache.need import CacheNeed
from ..kernels import ops
from .base import MIXERS, to_device
from .linear import Linear


def _up8(n):
    return -(-n // 8) * 8


@MIXERS.register("channel_delta")
class ChannelDelta:
    capturable = True  # its forward launches kernels only; nothing in it depends on the step's contents

    def __init__(self, spec):
        s = self.spec = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} heads do not divide into {s.n_kv_heads} key heads")
        if not 1 <= s.key_dim <= 256:
            raise ValueError(f"key_dim {s.key_dim}: the recurrence keeps up to 256 key channels a head")
        if not 1 <= s.conv_taps <= 8:
            raise ValueError(f"conv_taps {s.conv_taps}: the convolution takes 1 to 8 taps")
        self.qk_size, self.v_size = s.n_kv_heads * s.key_dim, s.n_heads * s.value_dim
        self.channels = 2 * self.qk_size + self.v_size  # what passes the convolution: q, k, v as they lie in a row
        # columns of the stacked product: q, k, v, then b, the decay's inner vector, the gate's; each of the last three
        # starts at a multiple of 8 elements, so that every part of a row is 16-byte aligned
        self.at_b = _up8(self.channels)
        self.at_decay = self.at_b + _up8(s.n_heads)
        self.at_gate = self.at_decay + _up8(s.decay_rank)
        self.width = self.at_gate + _up8(s.gate_rank)

    def param_shapes(self):
        s = self.spec
        return {"wq": (self.qk_size, s.hidden), "wk": (self.qk_size, s.hidden), "wv": (self.v_size, s.hidden),
                "conv_q": (self.qk_size, s.conv_taps), "conv_k": (self.qk_size, s.conv_taps),
                "conv_v": (self.v_size, s.conv_taps), "wb": (s.n_heads, s.hidden),
                "decay_in": (s.decay_rank, s.hidden), "decay_out": (s.n_heads * s.key_dim, s.decay_rank),
                "decay_log": (s.n_heads,), "decay_bias": (s.n_heads * s.key_dim,),
                "gate_in": (s.gate_rank, s.hidden), "gate_out": (self.v_size, s.gate_rank),
                "out_norm": (s.value_dim,), "wo": (s.hidden, self.v_size)}

    def bind(self, params, ctx):
        s, self.ctx = self.spec, ctx
        stacked = torch.zeros((self.width, s.hidden), dtype=params["wq"].dtype)
        stacked[:self.channels] = torch.cat([params["wq"], params["wk"], params["wv"]], dim=0)
        stacked[self.at_b:self.at_b + s.n_heads] = params["wb"]
        stacked[self.at_decay:self.at_decay + s.decay_rank] = params["decay_in"]
        stacked[self.at_gate:self.at_gate + s.gate_rank] = params["gate_in"]
        self.in_proj = Linear(to_device(stacked, ctx, ctx.dtype))

        # the two products that widen the inner vectors as one: their inputs lie side by side in a row of the stacked
        # product, their matrices on the diagonal of one (the zeros cost a product of a few dozen columns nothing)
        ra, rg = _up8(s.decay_rank), _up8(s.gate_rank)
        both = torch.zeros((s.n_heads * s.key_dim + self.v_size, ra + rg), dtype=params["decay_out"].dtype)
        both[:s.n_heads * s.key_dim, :s.decay_rank] = params["decay_out"]
        both[s.n_heads * s.key_dim:, ra:ra + s.gate_rank] = params["gate_out"]
        self.widen = Linear(to_device(both, ctx, ctx.dtype))
        self.conv = to_device(torch.cat([params["conv_q"], params["conv_k"], params["conv_v"]], dim=0), ctx, torch.float32)
        self.decay_log = to_device(params["decay_log"], ctx, torch.float32)
        self.decay_bias = to_device(params["decay_bias"], ctx, torch.float32)
        self.out_norm = to_device(params["out_norm"], ctx, torch.float32)
        self.o_proj = Linear(to_device(params["wo"], ctx, ctx.dtype))

    def step_weights(self):
        return [self.in_proj.weight, self.widen.weight, self.conv, self.decay_log,
                self.decay_bias, self.out_norm, self.o_proj.weight]

    def cache_need(self):
        s = self.spec
        return CacheNeed(states=(("delta", (s.n_heads, s.value_dim, s.key_dim), "float32"),
                                 ("conv_tail", (max(s.conv_taps - 1, 0), self.channels), "float32")))

    def state_bytes(self):
        """Bytes of state a sequence holds in one entry (what a decode step reads and writes for it)."""
        s = self.spec
        return 4 * (s.n_heads * s.value_dim * s.key_dim + max(s.conv_taps - 1, 0) * self.channels)

    def forward(self, xn, out, batch, cache, ws):
        s, n, dt = self.spec, batch.n_rows, self.ctx.dtype
        if not cache.owns_storage:
            raise ops.KernelRefused("a delta-rule entry keeps a state of its own; it cannot read another entry's")
        state, tail = cache.states["delta"], cache.states["conv_tail"]
        proj = ws.get("delta_proj", (n, self.width), dt)
        self.in_proj.forward(xn, proj, n)
        qkv = ws.get("delta_qkv", (n, self.channels), dt)
        # a step of one token a sequence: the convolution leaves the new tails itself (a graph replays one kind of step only)
        ops.short_conv(proj, self.channels, self.conv, tail, qkv, batch, update_tail=batch.is_decode)
        if s.conv_taps > 1 and not batch.is_decode:
            ops.short_conv_tail(proj, self.channels, s.conv_taps, tail, batch)
        widened = ws.get("delta_widened", (n, s.n_heads * s.key_dim + self.v_size), torch.float32)
        self.widen.forward(proj[:, self.at_decay:self.width], widened, n)
        decay, gate = widened[:, :s.n_heads * s.key_dim], widened[:, s.n_heads * s.key_dim:]
        o = ws.get("delta_o", (n, self.v_size), torch.float32)
        ops.delta_scan(qkv, decay, proj[:, self.at_b:self.at_decay], self.decay_log, self.decay_bias, state, o, batch,
                       s.n_heads, s.n_kv_heads, s.key_dim, s.value_dim, ws)
        normed = ws.get("delta_normed", (n, self.v_size), dt)
        ops.gated_head_norm(o, gate, self.out_norm, normed, n, s.n_heads, s.value_dim, s.norm_eps)
        self.o_proj.forward(normed, out, n)
        return out


# From how many rows of a step on the recurrence with one decay a head runs in chunks of 64 tokens rather than token by
# token.
CHUNKED_FROM = 32


@MIXERS.register("head_delta")
class HeadDelta:
    """The gated delta rule with one decay per head (config.specs.HeadDeltaSpec): the recurrence above with
    g = exp(-exp(A_h) * softplus(a_h . x + bias_h)) for all key channels of head h, and an output gate silu(G x) from a
    full matrix. One stacked product makes q, k, v, the write strengths, the decays' inputs and the gate."""
    capturable = True  # its forward launches kernels only; nothing in it depends on the step's contents

    def __init__(self, spec):
        s = self.spec = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} heads do not divide into {s.n_kv_heads} key heads")
        if not 1 <= s.key_dim <= 256:
            raise ValueError(f"key_dim {s.key_dim}: the recurrence keeps up to 256 key channels a head")
        if not 1 <= s.conv_taps <= 8:
            raise ValueError(f"conv_taps {s.conv_taps}: the convolution takes 1 to 8 taps")
        self.qk_size, self.v_size = s.n_kv_heads * s.key_dim, s.n_heads * s.value_dim
        self.channels = 2 * self.qk_size + self.v_size
        self.at_b = _up8(self.channels)
        self.at_a = self.at_b + _up8(s.n_heads)
        self.at_gate = self.at_a + _up8(s.n_heads)
        self.width = self.at_gate + _up8(self.v_size)

    def param_shapes(self):
        s = self.spec
        return {"wq": (self.qk_size, s.hidden), "wk": (self.qk_size, s.hidden), "wv": (self.v_size, s.hidden),
                "conv_q": (self.qk_size, s.conv_taps), "conv_k": (self.qk_size, s.conv_taps),
                "conv_v": (self.v_size, s.conv_taps), "wb": (s.n_heads, s.hidden), "wa": (s.n_heads, s.hidden),
                "decay_log": (s.n_heads,), "decay_bias": (s.n_heads,), "wg": (self.v_size, s.hidden),
                "out_norm": (s.value_dim,), "wo": (s.hidden, self.v_size)}

    def bind(self, params, ctx):
        s, self.ctx = self.spec, ctx
        stacked = torch.zeros((self.width, s.hidden), dtype=params["wq"].dtype)
        stacked[:self.channels] = torch.cat([params["wq"], params["wk"], params["wv"]], dim=0)
        stacked[self.at_b:self.at_b + s.n_heads] = params["wb"]
        stacked[self.at_a:self.at_a + s.n_heads] = params["wa"]
        stacked[self.at_gate:self.at_gate + self.v_size] = params["wg"]
        self.in_proj = Linear(to_device(stacked, ctx, ctx.dtype))
        self.conv = to_device(torch.cat([params["conv_q"], params["conv_k"], params["conv_v"]], dim=0), ctx, torch.float32)
        self.decay_log = to_device(params["decay_log"], ctx, torch.float32)
        self.decay_bias = to_device(params["decay_bias"], ctx, torch.float32)
        self.out_norm = to_device(params["out_norm"], ctx, torch.float32)
        self.o_proj = Linear(to_device(params["wo"], ctx, ctx.dtype))

    def step_weights(self):
        return [self.in_proj.weight, self.conv, self.decay_log, self.decay_bias, self.out_norm, self.o_proj.weight]

    def cache_need(self):
        s = self.spec
        return CacheNeed(states=(("delta", (s.n_heads, s.value_dim, s.key_dim), "float32"),
                                 ("conv_tail", (max(s.conv_taps - 1, 0), self.channels), "float32")))

    def state_bytes(self):
        """Bytes of state a sequence holds in one entry (what a decode step reads and writes for it)."""
        s = self.spec
        return 4 * (s.n_heads * s.value_dim * s.key_dim + max(s.conv_taps - 1, 0) * self.channels)

    def forward(self, xn, out, batch, cache, ws):
        s, n, dt = self.spec, batch.n_rows, self.ctx.dtype
        if not cache.owns_storage:
            raise ops.KernelRefused("a delta-rule entry keeps a state of its own; it cannot read another entry's")
        state, tail = cache.states["delta"], cache.states["conv_tail"]
        proj = ws.get("delta_proj", (n, self.width), dt)
        self.in_proj.forward(xn, proj, n)
        qkv = ws.get("delta_qkv", (n, self.channels), dt)
        ops.short_conv(proj, self.channels, self.conv, tail, qkv, batch, update_tail=batch.is_decode)
        if s.conv_taps > 1 and not batch.is_decode:
            ops.short_conv_tail(proj, self.channels, s.conv_taps, tail, batch)
        o = ws.get("delta_o", (n, self.v_size), torch.float32)
        ops.delta_scan(qkv, proj[:, self.at_a:self.at_gate], proj[:, self.at_b:self.at_a], self.decay_log, self.decay_bias,
                       state, o, batch, s.n_heads, s.n_kv_heads, s.key_dim, s.value_dim, ws, per_head=True,
                       chunks=not batch.is_decode and n >= CHUNKED_FROM)
        normed = ws.get("delta_normed", (n, self.v_size), dt)
        ops.gated_head_norm(o, proj[:, self.at_gate:self.at_gate + self.v_size], self.out_norm, normed, n, s.n_heads,
                            s.value_dim, s.norm_eps, silu=True)
        self.o_proj.forward(normed, out, n)
        return out
