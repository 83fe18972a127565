"""A recurrent mixer: a matrix memory per head with exponential gates (config.specs.MatrixMemorySpec), the recurrence of
an mLSTM layer.

Per head a float32 state C [key, value], n [key] and a running maximum m, all zero at a sequence's start:
    i = cap tanh((wi . x + bi) / cap)        f = logsigmoid(cap tanh((wf . x + bf) / cap))
    m' = max(f + m, i)    C' = e^(f + m - m') C + e^(i - m') k v^T    n' = e^(f + m - m') n + e^(i - m') k
    o = C'^T q / (max(|n' . q|, e^(-m')) + denom_eps),      q = key^-1/2 Wq x
The mixer owns what stands around it: one stacked product for q, k, v and the output gate, a small product of its own
for the two gates' pre-activations (float32 out of it: they stand in exponents), the per-head norm of o with its weight
and sigmoid(Wg x), the output product. Steps that bring prompts run the recurrence in chunks of 64 tokens (the same
numbers, summed in another order); a token a sequence runs it as it stands. It keeps no keys: its cache is the state, and its cost per token does not grow.
The gates, the state, the read-out, the norm and the gate's sigmoid are float32 in both number formats.
"""
import torch

from ..cache.need import CacheNeed
from ..kernels import ops
from .base import MIXERS, to_device
from .linear import Linear


# From how many rows of a step on the recurrence runs in chunks (three launches whose work lies side by side) rather than
# token by token (one launch that walks every sequence).
CHUNKED_FROM = 32


def _up8(n):
    return -(-n // 8) * 8


@MIXERS.register("matrix_memory")
class MatrixMemory:
    capturable = True  # its forward launches kernels only; nothing in it depends on the step's contents

    def __init__(self, spec):
        s = self.spec = spec
        if not 1 <= s.key_dim <= 256:
            raise ValueError(f"key_dim {s.key_dim}: the recurrence keeps up to 256 key channels a head")
        if s.n_heads < 1 or s.value_dim < 1:
            raise ValueError(f"{s.n_heads} heads of {s.value_dim} values")
        if not s.gate_cap > 0:
            raise ValueError(f"gate_cap {s.gate_cap}: the gates' cap is positive")
        self.qk_size, self.v_size = s.n_heads * s.key_dim, s.n_heads * s.value_dim
        # columns of the stacked product: q, k, v, the output gate, each from a multiple of 8 elements on
        self.at_k = _up8(self.qk_size)
        self.at_v = self.at_k + _up8(self.qk_size)
        self.at_g = self.at_v + _up8(self.v_size)
        self.width = self.at_g + _up8(self.v_size)
        self.gates_width = _up8(2 * s.n_heads)  # i's pre-activations, then f's

    def param_shapes(self):
        s = self.spec
        return {"wq": (self.qk_size, s.hidden), "wk": (self.qk_size, s.hidden), "wv": (self.v_size, s.hidden),
                "wg": (self.v_size, s.hidden), "wi": (s.n_heads, s.hidden), "bi": (s.n_heads,),
                "wf": (s.n_heads, s.hidden), "bf": (s.n_heads,), "out_norm": (self.v_size,), "wo": (s.hidden, self.v_size)}

    def bind(self, params, ctx):
        s, self.ctx = self.spec, ctx
        stacked = torch.zeros((self.width, s.hidden), dtype=params["wq"].dtype)
        for at, slot in ((0, "wq"), (self.at_k, "wk"), (self.at_v, "wv"), (self.at_g, "wg")):
            stacked[at:at + params[slot].shape[0]] = params[slot]
        self.in_proj = Linear(to_device(stacked, ctx, ctx.dtype))
        gates = torch.zeros((self.gates_width, s.hidden), dtype=params["wi"].dtype)
        gates[:s.n_heads], gates[s.n_heads:2 * s.n_heads] = params["wi"], params["wf"]
        self.gates_proj = Linear(to_device(gates, ctx, ctx.dtype))
        self.bias_i = to_device(params["bi"], ctx, torch.float32)
        self.bias_f = to_device(params["bf"], ctx, torch.float32)
        self.out_norm = to_device(params["out_norm"], ctx, torch.float32)
        self.o_proj = Linear(to_device(params["wo"], ctx, ctx.dtype))
        self.blocks = None

    def step_weights(self):
        return [self.in_proj.weight, self.gates_proj.weight, self.bias_i, self.bias_f, self.out_norm, self.o_proj.weight]

    def _blocks(self):
        return -(-self.spec.value_dim // 8)  # one copy of n and m per CTA that walks a head (8 value columns each)

    def cache_need(self):
        s, b = self.spec, self._blocks()
        return CacheNeed(states=(("memory", (s.n_heads, s.value_dim, s.key_dim), "float32"),
                                 ("memory_n", (s.n_heads, b, s.key_dim), "float32"),
                                 ("memory_m", (s.n_heads, b), "float32")))

    def state_bytes(self):
        """Bytes of state a sequence holds in one entry (what a decode step reads and writes for it)."""
        s, b = self.spec, self._blocks()
        return 4 * s.n_heads * (s.value_dim * s.key_dim + b * s.key_dim + b)

    def forward(self, xn, out, batch, cache, ws):
        s, n, dt = self.spec, batch.n_rows, self.ctx.dtype
        if not cache.owns_storage:
            raise ops.KernelRefused("a recurrent entry keeps a state of its own; it cannot read another entry's")
        if self.blocks is None:
            self.blocks = ops.matrix_memory_blocks(s.value_dim)
            assert self.blocks == self._blocks(), "the kernel's value columns a CTA differ from the state's layout"
        proj = ws.get("memory_proj", (n, self.width), dt)
        self.in_proj.forward(xn, proj, n)
        gates = ws.get("memory_gates", (n, self.gates_width), torch.float32)
        self.gates_proj.forward(xn, gates, n)
        o = ws.get("memory_o", (n, self.v_size), torch.float32)
        ops.matrix_memory(proj, 0, self.at_k, self.at_v, gates, self.bias_i, self.bias_f, s.gate_cap, s.denom_eps, s.n_heads,
                          s.key_dim, s.value_dim, cache.states["memory"], cache.states["memory_n"],
                          cache.states["memory_m"], o, batch,
                          ws=ws if not batch.is_decode and n >= CHUNKED_FROM else None)
        normed = ws.get("memory_normed", (n, self.v_size), dt)
        ops.gated_head_norm(o, proj[:, self.at_g:self.at_g + self.v_size], self.out_norm, normed, n, s.n_heads, s.value_dim,
                            s.norm_eps)
        self.o_proj.forward(normed, out, n)
        return out
