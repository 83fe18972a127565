"""Grouped-query causal attention over the paged cache (src/model.c:197-211, 247-259).

The mixer owns the q/k/v and output projections, the optional per-head norm of
q and k, and a position encoding; its sizes, scale, eps and window come from
its spec. q, k and v are one stacked matrix, as in src/model.c:88-93.

Options of the spec that only the general kernels take: values of another size than keys, a sequence's first keys
kept behind a window, a sink, float32 weights, a short causal convolution over time on every channel of q, k and v
right after their projection (its last inputs are part of the sequence's state, beside the keys and values), keys
seen only within the token's own chunk of positions, and capped scores.
"""
import os

import torch

from ..cache.need import CacheNeed
from ..kernels import ops
from .attention_plan import AttentionLists, AttentionStepPlan
from .base import MIXERS, POSITIONS, to_device
from .linear import Linear


# A decode step's attention kernel can norm and rotate q and k and write the new key and value to the cache itself: a
# launch less in every layer. ABACUS_DECODE_PREPARES=0 keeps the preparation a kernel of its own (for comparison).
DECODE_PREPARES = os.environ.get("ABACUS_DECODE_PREPARES", "1") != "0"
# The q/k/v product of a long prompt step can do the same in its epilogue (heads of 128): a kernel and a pass over
# q, k and v less. ABACUS_PRODUCT_PREPARES=0 keeps the preparation a kernel of its own (for comparison).
PRODUCT_PREPARES = os.environ.get("ABACUS_PRODUCT_PREPARES", "1") != "0"


@MIXERS.register("attention")
class Attention:
    capturable = True  # its forward launches kernels only; nothing in it depends on the step's contents

    def __init__(self, spec):
        s = self.spec = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} query heads do not divide into {s.n_kv_heads} kv heads")
        self.v_dim = s.v_head_dim or s.head_dim
        if self.v_dim < 1 or self.v_dim > 256:
            raise ValueError(f"v_head_dim {self.v_dim}: the attention kernels take value heads of up to 256")
        if s.keep_first and s.window is None:
            raise ValueError("keep_first goes with a window")
        # what only the general kernel takes: values of another size, kept first keys, a sink, float32 weights
        # q and k normed over their whole rows, values that are their keys, a gate per head: a preparation kernel of
        # their own (out of the projection's rows into the rows the attention kernels read), then the general kernels
        self.whole = s.norm_over == "projection" or s.values == "keys"
        if s.norm_over not in ("head", "projection") or s.values not in ("own", "keys"):
            raise ValueError(f"norm_over {s.norm_over!r} is neither head nor projection, or values {s.values!r} neither own nor keys")
        if self.whole and (s.conv_taps or (s.v_head_dim or s.head_dim) != s.head_dim
                           or (s.qk_norm_eps is not None and s.norm_over != "projection")):
            raise ValueError("values that are their keys and norms over the whole projection go with neither a convolution, "
                             "values of another size nor a norm per head")
        self.general = (self.v_dim != s.head_dim or bool(s.keep_first) or s.sink or s.exact_weights or s.conv_taps > 0
                        or bool(s.chunk) or bool(s.softcap) or self.whole or s.head_gate)
        if s.conv_taps < 0 or s.conv_taps > 8:
            raise ValueError(f"conv_taps {s.conv_taps}: the convolution takes 1 to 8 taps")
        if s.chunk is not None and s.chunk < 1:
            raise ValueError(f"chunk {s.chunk}: a chunk has at least one position")
        if s.softcap is not None and not s.softcap > 0:
            raise ValueError(f"softcap {s.softcap}: the cap of the scores is positive")
        if s.head_dim > 256 or s.head_dim < 1 or (s.head_dim % 8 and not self.general):
            raise ValueError(f"head_dim {s.head_dim}: the attention kernels take multiples of 8 up to 256 (the general "
                             "kernel, which a layer with a sink, kept first keys or values of their own size runs on, "
                             "any size up to 256)")
        self.position = POSITIONS.build(s.position) if s.position is not None else None
        self.q_size, self.kv_size = s.n_heads * s.head_dim, s.n_kv_heads * s.head_dim
        self.v_size = s.n_kv_heads * self.v_dim
        # a row of q, k and v is padded to a multiple of 8 elements, so that every row starts 16-byte aligned whatever
        # the values' size (nothing to pad where values are as large as keys: head_dim is a multiple of 8)
        self.row = -(-(self.q_size + self.kv_size + self.v_size) // 8) * 8
        # a row of the stacked product: q, k, v (if projected), then the heads' gates from a multiple of 8 on
        own_v = self.v_size if s.values == "own" else 0
        self.gate_at = -(-(self.q_size + self.kv_size + own_v) // 8) * 8
        self.proj_row = self.gate_at + (-(-s.n_heads // 8) * 8 if s.head_gate else 0) if (self.whole or s.head_gate) else self.row
        self.cos = self.sin = None
        # A step of several tokens of a windowed layer is checked on the host (it may have to be refused): such steps
        # cannot be replayed from a captured graph; single-token steps can. A layer with the general options decides on
        # the host whether a step reads its keys from the step's own rows; for steps whose sequences all start at
        # their first token the answer is always yes, so those may be captured ("from_start").
        self.capturable_prompts = "from_start" if self.general else s.window is None
        self.lists = AttentionStepPlan(s.n_heads)  # the prefill kernels' tiles and work list, made per step

    def step_plans(self):
        """What this mixer wants made on the host for every step and sent with the step's indices."""
        return [self.lists]

    def step_weights(self):
        """The tensors a step reads once whatever its size (for the bytes a decode step must move)."""
        return [self.qkv_proj.weight, self.o_proj.weight, self.q_norm, self.k_norm, self.sink, self.conv]

    def param_shapes(self):
        s = self.spec
        shapes = {"wq": (self.q_size, s.hidden), "wk": (self.kv_size, s.hidden), "wv": (self.v_size, s.hidden),
                  "wo": (s.hidden, s.n_heads * self.v_dim)}
        if s.values == "keys":
            del shapes["wv"]
        if s.head_gate:
            shapes["wg"] = (s.n_heads, s.hidden)
        if s.qk_norm_eps is not None and s.norm_over == "projection":
            shapes.update(q_norm=(self.q_size,), k_norm=(self.kv_size,))
        elif s.qk_norm_eps is not None:
            shapes.update(q_norm=(s.head_dim,), k_norm=(s.head_dim,))
        if s.sink:
            shapes["sink"] = (s.n_heads,)
        if s.conv_taps:
            shapes.update(conv_q=(self.q_size, s.conv_taps), conv_k=(self.kv_size, s.conv_taps),
                          conv_v=(self.v_size, s.conv_taps))
        return shapes

    def bind(self, params, ctx):
        self.ctx = ctx
        wqkv = torch.cat([params["wq"], params["wk"]] + ([params["wv"]] if "wv" in params else []), dim=0)
        if self.proj_row > wqkv.shape[0]:
            wqkv = torch.cat([wqkv, torch.zeros((self.proj_row - wqkv.shape[0], wqkv.shape[1]), dtype=wqkv.dtype, device=wqkv.device)], dim=0)
        if self.spec.head_gate:
            wqkv[self.gate_at:self.gate_at + self.spec.n_heads] = params["wg"]
        self.qkv_proj = Linear(to_device(wqkv, ctx, ctx.dtype))
        self.q_proj = Linear(self.qkv_proj.weight[:self.q_size])  # for entries that read another entry's cache
        self.o_proj = Linear(to_device(params["wo"], ctx, ctx.dtype))
        self.q_norm = to_device(params["q_norm"], ctx, torch.float32) if "q_norm" in params else None
        self.k_norm = to_device(params["k_norm"], ctx, torch.float32) if "k_norm" in params else None
        self.sink = to_device(params["sink"], ctx, torch.float32) if "sink" in params else None
        self.conv = None
        if self.spec.conv_taps:  # one table for the whole row of q, k and v; the row's padding has taps of zero
            taps = torch.cat([params["conv_q"], params["conv_k"], params["conv_v"]], dim=0).to(torch.float32)
            table = torch.zeros((self.row, self.spec.conv_taps), dtype=torch.float32)
            table[:taps.shape[0]] = taps
            self.conv = to_device(table, ctx, torch.float32)

    def cache_need(self):
        s = self.spec
        states = (("conv_tail", (s.conv_taps - 1, self.row), "float32"),) if s.conv_taps > 1 else ()
        return CacheNeed(n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window, v_head_dim=self.v_dim,
                         keep_first=s.keep_first if s.window is not None else 0, states=states)

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.cos, self.sin = self.position.tables(max_positions, device)

    def forward(self, xn, out, batch, cache, ws):
        s = self.spec
        n = batch.n_rows
        qkv = ws.get("qkv", (n, self.row), self.ctx.dtype)
        att = ws.get("att", (n, s.n_heads * self.v_dim), self.ctx.dtype)
        writes = cache.owns_storage
        rotary_dim = self.position.rotary_dim if self.position else 0
        interleaved = self.position.interleaved if self.position else False
        # A windowed cache keeps only the last keys; a prompt longer than that reads its keys from
        # this step's own rows, which hold all of them when the sequences start at position 0.
        from_step = s.window is not None and not batch.is_decode
        w = self.qkv_proj.weight
        prepared = False  # by the product's own kernel: a prompt's heads in its epilogue
        if (PRODUCT_PREPARES and writes and not batch.is_decode and not from_step and w.dtype == torch.bfloat16
                and not self.general
                and ops.gemm_tc_qkv_takes(xn, w, qkv, n, s.n_heads, s.n_kv_heads, s.head_dim, cache.kv, self.q_norm,
                                          self.k_norm, self.cos, self.sin, rotary_dim, interleaved)):
            ops.gemm_tc_qkv(xn, w, qkv, s.n_heads, s.n_kv_heads, batch, self.q_norm, self.k_norm, s.qk_norm_eps,
                            self.cos, self.sin, cache.kv, n)
            prepared = True
        elif self.whole or s.head_gate:
            # the projection into rows of its own (q, k, v if projected, the heads' gates); q, k and v go from there
            # into the rows the attention kernels read
            proj = ws.get("qkv_proj", (n, self.proj_row), self.ctx.dtype)
            if writes:
                self.qkv_proj.forward(xn, proj, n)
            else:
                raise ops.KernelRefused("an attention entry whose values are its keys, or with gated heads, keeps keys of its own")
            if self.whole:
                ops.qkv_prep_whole(proj, qkv, s.n_heads, s.n_kv_heads, s.head_dim, batch, self.q_norm, self.k_norm,
                                   s.qk_norm_eps, self.cos, self.sin, rotary_dim, interleaved, cache.kv)
                prepared = True
            else:
                qkv[:n, :self.gate_at].copy_(proj[:n, :self.gate_at])
        elif writes and self.conv is not None:
            # the projection, then the convolution over time into the row the kernels read; the slot's tail follows
            proj = ws.get("qkv_proj", (n, self.row), self.ctx.dtype)
            self.qkv_proj.forward(xn, proj, n)
            tail = cache.states["conv_tail"] if s.conv_taps > 1 else ws.get("no_tail", (1, 0, self.row), torch.float32)
            ops.short_conv(proj, self.row, self.conv, tail, qkv, batch, update_tail=batch.is_decode, plain=True)
            if s.conv_taps > 1 and not batch.is_decode:
                ops.short_conv_tail(proj, self.row, s.conv_taps, tail, batch)
        elif writes:
            self.qkv_proj.forward(xn, qkv, n)
        elif self.conv is not None:
            raise ops.KernelRefused("an attention entry with a convolution keeps a state of its own; it cannot read "
                                    "another entry's cache")
        else:  # keys and values are another entry's: only q is needed
            self.q_proj.forward(xn, qkv[:, :self.q_size], n)
        prepare = None
        if prepared:
            pass
        elif (DECODE_PREPARES and batch.is_decode and cache.kv is not None and not self.general
                and ops.attention_decode_prepares(qkv, s.n_heads, s.n_kv_heads, s.head_dim, cache.kv, self.q_norm,
                                                  self.k_norm, self.cos, self.sin, rotary_dim, interleaved)):
            prepare = dict(q_norm=self.q_norm, k_norm=self.k_norm, eps=s.qk_norm_eps, cos=self.cos, sin=self.sin, keep=writes)
        else:
            ops.qkv_prep(qkv, s.n_heads, s.n_kv_heads, s.head_dim, batch, self.q_norm, self.k_norm, s.qk_norm_eps,
                         self.cos, self.sin, rotary_dim, interleaved, cache.kv if writes else None, q_only=not writes,
                         v_dim=self.v_dim, row=self.row if self.general else None)
        if from_step and (batch.any_continuation or not writes):
            raise ops.KernelRefused("windowed attention takes several tokens of a sequence only at its start, "
                                    "and only with keys of its own")
        mine = batch.plan.get(self.lists.name)
        gates = ws.get("qkv_proj", (n, self.proj_row), self.ctx.dtype)[:, self.gate_at:] if s.head_gate else None
        gated = ops.attention(qkv, att, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, s.window, batch, cache.kv,
                      from_step=from_step, ws=ws, lists=AttentionLists(mine) if mine is not None else None, prepare=prepare,
                      v_dim=self.v_dim, keep_first=s.keep_first, sink=self.sink, exact_weights=s.exact_weights,
                      row=self.row if self.general else None, chunk=s.chunk, softcap=s.softcap, gate=gates)
        if s.head_gate and not gated:  # head h's output times sigmoid(g_h . x), where the attention kernel did not do it
            ops.gate_heads(att, gates, s.n_heads, self.v_dim, n)
        self.o_proj.forward(att, out, n)
        return out
