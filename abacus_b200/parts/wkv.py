"""A recurrent mixer: time mixing with a decay per head, key channel and token, and a bonus for the token's own key
(config.specs.WkvSpec).

Each of r, k, v, the gate and the decay reads a blend of the token's row with the row before it (the sequence's last row
is part of its state); per head a float32 state S [key, value], zero at a sequence's start:
    o = (S + diag(u) k v^T)^T r;    S <- diag(w) S + k v^T;    w = exp(-exp(W2 tanh(W1 m_w) + w0))
Each head's o is divided by its root mean square, the heads side by side are multiplied by a weight and by silu(Wg m_g),
then projected. The mixer keeps no keys: its cache is the state, and its cost per token does not grow. The blends, the
decay from its pre-activation on (the second product's float32 output, both exponentials), the state, the recurrence,
the norm and the gate's activation are float32 in both number formats.
"""
import torch

from ..cache.need import CacheNeed
from ..kernels import ops
from .base import MIXERS, to_device
from .linear import Linear, rows_kernel_wins

_BLENDS = ("r", "k", "v", "g", "w")


def _up8(n):
    return -(-n // 8) * 8


def _up16(n):
    return -(-n // 16) * 16


@MIXERS.register("wkv")
class Wkv:
    capturable = True  # its forward launches kernels only; nothing in it depends on the step's contents

    def __init__(self, spec):
        s = self.spec = spec
        if not 1 <= s.key_dim <= 256:
            raise ValueError(f"key_dim {s.key_dim}: the recurrence keeps up to 256 key channels a head")
        if s.decay_rank < 1:
            raise ValueError(f"decay_rank {s.decay_rank}: the decay's two matrices have an inner size")
        self.size = s.n_heads * s.key_dim
        # columns of the projections r, k, v, gate, each from a multiple of 16 on, and behind them the decay's inner vector
        self.block = _up16(self.size)
        self.at = {name: i * self.block for i, name in enumerate(("r", "k", "v", "g", "w"))}
        self.rank = _up8(s.decay_rank)
        self.width = 4 * self.block + self.rank

    def param_shapes(self):
        s = self.spec
        shapes = {f"mu_{b}": (s.hidden,) for b in _BLENDS}
        shapes.update({f"w{b}": (self.size, s.hidden) for b in ("r", "k", "v", "g")})
        shapes.update(w1=(s.decay_rank, s.hidden), w2=(self.size, s.decay_rank), w0=(self.size,),
                      bonus=(s.n_heads, s.key_dim), out_norm=(self.size,), wo=(s.hidden, self.size))
        return shapes

    def bind(self, params, ctx):
        s, self.ctx = self.spec, ctx
        self.mu = to_device(torch.stack([params[f"mu_{b}"].to(torch.float32) for b in _BLENDS]), ctx, torch.float32)
        # the five products that read the five blends, as one matrix: r, k, v, gate (each from a multiple of 16 rows on)
        # and the first of the decay's pair (its inner size padded with zeros to a multiple of 8). A step of a few rows
        # makes all five in one launch; else each is a product of its own on its rows of the matrix.
        stacked = torch.zeros((self.width, s.hidden), dtype=params["wr"].dtype)
        for b in ("r", "k", "v", "g"):
            stacked[self.at[b]:self.at[b] + self.size] = params[f"w{b}"]
        stacked[self.at["w"]:self.at["w"] + s.decay_rank] = params["w1"]
        self.stacked = to_device(stacked, ctx, ctx.dtype)
        self.proj = {b: Linear(self.stacked[self.at[b]:self.at[b] + self.size]) for b in ("r", "k", "v", "g")}
        self.w1 = Linear(self.stacked[self.at["w"]:])
        w2 = torch.zeros((self.size, self.rank), dtype=params["w2"].dtype)
        w2[:, :s.decay_rank] = params["w2"]
        self.w2 = Linear(to_device(w2, ctx, ctx.dtype))
        self.w0 = to_device(params["w0"], ctx, torch.float32)
        self.bonus = to_device(params["bonus"].reshape(-1), ctx, torch.float32)
        self.out_norm = to_device(params["out_norm"], ctx, torch.float32)
        self.o_proj = Linear(to_device(params["wo"], ctx, ctx.dtype))

    def step_weights(self):
        return [self.mu, self.stacked, self.w2.weight, self.w0, self.bonus,
                self.out_norm, self.o_proj.weight]

    def cache_need(self):
        s = self.spec
        return CacheNeed(states=(("wkv_state", (s.n_heads, s.key_dim, s.key_dim), "float32"),
                                 ("wkv_last", (s.hidden,), "float32")))

    def state_bytes(self):
        """Bytes of state a sequence holds in one entry (what a decode step reads and writes for it)."""
        s = self.spec
        return 4 * (s.n_heads * s.key_dim * s.key_dim + s.hidden)

    def forward(self, xn, out, batch, cache, ws):
        s, n, dt = self.spec, batch.n_rows, self.ctx.dtype
        if not cache.owns_storage:
            raise ops.KernelRefused("a recurrent entry keeps a state of its own; it cannot read another entry's")
        blends = ws.get("wkv_blends", (len(_BLENDS), n, s.hidden), dt)
        ops.token_shift(xn, self.mu, cache.states["wkv_last"], blends, batch)
        proj = ws.get("wkv_proj", (n, self.width), dt)
        inner = ws.get("wkv_inner", (n, self.rank), dt)
        if (dt == torch.bfloat16 and self.rank <= self.block and rows_kernel_wins(n, self.stacked)
                and ops.gemm_rows_takes(blends[0], self.stacked, proj, n)):
            # a few rows: the five products in one launch, each run of the matrix's rows against its own blend
            # (the decay's inner vector passes tanh where its product stores it)
            ops.gemm_rows_planes(blends, self.stacked, proj, self.block, n, tanh_from=self.at["w"])
            inner = proj[:, self.at["w"]:]
        else:
            for i, b in enumerate(("r", "k", "v", "g")):
                self.proj[b].forward(blends[i], proj[:, self.at[b]:self.at[b] + self.size], n)
            sums = ws.get("wkv_inner_sums", (n, self.rank), torch.float32)
            self.w1.forward(blends[4], sums, n)
            ops.tanh_rows(sums, inner, n)
        pre = ws.get("wkv_pre", (n, self.size), torch.float32)
        self.w2.forward(inner, pre, n)
        o = ws.get("wkv_o", (n, self.size), torch.float32)
        ops.wkv_scan(proj, self.at["r"], self.at["k"], self.at["v"], s.n_heads, s.key_dim, pre, self.w0, self.bonus,
                     cache.states["wkv_state"], o, batch, ws=ws)
        normed = ws.get("wkv_normed", (n, self.size), dt)
        ops.gated_head_norm(o, proj[:, self.at["g"]:self.at["g"] + self.size], self.out_norm, normed, n, s.n_heads, s.key_dim,
                            s.norm_eps, silu=True)
        self.o_proj.forward(normed, out, n)
        return out
