"""Latent attention: causal attention whose keys and values are kept as one low-rank latent row per token that all
heads share (config.specs.LatentAttentionSpec).

Per token the cache holds [c | r]: c, the normed down-projection (rank elements), and r, one rotated key part
(rot_dim) common to the heads. Head h's key is [Uk_h c | r] and its value Uv_h c. Two ways to the same scores:

  over the cache (any step):  (Uk_h c) . q = c . (Uk_h^T q), so each query head is carried into the latent space,
      [Uk_h^T q_plain | q_rotated], and attention runs over the cache rows with one kv head whose values are the first
      `rank` elements of its keys; Uv_h is applied to the weighted sum of latents. A decode step reads rank + rot_dim
      elements a token for all heads together.
  in full size (bfloat16 prompts from their first token): keys and values of every head are made from the step's own
      latents by one product, the shared part copied behind each head's keys, and the prompt kernels for ordinary heads
      run on them.

Scores, softmax weights, the norm of the latent and the rotation are float32 in both number formats.
"""
import torch

from ..cache.need import CacheNeed
from ..kernels import ops
from .base import MIXERS, POSITIONS, to_device
from .linear import Linear


def _up8(n):
    return -(-n // 8) * 8


@MIXERS.register("latent_attention")
class LatentAttention:
    capturable = True  # its forward launches kernels only
    # which of the two ways a step of several tokens takes depends on whether its sequences start at their first
    # token: a captured prompt step is replayed only for steps that do
    capturable_prompts = "from_start"

    def __init__(self, spec):
        s = self.spec = spec
        if s.rot_dim % 2 or s.rot_dim < 0:
            raise ValueError(f"rot_dim {s.rot_dim} must be even")
        self.position = POSITIONS.build(s.position) if s.position is not None and s.rot_dim else None
        if self.position is not None and self.position.rotary_dim > s.rot_dim:
            raise ValueError("latent attention rotates pairs of at most rot_dim elements")
        self.interleaved = self.position.interleaved if self.position is not None else True
        self.per_head = s.head_dim + s.rot_dim
        self.q_size = s.n_heads * self.per_head
        self.row = _up8(s.rank + s.rot_dim)          # a cache row, and a query head in the latent space
        self.down_at = _up8(self.q_size)             # where the down-projection starts in a row of the first product
        self.proj_width = self.down_at + (0 if s.shares_latents else _up8(s.rank + s.rot_dim))
        # behind them, where the layer has them: the queries' own latent (its product then fills the first columns from
        # the normed latent) and the heads' gates
        self.q_latent_at = self.proj_width
        self.q_rank8 = _up8(s.q_rank) if s.q_rank else 0
        self.gate_at = self.q_latent_at + self.q_rank8
        self.proj_width = self.gate_at + (_up8(s.n_heads) if s.head_gate else 0)
        self.cos = self.sin = None
        if self.row > 640:
            raise ValueError(f"rank {s.rank} + rot_dim {s.rot_dim}: the attention kernels take rows of up to 640")

    def param_shapes(self):
        s = self.spec
        shapes = {"wq": (self.q_size, s.q_rank or s.hidden), "wuk": (s.n_heads * s.head_dim, s.rank),
                  "wuv": (s.n_heads * s.v_head_dim, s.rank), "wo": (s.hidden, s.n_heads * s.v_head_dim)}
        if not s.shares_latents:
            shapes.update(wdown=(s.rank + s.rot_dim, s.hidden), down_norm=(s.rank,))
        if s.sink:
            shapes["sink"] = (s.n_heads,)
        if s.q_rank:
            shapes.update(wdq=(s.q_rank, s.hidden), q_norm=(s.q_rank,))
        if s.head_gate:
            shapes["wg"] = (s.n_heads, s.hidden)
        return shapes

    def bind(self, params, ctx):
        s, self.ctx = self.spec, ctx
        # the first product's matrix: the queries (or, where they pass a latent of their own, that latent's rows behind
        # the others), the down-projection, the heads' gates, each from a multiple of 8 rows on
        base = self.down_at if s.q_rank else 0  # with a latent of their own the queries are no part of the first product
        stacked = torch.zeros((self.proj_width - base, s.hidden), dtype=params["wq"].dtype)
        if not s.q_rank:
            stacked[:self.q_size] = params["wq"]
        if not s.shares_latents:
            stacked[self.down_at - base:self.down_at - base + s.rank + s.rot_dim] = params["wdown"]
        self.q_up = self.q_norm = None
        if s.q_rank:  # a second product makes the queries from the normed latent
            stacked[self.q_latent_at - base:self.q_latent_at - base + s.q_rank] = params["wdq"]
            up = torch.zeros((self.q_size, self.q_rank8), dtype=params["wq"].dtype)
            up[:, :s.q_rank] = params["wq"]
            self.q_up = Linear(to_device(up, ctx, ctx.dtype))
            self.q_norm = to_device(params["q_norm"], ctx, torch.float32)
        if s.head_gate:
            stacked[self.gate_at - base:self.gate_at - base + s.n_heads] = params["wg"]
        self.in_proj = Linear(to_device(stacked, ctx, ctx.dtype))
        uk = params["wuk"].reshape(s.n_heads, s.head_dim, s.rank)
        self.uk_t = to_device(uk.transpose(1, 2).contiguous(), ctx, ctx.dtype)          # [heads, rank, head_dim]
        self.uv = to_device(params["wuv"].reshape(s.n_heads, s.v_head_dim, s.rank), ctx, ctx.dtype)
        # for prompts in full size: every head's keys (a head's rows, then rot_dim rows of zeros where the shared
        # part is copied to) and values from the latents in one product
        full = torch.zeros((self.q_size + s.n_heads * s.v_head_dim, _up8(s.rank)), dtype=params["wuk"].dtype)
        full[:self.q_size].view(s.n_heads, self.per_head, -1)[:, :s.head_dim, :s.rank] = uk
        full[self.q_size:, :s.rank] = params["wuv"]
        self.up_full = Linear(to_device(full, ctx, ctx.dtype))
        self.o_proj = Linear(to_device(params["wo"], ctx, ctx.dtype))
        self.down_norm = to_device(params["down_norm"], ctx, torch.float32) if "down_norm" in params else None
        self.sink = to_device(params["sink"], ctx, torch.float32) if "sink" in params else None

    def step_weights(self):
        return [self.in_proj.weight, self.uk_t, self.uv, self.o_proj.weight, self.down_norm, self.sink, self.q_norm,
                self.q_up.weight if self.q_up is not None else None]

    def cache_need(self):
        s = self.spec
        return CacheNeed(n_kv_heads=1, head_dim=self.row, v_head_dim=s.rank, values_in_keys=True)

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.cos, self.sin = self.position.tables(max_positions, device)

    def full_size_takes(self, batch):
        """Whether this step makes keys and values in full size: bfloat16 prompts that start at their first token, with
        sizes the prompt kernel for ordinary heads takes (else the general kernel would run them, and over the cache
        it has less to read)."""
        s = self.spec
        return (self.ctx.dtype == torch.bfloat16 and not batch.is_decode and not batch.any_continuation
                and self.per_head % 8 == 0 and self.per_head <= 256 and s.v_head_dim % 8 == 0 and 8 <= s.v_head_dim <= 128
                and s.rank % 8 == 0)

    def forward(self, xn, out, batch, cache, ws):
        s, n, dt = self.spec, batch.n_rows, self.ctx.dtype
        if cache.owns_storage == s.shares_latents:
            raise ops.KernelRefused("a latent-attention entry either has a down-projection and a cache of its own, or "
                                    "neither and another entry's cache")
        rot_dims = self.position.rotary_dim if self.position is not None else 0
        proj = ws.get("latent_proj", (n, self.proj_width), dt)
        if self.q_up is not None:
            self.in_proj.forward(xn, proj[:, self.down_at:], n)
            q_latent = proj[:, self.q_latent_at:self.q_latent_at + self.q_rank8]  # (its padding columns are zeros)
            ops.columns_norm(q_latent, q_latent, s.q_rank, self.q_norm, s.norm_eps, n)
            self.q_up.forward(q_latent, proj[:, :self.q_size], n)
        else:
            self.in_proj.forward(xn, proj, n)
        att = ws.get("att", (n, s.n_heads * s.v_head_dim), dt)
        kv = cache.kv
        gated = False
        if self.full_size_takes(batch):
            heads_size = 2 * self.q_size + s.n_heads * s.v_head_dim
            qkv = ws.get("latent_qkv", (n, _up8(heads_size)), dt)
            ops.latent_prep(proj, self.down_at, s.n_heads, s.head_dim, s.rot_dim, s.rank, rot_dims, self.down_norm,
                            s.norm_eps, self.cos, self.sin, qkv, self.per_head, s.head_dim, True,
                            kv if cache.owns_storage else None, batch, interleaved=self.interleaved)
            rows = ws.get("latent_rows", (n, self.row), dt)
            ops.latent_rows(kv, rows, self.row, batch)
            self.up_full.forward(rows[:, :_up8(s.rank)], qkv[:, self.q_size:heads_size], n)
            ops.spread_shared(rows[:, s.rank:], qkv[:, self.q_size:], self.per_head, s.head_dim, s.rot_dim, s.n_heads, n)
            ops.attention(qkv, att, s.n_heads, s.n_heads, self.per_head, s.scale, None, batch, None, from_step=True, ws=ws,
                          v_dim=s.v_head_dim, sink=self.sink, exact_weights=True, row=qkv.shape[1])
        else:
            q_lat = ws.get("latent_q", (n, s.n_heads * self.row), dt)
            ops.latent_prep(proj, self.down_at, s.n_heads, s.head_dim, s.rot_dim, s.rank, rot_dims, self.down_norm,
                            s.norm_eps, self.cos, self.sin, q_lat, self.row, s.rank, False,
                            kv if cache.owns_storage else None, batch, interleaved=self.interleaved)
            ops.head_product(proj, self.per_head, self.uk_t, q_lat, self.row, n)
            mixed = ws.get("latent_mixed", (n, s.n_heads * s.rank), dt)
            ops.attention_values_in_keys(q_lat, mixed, s.n_heads, self.row, s.rank, s.scale, batch, kv, self.sink, ws)
            # (head h's output times sigmoid(g_h . x) where the values leave the latent space)
            ops.head_product(mixed, s.rank, self.uv, att, s.v_head_dim, n, gate=proj[:, self.gate_at:] if s.head_gate else None)
            gated = True
        if s.head_gate and not gated:  # head h's output times sigmoid(g_h . x)
            ops.gate_heads(att, proj[:, self.gate_at:], s.n_heads, s.v_head_dim, n)
        self.o_proj.forward(att, out, n)
        return out
