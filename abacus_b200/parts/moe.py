"""A feed-forward of routed experts (config.specs.RoutedMLPSpec): a router picks `top` of `experts` small
feed-forward layers for every token, an optional shared one runs for all.

The router's logits, the scores and the choice are float32. A pair is (token, k-th choice); the experts' products run
over pairs, and a token's pairs are summed in the order of k, so a token's result does not depend on what else is in
the step. The experts' matrices are kept stacked, [experts, out, in]. A handful of pairs (a decode step) runs each row
against the matrices of its own expert as they stream from memory (csrc/moe.cu); more than GROUPED_FROM pairs in
bfloat16 are sorted by expert, each expert's run padded to whole row tiles, and multiplied on the tensor cores
(csrc/gemm_grouped.cu).
"""
import torch

from ..kernels import ops
from .base import FEED_FORWARDS, to_device
from .linear import Linear

_ACTIVATIONS = {"relu_squared": ops.RELU_SQUARED, "silu_gated": ops.SILU_GATED}
# Up to which size of an expert's matrix a shared expert of the same size lies stacked behind the routed ones: small
# experts are bound by their launches, and the shared one then costs none of its own (width 1,024, experts of 768:
# 1.94 -> 1.76 ms a decode step of 8 rows); large ones by their bytes, and a product by expert reads the shared matrices
# once per row where the ordinary product reads them once (width 2,560, experts of 2,432: 6.13 -> 6.32 ms).
STACK_SHARED_UP_TO = 4 << 20
# From how many pairs on the rows are sorted by expert for the tensor cores: below, a pair's expert streams once for
# its one row, which is what a tile of 128 rows with one row in it would do with more set-up.
GROUPED_FROM = 64


@FEED_FORWARDS.register("routed_mlp")
class RoutedMLP:
    capturable = True  # its forward launches kernels only; the routing stays on the device

    def __init__(self, spec):
        s = self.spec = spec
        if not 1 <= s.top <= s.experts + s.identity:
            raise ValueError(f"top {s.top} of {s.experts + s.identity} experts")
        if s.score not in ("sigmoid", "softmax_chosen", "softmax_all", "table"):
            raise ValueError(f"router score {s.score!r} is none of sigmoid, softmax_chosen, softmax_all, table")
        self.by_table = s.score == "table"  # no router: a table names every token id's experts, each with weight 1 / top
        if self.by_table and (s.identity or s.correction or s.shared is not None or s.weight_on != "output" or s.vocab < 1):
            raise ValueError("experts picked by a table have their weight 1 / top on the outputs, a table of `vocab` rows "
                             "and neither a shared expert, experts that return their input nor a correction")
        if s.identity < 0 or (s.identity and s.weight_on != "output"):
            raise ValueError("experts that return their input go with the weight on the experts' outputs")
        if (s.correction or s.weight_scale != 1.0) and s.score != "softmax_all":
            raise ValueError("a correction of the choice and a scale of the weights go with the score softmax_all")
        if s.top > s.experts + s.identity:
            raise ValueError(f"top {s.top} of {s.experts + s.identity} router outputs")
        # the weight applied in float32 where a token's pairs are summed (else on the row that enters the last product)
        self.weighted_sum = s.weight_on == "output" and (s.identity > 0 or s.score in ("softmax_all", "table"))
        if self.weighted_sum and s.shared is not None:
            raise ValueError("a shared expert beside weights on the outputs is not built")
        self.gated = s.expert.activation == "silu_gated"
        if s.weight_on not in ("input", "output"):
            raise ValueError(f"weight_on {s.weight_on!r} is neither input nor output")
        for e in (s.expert, s.shared):
            if e is not None and e.activation not in _ACTIVATIONS:
                raise ValueError(f"expert activation {e.activation!r} is not built (relu_squared, silu_gated)")
        if s.shared is not None and s.shared.activation != "relu_squared":
            raise ValueError("a shared expert is built with relu_squared only")

    def param_shapes(self):
        s = self.spec
        shapes = {"table": (s.vocab, s.top)} if self.by_table else {"router": (s.experts + s.identity, s.hidden)}
        if s.correction:
            shapes["correction"] = (s.experts + s.identity,)
        for e in range(s.experts):
            if self.gated:
                shapes[f"gate{e}"] = (s.expert.inter, s.hidden)
            shapes[f"up{e}"] = (s.expert.inter, s.hidden)
            shapes[f"down{e}"] = (s.hidden, s.expert.inter)
        if s.shared is not None:
            shapes.update(shared_up=(s.shared.inter, s.hidden), shared_down=(s.hidden, s.shared.inter))
        return shapes

    def bind(self, params, ctx):
        s, self.ctx = self.spec, ctx
        self.router = None if self.by_table else to_device(params["router"], ctx, torch.float32)
        self.table = to_device(params["table"], ctx, torch.int32) if self.by_table else None
        self.correction = to_device(params["correction"], ctx, torch.float32) if s.correction else None
        ups, downs = [params[f"up{e}"] for e in range(s.experts)], [params[f"down{e}"] for e in range(s.experts)]
        if self.gated:  # an expert's first matrix: its gate rows, then its up rows
            ups = [torch.cat([params[f"gate{e}"], up], dim=0) for e, up in enumerate(ups)]
        # a shared expert of the routed experts' own size and activation lies stacked behind them, and every token has
        # one more pair: that expert, with weight 1 (no launches of its own; in a prompt it rides the grouped product)
        self.stacked_shared = (s.shared is not None and s.shared.inter == s.expert.inter
                               and s.shared.activation == s.expert.activation and s.weight_on == "input"
                               and s.expert.inter * s.hidden * ups[0].element_size() <= STACK_SHARED_UP_TO)
        if self.stacked_shared:
            ups, downs = ups + [params["shared_up"]], downs + [params["shared_down"]]
        self.up = to_device(torch.stack(ups), ctx, ctx.dtype)
        self.down = to_device(torch.stack(downs), ctx, ctx.dtype)
        self.shared_up = self.shared_down = None
        if s.shared is not None and not self.stacked_shared:
            self.shared_up = Linear(to_device(params["shared_up"], ctx, ctx.dtype))
            self.shared_down = Linear(to_device(params["shared_down"], ctx, ctx.dtype))

    def step_weights(self):
        # of the experts a step reads only those its tokens chose; the router and the shared expert it reads whole
        if self.stacked_shared:
            return [self.router, self.up[self.spec.experts], self.down[self.spec.experts]]
        shared = [self.shared_up.weight, self.shared_down.weight] if self.shared_up is not None else []
        return [self.router, self.correction, *shared]

    def forward(self, xn, out, batch, ws):
        s, n, dt = self.spec, batch.n_rows, self.ctx.dtype
        top = s.top + (1 if self.stacked_shared else 0)   # pairs a token has
        n_experts = s.experts + (1 if self.stacked_shared else 0)
        pairs = n * top
        expert = ws.get("moe_expert", (pairs,), torch.int32)
        weight = ws.get("moe_weight", (pairs,), torch.float32)
        if self.by_table:
            ops.moe_table(batch, self.table, s.experts, s.top, expert, weight, ops.kernel_status(self.ctx.device)[:1])
        else:
            ops.moe_route(xn, self.router, s.top, batch, expert, weight, softmax_chosen=s.score == "softmax_chosen",
                          always=s.experts if self.stacked_shared else None, softmax_all=s.score == "softmax_all",
                          correction=self.correction, weight_scale=s.weight_scale, n_real=s.experts)
        on_input = s.weight_on == "input"
        if self.weighted_sum:
            return self.forward_weighted_sum(xn, out, expert, weight, n, pairs, ws)
        if self.shared_up is not None:
            shared_act = ws.get("moe_shared_act", (n, s.shared.inter), dt)
            self.shared_up.forward(xn, shared_act, n)
            ops.relu_squared(shared_act, n)
            self.shared_down.forward(shared_act, out, n)
        if pairs > GROUPED_FROM and on_input and ops.grouped_takes(xn, self.up, self.down):
            tiles = ops.grouped_tiles(pairs, n_experts)
            rows = tiles * ops.GROUPED_ROWS
            scratch = ws.get("moe_sort", (2 * n_experts + pairs,), torch.int32)
            place = ws.get("moe_place", (pairs,), torch.int32)
            tile_expert = ws.get("moe_tile_expert", (tiles,), torch.int32)
            sorted_rows = ws.get("moe_sorted", (rows, s.hidden), dt)
            ops.moe_sort(xn, top, expert, weight, pairs, n_experts, scratch, place, tile_expert, sorted_rows)
            act = ws.get("moe_act", (rows, s.expert.inter), dt)
            ops.gemm_grouped(sorted_rows, self.up, act, tile_expert, activation=_ACTIVATIONS[s.expert.activation])
            sorted_out = ws.get("moe_pair_out", (rows, s.hidden), torch.float32)
            ops.gemm_grouped(act, self.down, sorted_out, tile_expert)
            ops.moe_unsort(sorted_out, place, out, n, top, add=self.shared_up is not None)
            return out
        act = ws.get("moe_act", (pairs, s.expert.inter), dt)
        ops.routed_product(xn, top, self.up, expert, weight if on_input else None, act, pairs,
                           activation=_ACTIVATIONS[s.expert.activation])
        pair_out = ws.get("moe_pair_out", (pairs, s.hidden), torch.float32)
        ops.routed_product(act, 1, self.down, expert, None if on_input else weight, pair_out, pairs)
        ops.moe_combine(pair_out, out, n, top, add=self.shared_up is not None)
        return out

    def forward_weighted_sum(self, xn, out, expert, weight, n, pairs, ws):
        """The experts' outputs, unweighted, then out[t] = sum_k weight[t, k] * (output of the k-th choice, or the token's
        own row where the choice returns its input), in float32."""
        s, dt = self.spec, self.ctx.dtype
        if pairs > GROUPED_FROM and ops.grouped_takes(xn, self.up, self.down) and s.expert.inter % 8 == 0:
            # many rows: sorted by expert for the tensor cores (pairs that return their input have no place there); a
            # gated expert's first product leaves gate and up side by side, as stored tensors, then the activation
            tiles = ops.grouped_tiles(pairs, s.experts)
            rows = tiles * ops.GROUPED_ROWS
            scratch = ws.get("moe_sort", (2 * s.experts + pairs,), torch.int32)
            place = ws.get("moe_place", (pairs,), torch.int32)
            tile_expert = ws.get("moe_tile_expert", (tiles,), torch.int32)
            sorted_rows = ws.get("moe_sorted", (rows, s.hidden), dt)
            ops.moe_sort(xn, s.top, expert, None, pairs, s.experts, scratch, place, tile_expert, sorted_rows)
            act = ws.get("moe_act", (rows, s.expert.inter), dt)
            if self.gated:
                gate_up = ws.get("moe_gate_up", (rows, 2 * s.expert.inter), dt)
                ops.gemm_grouped(sorted_rows, self.up, gate_up, tile_expert)
                ops.swiglu(gate_up, act)
            else:
                ops.gemm_grouped(sorted_rows, self.up, act, tile_expert, activation=_ACTIVATIONS[s.expert.activation])
            sorted_out = ws.get("moe_pair_out", (rows, s.hidden), torch.float32)
            ops.gemm_grouped(act, self.down, sorted_out, tile_expert)
            ops.moe_combine_weighted(sorted_out, weight, expert, xn, out, n, s.top, place=place)
            return out
        act = ws.get("moe_act", (pairs, s.expert.inter), dt)
        ops.routed_product(xn, s.top, self.up, expert, None, act, pairs, activation=_ACTIVATIONS[s.expert.activation])
        pair_out = ws.get("moe_pair_out", (pairs, s.hidden), torch.float32)
        ops.routed_product(act, 1, self.down, expert, None, pair_out, pairs)
        ops.moe_combine_weighted(pair_out, weight, expert, xn, out, n, s.top)
        return out
