"""A mixer made of two mixers that read the same input (config.specs.SideBySideSpec):
    out = share * (norm(left(x); w_left) + norm(right(x); w_right))
each side's output normed over the model's width with a plain weight of its own before the two are joined.

The sides are mixers of the registry, whatever their kinds; each keeps what it keeps (keys and values, states) under
its own names: the entry's cache need is the two sides' needs together, the states' names prefixed "left." and
"right.". At most one side may keep keys and values (an entry has one set of pages).
"""
import torch

from ..cache.kv import EntryView
from ..cache.need import CacheNeed
from ..kernels import ops
from .base import MIXERS, to_device


def _side_view(cache, prefix, with_kv):
    states = {name[len(prefix):]: t for name, t in (cache.states or {}).items() if name.startswith(prefix)}
    return EntryView(cache.owns_storage, cache.kv if with_kv else None, None, states)


@MIXERS.register("side_by_side")
class SideBySide:
    def __init__(self, spec):
        self.spec = spec
        self.left, self.right = MIXERS.build(spec.left), MIXERS.build(spec.right)
        self.needs = (self.left.cache_need(), self.right.cache_need())
        if sum(1 for need in self.needs if need.n_kv_heads > 0) > 1:
            raise ValueError("side by side: at most one side keeps keys and values")
        if any(need.state_shape for need in self.needs):
            raise ValueError("side by side: the sides name their states")
        self.capturable = bool(getattr(self.left, "capturable", False) and getattr(self.right, "capturable", False))
        prompts = [getattr(m, "capturable_prompts", True) for m in (self.left, self.right)]
        self.capturable_prompts = False if False in prompts else "from_start" if "from_start" in prompts else True

    def sides(self):
        return (("left", self.left), ("right", self.right))

    def param_shapes(self):
        shapes = {"left_out": (self.spec.hidden,), "right_out": (self.spec.hidden,)}
        for name, side in self.sides():
            shapes.update({f"{name}.{slot}": shape for slot, shape in side.param_shapes().items()})
        return shapes

    def bind(self, params, ctx):
        self.ctx = ctx
        for name, side in self.sides():
            side.bind({slot[len(name) + 1:]: t for slot, t in params.items() if slot.startswith(name + ".")}, ctx)
        self.left_out = to_device(params["left_out"], ctx, torch.float32)
        self.right_out = to_device(params["right_out"], ctx, torch.float32)

    def step_weights(self):
        own = [self.left_out, self.right_out]
        return own + [t for _, side in self.sides() for t in getattr(side, "step_weights", lambda: [])()]

    def step_plans(self):
        return [p for _, side in self.sides() for p in getattr(side, "step_plans", lambda: [])()]

    def prepare(self, max_positions, device):
        for _, side in self.sides():
            prepare = getattr(side, "prepare", None)
            if prepare:
                prepare(max_positions, device)

    def cache_need(self):
        with_kv = next((need for need in self.needs if need.n_kv_heads > 0), CacheNeed())
        states = tuple((f"{name}.{state}", shape, kind) for (name, _), need in zip(self.sides(), self.needs)
                       for state, shape, kind in need.states)
        return CacheNeed(n_kv_heads=with_kv.n_kv_heads, head_dim=with_kv.head_dim, window=with_kv.window,
                         v_head_dim=with_kv.v_head_dim, keep_first=with_kv.keep_first, states=states,
                         values_in_keys=with_kv.values_in_keys)

    def state_bytes(self):
        return sum(getattr(side, "state_bytes", lambda: 0)() for _, side in self.sides())

    def forward(self, xn, out, batch, cache, ws):
        n, d = batch.n_rows, self.spec.hidden
        a = ws.get("side_left", (n, d), torch.float32)
        b = ws.get("side_right", (n, d), torch.float32)
        for (name, side), need, y in zip(self.sides(), self.needs, (a, b)):
            side.forward(xn, y, batch, _side_view(cache, name + ".", need.n_kv_heads > 0), ws)
        ops.normed_pair(a, b, self.left_out, self.right_out, out, n, self.spec.norm_eps, self.spec.share)
        return out
