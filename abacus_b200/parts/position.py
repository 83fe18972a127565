"""Rotary position encoding: the table of angles (src/model.c:116-124).

A position encoding of the rotary family gives the attention mixer
  tables(n_positions, device) -> (cos, sin), float32 [n_positions, rotary_dim / 2]
  rotary_dim, interleaved
and the q/k preparation kernel applies them. The angles are made on the host
in float32 with abacus's own expression, pos * (1 / theta^(2i / rotary_dim)).
"""
import math

import numpy as np
import torch

from .base import POSITIONS


@POSITIONS.register("rotary")
class Rotary:
    def __init__(self, spec):
        if spec.pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing {spec.pairing!r} is neither half nor interleaved")
        if spec.rotary_dim < 2 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even")
        if (getattr(spec, "linear_factor", 1.0) != 1.0 or getattr(spec, "blend", None)) and not spec.exact_angles:
            raise ValueError("scaled frequencies are made with exact_angles")
        self.spec = spec
        self.rotary_dim = spec.rotary_dim
        self.interleaved = spec.pairing == "interleaved"
        self._tables = {}

    def frequencies(self):
        """(the pairs' frequencies float64 [rotary_dim / 2], the factor on cosines and sines) with the spec's scaling."""
        s, dims = self.spec, self.rotary_dim
        i = np.arange(dims // 2, dtype=np.float64)
        freq = np.power(float(s.theta), -2.0 * i / dims) / float(getattr(s, "linear_factor", 1.0))
        blend = getattr(s, "blend", None)
        if blend is None:
            return freq, 1.0
        factor, original, fast, slow = (float(v) for v in blend)

        def where(turns):  # the pair that makes `turns` turns over the original context
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(s.theta)))
        lo, hi = max(math.floor(where(fast)), 0), min(math.ceil(where(slow)), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0

    def tables(self, n_positions, device):
        key = str(device)
        have = self._tables.get(key)
        if have is None or have[0].shape[0] < n_positions:
            half = self.rotary_dim // 2
            if getattr(self.spec, "exact_angles", False):  # position * theta^(-2i / rotary_dim) in float64
                freq, amplitude = self.frequencies()
                angle = np.arange(n_positions, dtype=np.float64)[:, None] * freq[None, :]
                have = (torch.from_numpy((np.cos(angle) * amplitude).astype(np.float32)).to(device),
                        torch.from_numpy((np.sin(angle) * amplitude).astype(np.float32)).to(device))
                self._tables[key] = have
                return have
            i = np.arange(half, dtype=np.float32)
            inv = np.float32(1.0) / np.power(np.float32(self.spec.theta),
                                             (np.float32(2.0) * i) / np.float32(self.rotary_dim), dtype=np.float32)
            angle = (np.arange(n_positions, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
            have = (torch.from_numpy(np.cos(angle, dtype=np.float32)).to(device),
                    torch.from_numpy(np.sin(angle, dtype=np.float32)).to(device))
            self._tables[key] = have
        return have
