"""Linonex on the GPU against the plain implementation (tests/plain/linonex_plain.py): every mechanism alone as the
part the model uses (whole, in portions, token by token, in unequal batches, in slots used before), keys at the edges
of chunks and pages, then whole models through the engine: prompts, decoding, batches, captured graphs, greedy
generation through the library's entry point, and the trace replay."""
import numpy as np
import pytest
import torch

import linonex_models as lm
from helpers import TraceRun, assert_logits
from plain import linonex_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _rnd(dtype):
    return lm.bf16_round if dtype == "bfloat16" else (lambda a: np.asarray(a, dtype=np.float32))


def _close(got, want, dtype, what, f32=2e-4, bf16=0.1):
    """float32: within a fraction of the largest value (sums taken in another order). bfloat16 (projections and
    activations rounded where the plain implementation rounds nothing): single values within a tenth of the largest, and
    the whole within 3 % in the root mean square."""
    want = np.asarray(want, dtype=np.float64)
    assert np.isfinite(got).all(), f"{what}: not finite"
    limit = (f32 if dtype == "float32" else bf16) * max(np.abs(want).max(), 1e-3)
    diff = np.abs(got - want)
    assert diff.max() <= limit, f"{what}: off by {diff.max():.3g} at row {int(diff.max(-1).argmax())} (limit {limit:.3g})"
    if dtype == "bfloat16" and want.size >= 64:
        rel = np.sqrt((diff ** 2).mean() / max((want ** 2).mean(), 1e-12))
        assert rel <= 0.03, f"{what}: {rel:.3g} of the root mean square away"


class PartRun:
    """A mixer or a feed-forward of the registry alone: bound to given tensors, with a cache of its own, stepped with
    given rows."""

    def __init__(self, spec, params, dtype, feed_forward=False):
        from abacus_b200.cache import SequenceCache
        from abacus_b200.parts import FEED_FORWARDS, MIXERS, BuildContext, Workspace
        self.dtype, self.feed_forward = dtype, feed_forward
        self.part = (FEED_FORWARDS if feed_forward else MIXERS).build(spec)
        assert set(self.part.param_shapes()) == set(params), set(self.part.param_shapes()) ^ set(params)
        device = torch.device(DEV, torch.cuda.current_device())
        self.part.bind({n: torch.from_numpy(np.ascontiguousarray(t, dtype=np.float32)) for n, t in params.items()},
                       BuildContext(device=device, dtype=DT[dtype]))
        self.ws = Workspace(device)
        self.cache = None
        if not feed_forward:
            self.cache = SequenceCache([self.part.cache_need()], [None], 64 * 48, DT[dtype], DEV)
            prepare = getattr(self.part, "prepare", None)
            if prepare:
                prepare(4096, device)
        self.length = {}

    def open(self, dirty=False):
        """A slot; dirty: what a former user left in its states stays there until the slot is opened again."""
        slot = self.cache.open_slot()
        if dirty:
            for state in self.cache._all_states():
                state[slot].fill_(3.0)
            self.cache.close_slot(slot)
            again = self.cache.open_slot()
            assert again == slot
        self.length[slot] = 0
        return slot

    def step(self, entries):
        """entries: [(slot or None, rows [n, d])] -> [out [n, d]] float32."""
        from abacus_b200.engine.batch import Sequence, StepBatch
        plans = getattr(self.part, "step_plans", lambda: [])()
        n = sum(len(h) for _, h in entries)
        seqs = []
        for i, (slot, h) in enumerate(entries):
            start = self.length.get(slot, 0)
            if self.cache is not None:
                self.cache.reserve(slot, start + len(h))
                self.length[slot] = start + len(h)
            seqs.append(Sequence(slot if slot is not None else i, [0] * len(h), start, []))
        batch = StepBatch(n, len(entries), 1, DEV, plans=plans).fill(seqs, exact=True)
        xn = torch.from_numpy(np.concatenate([np.asarray(h, dtype=np.float32) for _, h in entries])).to(DEV).to(DT[self.dtype])
        out = torch.full((n, xn.shape[1]), 7.0, dtype=torch.float32, device=DEV)
        if self.feed_forward:
            self.part.forward(xn.contiguous(), out, batch, self.ws)
        else:
            self.part.forward(xn.contiguous(), out, batch, self.cache.views[0], self.ws)
        torch.cuda.synchronize()
        got, at = out.cpu().numpy(), 0
        outs = []
        for _, h in entries:
            outs.append(got[at:at + len(h)])
            at += len(h)
        return outs


def _every_way(run, h, want, dtype, what, portions=(60, 2, 7, 1, 64, 16)):
    """The rows h of one sequence: whole, in portions down to two tokens and one, token by token, and in an unequal batch
    in slots that were used before; all against `want`."""
    T = len(h)
    slot = run.open()
    _close(run.step([(slot, h)])[0], want, dtype, f"{what}, whole")
    run.cache.close_slot(slot)
    slot, at, got = run.open(dirty=True), 0, []
    for size in portions:
        got.append(run.step([(slot, h[at:at + size])])[0])
        at += size
    assert at == T
    _close(np.concatenate(got), want, dtype, f"{what}, in portions")
    run.cache.close_slot(slot)
    slot = run.open(dirty=True)
    got = np.concatenate([run.step([(slot, h[t:t + 1])])[0] for t in range(40)])
    _close(got, want[:40], dtype, f"{what}, token by token")
    run.cache.close_slot(slot)
    # three sequences of the same rows: 120 of them, a single one, 70; then decoded together
    a, b, c = run.open(dirty=True), run.open(dirty=True), run.open(dirty=True)
    first = run.step([(a, h[:120]), (b, h[:1]), (c, h[:70])])
    for got, n in zip(first, (120, 1, 70)):
        _close(got, want[:n], dtype, f"{what}, unequal batch, {n} rows")
    for t in range(5):
        nxt = run.step([(a, h[120 + t:121 + t]), (b, h[1 + t:2 + t]), (c, h[70 + t:71 + t])])
        for got, at in zip(nxt, (120 + t, 1 + t, 70 + t)):
            _close(got, want[at:at + 1], dtype, f"{what}, decoded together at {at}", f32=5e-4)
    for s in (a, b, c):
        run.cache.close_slot(s)


def _memory(rng, d, H, K, V, rnd):
    p = {"q": rng.standard_normal((H * K, d)) * 2 / np.sqrt(d), "k": rng.standard_normal((H * K, d)) * 2 / np.sqrt(d),
         "v": rng.standard_normal((H * V, d)) / np.sqrt(d), "g": rng.standard_normal((H * V, d)) / np.sqrt(d),
         "i": rng.standard_normal((H, d)) * 3 / np.sqrt(d), "f": rng.standard_normal((H, d)) * 3 / np.sqrt(d),
         "i.b": rng.standard_normal(H), "f.b": 2.0 + rng.standard_normal(H) * 1.5, "norm": 1 + rng.standard_normal(H * V) * 0.1,
         "o": rng.standard_normal((d, H * V)) / np.sqrt(H * V)}
    return {n: rnd(t) for n, t in p.items()}


_MEMORY_SLOTS = {"wq": "q", "wk": "k", "wv": "v", "wg": "g", "wi": "i", "bi": "i.b", "wf": "f", "bf": "f.b",
                 "out_norm": "norm", "wo": "o"}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,K,V,cap", [(2, 5, 3, 6.0), (3, 16, 8, 15.0), (1, 40, 24, 10.0), (2, 128, 70, 12.0), (1, 200, 133, 4.0)])
def test_the_matrix_memory_every_way(dtype, H, K, V, cap):
    from abacus_b200.config.specs import MatrixMemorySpec
    rng, rnd, d = np.random.default_rng(K), _rnd(dtype), 40
    p = _memory(rng, d, H, K, V, rnd)
    h = rnd(rng.standard_normal((150, d)))
    want, _ = plain.matrix_memory(h.astype(np.float64), {n: t.astype(np.float64) for n, t in p.items()},
                                  {"heads": H, "dim": K, "vdim": V, "gate_cap": cap}, 1e-5, None)
    run = PartRun(MatrixMemorySpec(hidden=d, n_heads=H, key_dim=K, value_dim=V, gate_cap=cap, norm_eps=1e-5),
                  {slot: p[name] for slot, name in _MEMORY_SLOTS.items()}, dtype)
    _every_way(run, h, want, dtype, f"matrix memory {H}x{K}x{V}")


def test_the_matrix_memory_keeps_a_token_over_a_long_decoding():
    """Forget gates near one and a single loud input gate early on: 400 tokens later, one by one, the memory still
    answers with that token's value; the running maximum has moved by hundreds meanwhile."""
    from abacus_b200.config.specs import MatrixMemorySpec
    rng, d, H, K, V = np.random.default_rng(1), 16, 2, 8, 8
    p = _memory(rng, d, H, K, V, _rnd("float32"))
    p["f"] *= 0.0
    p["f.b"] = np.full(H, 9.0, dtype=np.float32)
    p["i.b"] = np.full(H, -6.0, dtype=np.float32)
    h = rng.standard_normal((440, d)).astype(np.float32)
    h[3] += 4.0 * p["i"][0] / np.linalg.norm(p["i"][0])  # token 3 opens head 0's input gate wide
    want, _ = plain.matrix_memory(h.astype(np.float64), {n: t.astype(np.float64) for n, t in p.items()},
                                  {"heads": H, "dim": K, "vdim": V, "gate_cap": 14.0}, 1e-5, None)
    run = PartRun(MatrixMemorySpec(hidden=d, n_heads=H, key_dim=K, value_dim=V, gate_cap=14.0, norm_eps=1e-5),
                  {slot: p[name] for slot, name in _MEMORY_SLOTS.items()}, "float32")
    slot = run.open(dirty=True)
    got = [run.step([(slot, h[:40])])[0]] + [run.step([(slot, h[t:t + 1])])[0] for t in range(40, 440)]
    _close(np.concatenate(got), want, "float32", "long decoding", f32=1e-3)


def _delta(rng, d, H, G, K, V, taps, rnd):
    s = 1 / np.sqrt(d)
    p = {"q": rng.standard_normal((G * K, d)) * 2 * s, "k": rng.standard_normal((G * K, d)) * 2 * s,
         "v": rng.standard_normal((H * V, d)) * s, "q.conv": rng.standard_normal((G * K, taps)) * 0.6,
         "k.conv": rng.standard_normal((G * K, taps)) * 0.6, "v.conv": rng.standard_normal((H * V, taps)) * 0.6,
         "b": rng.standard_normal((H, d)) * 2 * s, "a": rng.standard_normal((H, d)) * 2 * s,
         "A_log": -1.0 + rng.standard_normal(H), "dt_bias": rng.standard_normal(H), "g": rng.standard_normal((H * V, d)) * s,
         "norm": 1 + rng.standard_normal(V) * 0.1, "o": rng.standard_normal((d, H * V)) / np.sqrt(H * V)}
    return {n: rnd(t) for n, t in p.items()}


_DELTA_SLOTS = {"wq": "q", "wk": "k", "wv": "v", "conv_q": "q.conv", "conv_k": "k.conv", "conv_v": "v.conv", "wb": "b",
                "wa": "a", "decay_log": "A_log", "decay_bias": "dt_bias", "wg": "g", "out_norm": "norm", "wo": "o"}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,K,V,taps", [(2, 2, 5, 3, 2), (4, 2, 8, 16, 3), (2, 1, 20, 6, 1), (3, 3, 64, 40, 4), (1, 1, 128, 8, 5)])
def test_the_delta_rule_with_a_decay_per_head_every_way(dtype, H, G, K, V, taps):
    from abacus_b200.config.specs import HeadDeltaSpec
    rng, rnd, d = np.random.default_rng(K + taps), _rnd(dtype), 48
    p = _delta(rng, d, H, G, K, V, taps, rnd)
    h = rnd(rng.standard_normal((150, d)))
    want, _ = plain.scalar_delta_rule(h.astype(np.float64), {n: t.astype(np.float64) for n, t in p.items()},
                                      {"heads": H, "kv_heads": G, "dim": K, "vdim": V}, 1e-6, None)
    run = PartRun(HeadDeltaSpec(hidden=d, n_heads=H, n_kv_heads=G, key_dim=K, value_dim=V, conv_taps=taps, norm_eps=1e-6),
                  {slot: p[name] for slot, name in _DELTA_SLOTS.items()}, dtype)
    _every_way(run, h, want, dtype, f"delta rule {H}/{G}x{K}x{V}, {taps} taps", portions=(60, 2, 7, 1, 64, 16))


def test_the_delta_rule_in_many_chunks_with_decays_from_nothing_to_one():
    """520 tokens (eight chunks and a ragged one), heads whose decay is all but 1, all but 0 (below what float32 holds
    over a chunk) and in between, write strengths near 1: whole, and continued from a state in portions that end inside
    chunks; against the plain recurrence."""
    from abacus_b200.config.specs import HeadDeltaSpec
    rng, d, H, G, K, V, taps = np.random.default_rng(8), 32, 4, 2, 24, 20, 3
    p = _delta(rng, d, H, G, K, V, taps, _rnd("float32"))
    p["A_log"] = np.array([-9.0, 5.0, 0.0, 2.0], dtype=np.float32)
    p["dt_bias"] = np.array([-2.0, 3.0, 0.0, 1.0], dtype=np.float32)
    p["b"] = (p["b"] * 0).astype(np.float32)
    p["b"][:, 0] = 3.0
    h = rng.standard_normal((520, d)).astype(np.float32)
    h[:, 0] = 1.0 + 0.2 * rng.standard_normal(520)  # b = sigmoid(about 3)
    want, _ = plain.scalar_delta_rule(h.astype(np.float64), {n: t.astype(np.float64) for n, t in p.items()},
                                      {"heads": H, "kv_heads": G, "dim": K, "vdim": V}, 1e-6, None)
    run = PartRun(HeadDeltaSpec(hidden=d, n_heads=H, n_kv_heads=G, key_dim=K, value_dim=V, conv_taps=taps, norm_eps=1e-6),
                  {slot: p[name] for slot, name in _DELTA_SLOTS.items()}, "float32")
    slot = run.open(dirty=True)
    _close(run.step([(slot, h)])[0], want, "float32", "delta rule, 520 tokens whole", f32=5e-4)
    run.cache.close_slot(slot)
    slot, at, got = run.open(dirty=True), 0, []
    for size in (100, 1, 200, 33, 186):
        got.append(run.step([(slot, h[at:at + size])])[0])
        at += size
    _close(np.concatenate(got), want, "float32", "delta rule, 520 tokens in portions", f32=5e-4)


def test_the_matrix_memory_in_many_chunks():
    """520 tokens with gates that swing between closed and wide open, whole and in portions that end inside chunks."""
    from abacus_b200.config.specs import MatrixMemorySpec
    rng, d, H, K, V = np.random.default_rng(12), 32, 3, 20, 36
    p = _memory(rng, d, H, K, V, _rnd("float32"))
    p["i"], p["f"] = (p["i"] * 4).astype(np.float32), (p["f"] * 4).astype(np.float32)
    h = rng.standard_normal((520, d)).astype(np.float32)
    want, _ = plain.matrix_memory(h.astype(np.float64), {n: t.astype(np.float64) for n, t in p.items()},
                                  {"heads": H, "dim": K, "vdim": V, "gate_cap": 15.0}, 1e-5, None)
    run = PartRun(MatrixMemorySpec(hidden=d, n_heads=H, key_dim=K, value_dim=V, gate_cap=15.0, norm_eps=1e-5),
                  {slot: p[name] for slot, name in _MEMORY_SLOTS.items()}, "float32")
    slot = run.open(dirty=True)
    _close(run.step([(slot, h)])[0], want, "float32", "matrix memory, 520 tokens whole", f32=5e-4)
    run.cache.close_slot(slot)
    slot, at, got = run.open(dirty=True), 0, []
    for size in (100, 1, 200, 33, 186):
        got.append(run.step([(slot, h[at:at + size])])[0])
        at += size
    _close(np.concatenate(got), want, "float32", "matrix memory, 520 tokens in portions", f32=5e-4)


def _attention_spec(d, H, G, K, V, scale, taps, chunk, cap):
    from abacus_b200.config.specs import AttentionSpec
    return AttentionSpec(hidden=d, n_heads=H, n_kv_heads=G, head_dim=K, scale=scale, qk_norm_eps=None, position=None,
                         v_head_dim=V, exact_weights=True, conv_taps=taps, chunk=chunk, softcap=cap)


_LEFT_SLOTS = {"wq": "q", "wk": "k", "wv": "v", "conv_q": "q.conv", "conv_k": "k.conv", "conv_v": "v.conv", "wo": "o"}


def _attention_params(p, taps):
    return {slot: p[name] for slot, name in _LEFT_SLOTS.items() if taps or not slot.startswith("conv")}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,K,V,taps,chunk,cap", [(4, 2, 16, 8, 2, 48, 20.0), (3, 3, 10, 7, 4, 7, 5.0), (6, 1, 8, 8, 0, None, None),
                                                     (2, 1, 32, 16, 5, 64, None), (1, 1, 24, 40, 3, None, 9.0), (2, 2, 64, 64, 1, 1, 30.0)])
def test_attention_with_a_convolution_chunks_and_a_cap_every_way(dtype, H, G, K, V, taps, chunk, cap):
    rng, rnd, d = np.random.default_rng(K + (chunk or 0)), _rnd(dtype), 40
    s = 1 / np.sqrt(d)
    p = {"q": rng.standard_normal((H * K, d)) * 3 * s, "k": rng.standard_normal((G * K, d)) * 3 * s,
         "v": rng.standard_normal((G * V, d)) * s, "o": rng.standard_normal((d, H * V)) / np.sqrt(H * V)}
    for t, rows in (("q", H * K), ("k", G * K), ("v", G * V)):
        p[t + ".conv"] = rng.standard_normal((rows, max(taps, 1))) * 0.6 if taps else np.ones((rows, 1))
    p = {n: rnd(t) for n, t in p.items()}
    h = rnd(rng.standard_normal((150, d)))
    m = {"heads": H, "kv_heads": G, "dim": K, "vdim": V, "mask": {"size": chunk or 10 ** 6}, "softcap": cap or 1e9, "scale": 0.3}
    want, _ = plain.chunked_attention(h.astype(np.float64), {n: t.astype(np.float64) for n, t in p.items()}, m, None)
    run = PartRun(_attention_spec(d, H, G, K, V, 0.3, taps, chunk, cap), _attention_params(p, taps), dtype)
    run.cache.views[0].kv.k.fill_(9.0), run.cache.views[0].kv.v.fill_(9.0)  # what former users left in the pages
    _every_way(run, h, want, dtype, f"attention {H}/{G}x{K}x{V}, {taps} taps, chunks of {chunk}, cap {cap}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [48, 64, 130, 200])
def test_one_loud_key_at_the_edges_of_chunks_and_pages(chunk, dtype):
    """Queries read one part of the input row, keys another, values a third, so a key can be made loud for one query
    alone: the first and the last key of the query's chunk, the last key of the chunk before (which must not count), keys
    on both sides of a page's border, the far end of a long chunk; in a prompt and for tokens that come one by one. In
    bfloat16 whole prompts run on the tensor-core kernel, whose tiles of 64 keys have edges of their own."""
    rng, K, V, T = np.random.default_rng(chunk), 8, 8, 210
    d = 2 * K + V
    p = {"q": np.eye(d)[:K], "k": np.eye(d)[K:2 * K], "v": np.eye(d)[2 * K:], "o": np.eye(d)[:, :V],
         "q.conv": np.tile([0.0, 1.0], (K, 1)), "k.conv": np.tile([0.0, 1.0], (K, 1)), "v.conv": np.tile([0.0, 1.0], (V, 1))}
    m = {"heads": 1, "kv_heads": 1, "dim": K, "vdim": V, "mask": {"size": chunk}, "softcap": 25.0, "scale": 1.0}
    u = rng.standard_normal(K)
    u /= np.linalg.norm(u)
    pairs = []  # (query position, key position)
    for i in (chunk - 1, chunk, chunk + 1, 2 * chunk - 1, 63, 64, 65, 128, T - 1):
        if i >= T:
            continue
        first = i // chunk * chunk
        pairs += [(i, first), (i, i), (i, max(first - 1, 0)), (i, max(i - 1, 0)), (i, min(first + 63, i)), (i, min(first + 64, i))]
    run = PartRun(_attention_spec(d, 1, 1, K, V, 1.0, 2, chunk, 25.0),
                  _attention_params({n: t.astype(np.float32) for n, t in p.items()}, 2), dtype)
    for i, j in sorted(set(pairs)):
        h = rng.standard_normal((T, d)) * 0.2
        h[i, :K] = 6.0 * u
        h[j, K:2 * K] = 6.0 * u
        h = _rnd(dtype)(h)
        want, _ = plain.chunked_attention(h.astype(np.float64), {n: t.astype(np.float64) for n, t in p.items()}, m, None)
        seen = j // chunk == i // chunk and j <= i
        if j != i:  # the loud key decides the answer if and only if it lies in the query's chunk
            assert (np.abs(want[i, :V] - h[j, 2 * K:]).max() < 0.05) == seen
        run.cache.views[0].kv.k.fill_(9.0), run.cache.views[0].kv.v.fill_(9.0)  # what former users left in the pages
        slot = run.open(dirty=True)
        _close(run.step([(slot, h[:i + 1])])[0], want[:i + 1], dtype, f"query {i}, loud key {j}, prompt")
        run.cache.close_slot(slot)
        # the prompt ends a few tokens before the query, or right before the key if that comes later
        slot, cut = run.open(dirty=True), max(1, i - 3 if j < i - 3 else j - 1)
        got = [run.step([(slot, h[:cut])])[0]] + [run.step([(slot, h[t:t + 1])])[0] for t in range(cut, i + 1)]
        _close(np.concatenate(got), want[:i + 1], dtype, f"query {i}, loud key {j}, decoded from {cut}")
        run.cache.close_slot(slot)


def _routed_spec(d, E, ident, top, scale, ff):
    from abacus_b200.config.specs import ExpertSpec, RoutedMLPSpec
    return RoutedMLPSpec(hidden=d, experts=E, top=top, expert=ExpertSpec(ff, "silu_gated"), shared=None, score="softmax_all",
                         weight_on="output", correction=True, weight_scale=scale, identity=ident)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,ident,top,d,ff", [(5, 1, 3, 64, 24), (1, 2, 3, 32, 8), (3, 0, 1, 48, 16), (20, 4, 6, 40, 9), (8, 3, 4, 128, 64)])
def test_routed_experts_with_weights_on_the_outputs(dtype, E, ident, top, d, ff):
    rng, rnd = np.random.default_rng(E), _rnd(dtype)
    p = {"router": rnd(rng.standard_normal((E + ident, d)) * 2 / np.sqrt(d)), "correction": rnd(rng.standard_normal(E + ident) * 0.3)}
    for e in range(E):
        p[f"e{e}.gate"], p[f"e{e}.up"] = rnd(rng.standard_normal((ff, d)) / np.sqrt(d)), rnd(rng.standard_normal((ff, d)) / np.sqrt(d))
        p[f"e{e}.down"] = rnd(rng.standard_normal((d, ff)) / np.sqrt(ff))
    params = {"router": p["router"], "correction": p["correction"]}
    for e in range(E):
        params.update({f"gate{e}": p[f"e{e}.gate"], f"up{e}": p[f"e{e}.up"], f"down{e}": p[f"e{e}.down"]})
    run = PartRun(_routed_spec(d, E, ident, top, 1.7, ff), params, dtype, feed_forward=True)
    mlp = {"router": {"experts": E, "identity": ident, "top": top, "scale": 1.7}, "expert": {"ff": ff}}
    for n in (1, 9, 70, 300):  # a decode step, a few rows, and enough pairs for the products sorted by expert
        h = rnd(rng.standard_normal((n, d)))
        z = h.astype(np.float64) @ p["router"].astype(np.float64).T
        s = np.exp(z - z.max(-1, keepdims=True))
        key = np.sort(s / s.sum(-1, keepdims=True) + p["correction"], axis=-1)[:, ::-1]
        clear = (key[:, top - 1] - key[:, min(top, E + ident - 1)] > 1e-4) | (top == E + ident)  # rows whose choice is no close call
        want = plain.routed_ff(h.astype(np.float64), {n_: t.astype(np.float64) for n_, t in p.items()}, mlp)
        got = run.step([(None, h)])[0]
        assert clear.mean() > 0.9
        _close(got[clear], want[clear], dtype, f"routed experts, {n} rows")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_mixers_side_by_side_every_way(dtype):
    from abacus_b200.config.specs import HeadDeltaSpec, SideBySideSpec
    rng, rnd, d = np.random.default_rng(5), _rnd(dtype), 48
    s = 1 / np.sqrt(d)
    a = {"q": rng.standard_normal((4 * 16, d)) * 3 * s, "k": rng.standard_normal((2 * 16, d)) * 3 * s,
         "v": rng.standard_normal((2 * 8, d)) * s, "o": rng.standard_normal((d, 4 * 8)) / np.sqrt(32), "out": 1 + rng.standard_normal(d) * 0.2}
    for t, rows in (("q", 64), ("k", 32), ("v", 16)):
        a[t + ".conv"] = rng.standard_normal((rows, 3)) * 0.6
    a = {n: rnd(t) for n, t in a.items()}
    b = _delta(rng, d, 4, 2, 8, 16, 2, rnd)
    b["out"] = rnd(1 + rng.standard_normal(d) * 0.2)
    p = {**{"left." + n: t for n, t in a.items()}, **{"right." + n: t for n, t in b.items()}}
    m = {"left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "mask": {"size": 33}, "softcap": 11.0, "scale": 0.25},
         "right": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 16}}
    h = rnd(rng.standard_normal((150, d)))
    want, _ = plain.side_by_side(h.astype(np.float64), {n: t.astype(np.float64) for n, t in p.items()}, m, 1e-5, None)
    spec = SideBySideSpec(hidden=d, left=_attention_spec(d, 4, 2, 16, 8, 0.25, 3, 33, 11.0),
                          right=HeadDeltaSpec(hidden=d, n_heads=4, n_kv_heads=2, key_dim=8, value_dim=16, conv_taps=2, norm_eps=1e-5),
                          norm_eps=1e-5, share=0.5)
    params = {"left_out": a["out"], "right_out": b["out"]}
    params.update({"left." + slot: a[name] for slot, name in _LEFT_SLOTS.items()})
    params.update({"right." + slot: b[name] for slot, name in _DELTA_SLOTS.items()})
    _every_way(PartRun(spec, params, dtype), h, want, dtype, "side by side")


# ------------------------------------------------------------------ whole models through the engine
def _engine(tmp, name, dtype, raw=None, seed=0, tensors=None, **kw):
    from abacus_b200.engine import Engine, load_model
    folder, raw, tensors = lm.write_folder(tmp, name, seed=seed, raw=raw, tensors=tensors)
    return Engine(load_model(folder, dtype), max_tokens=64 * 24, **kw), raw, tensors, folder


def _oracle(raw, tensors, tokens):
    """(the plain model's logits in float64, the noise float32 itself shows on them)."""
    want = plain.Plain(raw, tensors).feed(tokens)[0]
    return want, float(np.abs(want - plain.Plain(raw, tensors, real=np.float32).feed(tokens)[0]).max())


class Bf16Count:
    """bfloat16 against float64: the distance of two roundings of one model, a few per cent of the logits' spread (the
    test models' queries and keys are large, so that a wrong key shows; rounding them moves the weights by per cents). A
    rounded router input now and then chooses another expert where two choice scores nearly tie, and that position's
    logits then differ by much: such positions are counted, and few are allowed over a whole test."""

    def __init__(self):
        self.rows = self.far = 0

    def add(self, got, want, what):
        d = got - want
        d = d - d.mean(-1, keepdims=True)
        rel = np.sqrt((d * d).mean(-1)) / want.std()
        assert np.isfinite(got).all(), f"{what}: not finite"
        self.rows += len(rel)
        self.far += int((rel >= 0.25).sum())
        if len(rel) >= 20:
            assert np.median(rel) < 0.08, f"{what}: bfloat16 logits are {np.median(rel):.3g} of the spread away in the median"

    def settle(self, what):
        assert self.far <= 0.05 * self.rows, f"{what}: {self.far} of {self.rows} positions' bfloat16 logits are far away"


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("Q", "float32"), ("R", "float32"), ("P", "bfloat16"), ("R", "bfloat16")])
def test_prompts_decoding_batches_and_used_slots_against_the_plain_model(tmp_path, name, dtype):
    raw = lm.config(name)
    tensors = lm.weights(raw)
    if dtype == "bfloat16":  # routers that decide clearly, so that rounding their input seldom changes the choice
        tensors = {n: t * 4 if n.endswith("mlp.router") else t for n, t in tensors.items()}
    engine, raw, tensors, _ = _engine(tmp_path, name, dtype, raw=raw, tensors=tensors)
    rng = np.random.default_rng(7)
    lens = [150, 1, 37, 80]
    seqs = [[int(t) for t in rng.integers(0, raw["vocab"], n)] for n in lens]
    oracle = [_oracle(raw, tensors, s) for s in seqs]

    count = Bf16Count()

    def check(got, want, noise, what):
        if dtype == "float32":
            assert_logits(got, want, dtype, what, noise)
        else:
            count.add(got, want, what)
    # each alone, whole, all logits wanted; the slot is given back and used again by the next
    for s, (want, noise) in zip(seqs, oracle):
        slot = engine.open()
        got = engine.step([(slot, s, list(range(len(s))))]).cpu().numpy()
        engine.close(slot)
        check(got, want, noise, f"{name} whole, {len(s)} tokens")
    # together in one batch of unequal prompts, cut before their ends, then decoded together; early enders leave
    cut = [100, 1, 20, 64]
    slots = [engine.open() for _ in seqs]
    got = engine.step([(slot, s[:c], [c - 1]) for slot, s, c in zip(slots, seqs, cut)]).cpu().numpy()
    for i, (want, noise) in enumerate(oracle):
        check(got[i:i + 1], want[cut[i] - 1:cut[i]], noise, f"{name} batch prompt {i}")
    step = 0
    while True:
        live = [i for i in range(len(seqs)) if cut[i] + step < len(seqs[i])]
        for i in range(len(seqs)):
            if cut[i] + step == len(seqs[i]) and slots[i] is not None:
                engine.close(slots[i])
                slots[i] = None
        if not live:
            break
        got = engine.step([(slots[i], [seqs[i][cut[i] + step]], [0]) for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            check(got[j:j + 1], oracle[i][0][cut[i] + step:cut[i] + step + 1], oracle[i][1],
                  f"{name} batch decode, request {i}, position {cut[i] + step}")
        step += 1
    engine.check_status()
    count.settle(f"{name} {dtype}")


@pytest.mark.parametrize("name", ["P", "R"])
def test_portions_of_a_prompt_give_the_whole_prompts_logits(tmp_path, name):
    engine, raw, tensors, _ = _engine(tmp_path, name, "float32")
    rng = np.random.default_rng(5)
    tokens = [int(t) for t in rng.integers(0, raw["vocab"], 140)]
    want, noise = _oracle(raw, tensors, tokens)
    slot, got, at = engine.open(), [], 0
    for size in (60, 2, 7, 1, 64, 6):
        got.append(engine.step([(slot, tokens[at:at + size], list(range(size)))]).cpu().numpy())
        at += size
    engine.close(slot)
    assert at == len(tokens)
    assert_logits(np.concatenate(got), want, "float32", f"{name} in portions", noise)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_token_by_token_from_the_first_token_and_long_decoding(tmp_path, name):
    engine, raw, tensors, _ = _engine(tmp_path, name, "float32")
    rng = np.random.default_rng(3)
    tokens = [int(t) for t in rng.integers(0, raw["vocab"], 200)]
    want, noise = _oracle(raw, tensors, tokens)
    slot = engine.open()
    got = np.concatenate([engine.step([(slot, [t], [0])]).cpu().numpy() for t in tokens])
    engine.close(slot)
    assert_logits(got, want, "float32", f"{name} token by token", noise)


def test_a_far_token_decides_the_answer(tmp_path):
    """The same long prompts but for one early token: the last position's logits must follow the plain model's, which
    move (the recurrent states carry the token; the chunks of attention do not reach it)."""
    raw = lm.config("P")
    tensors = lm.weights(raw)
    for n in tensors:  # states that fade slowly: forget gates near one whatever the input, decays near one
        if n.endswith("mix.f"):
            tensors[n] = tensors[n] * 0
        elif n.endswith("mix.f.b"):
            tensors[n] = np.full_like(tensors[n], 8.0)
        elif n.endswith("A_log"):
            tensors[n] = np.full_like(tensors[n], -6.0)
        elif n.endswith("dt_bias"):
            tensors[n] = np.full_like(tensors[n], -3.0)
    engine, raw, tensors, _ = _engine(tmp_path, "P", "float32", raw=raw, tensors=tensors)
    rng = np.random.default_rng(9)
    tokens = [int(t) for t in rng.integers(0, raw["vocab"], 190)]
    other = list(tokens)
    other[3] = (tokens[3] + 1) % raw["vocab"]
    wants = [plain.Plain(raw, tensors).feed(t)[0][-1] for t in (tokens, other)]
    assert np.abs(wants[0] - wants[1]).max() > 0.1
    for t, want in zip((tokens, other), wants):
        slot = engine.open()
        engine.step([(slot, t[:130], [])])
        for tok in t[130:-1]:
            engine.step([(slot, [tok], [])])
        got = engine.step([(slot, t[-1:], [0])]).cpu().numpy()[0]
        engine.close(slot)
        assert np.abs(got - want).max() < 0.05 * np.abs(wants[0] - wants[1]).max() + 2e-4


def test_graphs_and_plain_launches_give_the_same_bits_and_states_survive_a_capture(tmp_path):
    from abacus_b200.engine import Engine
    engine, raw, tensors, _ = _engine(tmp_path, "P", "float32")
    eager = Engine(engine.model, max_tokens=64 * 24, use_graphs=False)
    rng = np.random.default_rng(11)
    seqs = [[int(t) for t in rng.integers(0, raw["vocab"], n)] for n in (30, 9)]
    outs = []
    for e in (engine, eager):
        slots = [e.open() for _ in seqs]
        got = [e.step([(slot, s[:5], [4]) for slot, s in zip(slots, seqs)]).cpu().numpy()]
        for i in range(5, 9):
            got.append(e.step([(slot, [s[i]], [0]) for slot, s in zip(slots, seqs)]).cpu().numpy())
        for i in range(9, 30):  # the second has ended: another graph (one row) is captured in mid-sequence
            got.append(e.step([(slots[0], [seqs[0][i]], [0])]).cpu().numpy())
        for slot in slots:
            e.close(slot)
        outs.append(np.concatenate(got))
    assert engine.graphs is not None and engine.graphs.graphs, "the engine did not replay captured graphs"
    np.testing.assert_array_equal(outs[0], outs[1])


def test_greedy_generation_through_the_entry_point(tmp_path):
    from abacus_b200 import LM
    folder, raw, tensors = lm.write_folder(tmp_path, "Q")
    model = LM(folder, dtype="float32", max_tokens=64 * 16)
    rng = np.random.default_rng(2)
    prompts = [[int(t) for t in rng.integers(0, raw["vocab"], n)] for n in (12, 3, 30)]
    outs = model.generate(prompts, max_new_tokens=20, temperature=0.0, stop_tokens=[])
    for p, out in zip(prompts, outs):
        assert len(out) == 20
        logits = plain.Plain(raw, tensors).feed(p + out)[0]
        for i, t in enumerate(out):  # each token is the plain model's choice, or within rounding of it
            row = logits[len(p) + i - 1]
            assert row[t] >= row.max() - 1e-3, f"token {i}: the engine chose {t}, the plain model {int(row.argmax())}"
    again = model.generate(prompts[::-1], max_new_tokens=20, temperature=0.0, stop_tokens=[], batch_size=2)
    assert again == outs[::-1]


def test_trace_replay_of_a_model_folder(tmp_path):
    folder, raw, tensors = lm.write_folder(tmp_path, "R")
    rng = np.random.default_rng(4)
    a, b = ([int(t) for t in rng.integers(0, raw["vocab"], n)] for n in (70, 9))
    run = TraceRun(folder, "float32", tmp_path / "out", 64 * 8)
    got = run.step([("a", a[:66], [0, 65]), ("b", b[:8], [7])]).reshape(3, -1)
    more = [run.step([("a", [a[66 + i]], [0])] + ([("b", [b[8]], [0])] if i == 0 else []), end=["b"] if i == 0 else []) for i in range(4)]
    run.step([], end=["a"])
    run.close()
    (wa, noise), (wb, _) = _oracle(raw, tensors, a), _oracle(raw, tensors, b)
    assert_logits(got, np.stack([wa[0], wa[65], wb[7]]), "float32", "replayed prompt", noise)
    assert_logits(more[0].reshape(2, -1), np.stack([wa[66], wb[8]]), "float32", "replayed decode", noise)
    assert_logits(np.stack([m.reshape(-1, raw["vocab"])[0] for m in more[1:]]), wa[67:70], "float32", "replayed decode", noise)


@pytest.mark.parametrize("width,vocab,ff,expert_ff", [(37, 61, 33, 9), (100, 203, 72, 20)])
def test_a_width_that_fits_no_vector(tmp_path, width, vocab, ff, expert_ff):
    """Every size odd or a multiple of 4 at most: width, vocabulary, feed-forwards, heads of 7, 9, 10 and 12 channels with
    values of 5, 7, 14 and 20; a prompt, then tokens one by one, in float32 against the plain model."""
    raw = {"architecture": "Linonex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "max_positions": 512,
           "layers": [lm.memory_layer(3, 10, 14, 9.0, lm.dense(ff)),
                      lm.parallel_layer(lm.left(6, 2, 12, 20, 0.2, 3, 50, 20.0), lm.right(4, 2, 12, 10, 4),
                                        lm.experts(5, 1, 2, 1.3, expert_ff)),
                      lm.parallel_layer(lm.left(3, 1, 7, 5, 0.3, 2, 9, 8.0), lm.right(3, 3, 9, 7, 2), lm.dense(ff))],
           "loop": {"start": 1, "stop": 3, "times": 2}}
    engine, raw, tensors, _ = _engine(tmp_path, f"odd{width}", "float32", raw=raw, seed=3)
    rng = np.random.default_rng(1)
    tokens = [int(t) for t in rng.integers(0, vocab, 200)]
    want, noise = _oracle(raw, tensors, tokens)
    slot = engine.open()
    got = [engine.step([(slot, tokens[:170], list(range(170)))]).cpu().numpy()]
    got += [engine.step([(slot, [t], [0])]).cpu().numpy() for t in tokens[170:]]
    engine.close(slot)
    engine.check_status()
    assert_logits(np.concatenate(got), want, "float32", f"width {width}", noise)


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_against_the_plain_model(tmp_path, seed):
    rng = np.random.default_rng(100 + seed)
    raw = lm.random_config(rng)
    engine, raw, tensors, _ = _engine(tmp_path, f"fuzz{seed}", "float32", raw=raw, seed=seed)
    seqs = [[int(t) for t in rng.integers(0, raw["vocab"], n)] for n in (75, 2, 130)]
    cut = [70, 1, 66]
    oracle = [_oracle(raw, tensors, s) for s in seqs]
    slots = [engine.open() for _ in seqs]
    got = engine.step([(slot, s[:c], list(range(c))) for slot, s, c in zip(slots, seqs, cut)]).cpu().numpy()
    at = 0
    for i, c in enumerate(cut):
        assert_logits(got[at:at + c], oracle[i][0][:c], "float32", f"{json_of(raw)} prompt {i}", oracle[i][1])
        at += c
    got = engine.step([(slot, [s[c]], [0]) for slot, s, c in zip(slots, seqs, cut)]).cpu().numpy()
    for i, c in enumerate(cut):
        assert_logits(got[i:i + 1], oracle[i][0][c:c + 1], "float32", f"{json_of(raw)} decode {i}", oracle[i][1])
    engine.check_status()


def json_of(raw):
    import json
    return json.dumps(raw["layers"])[:400]
