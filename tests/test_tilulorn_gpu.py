"""Tilulorn on the GPU against the plain implementation (tests/plain/tilulorn_plain.py): every mechanism alone as the
part the model uses (whole, in portions where the part takes them, token by token, in unequal batches, in slots used
before), keys far away and at the edges of windows and pages, then whole models through the engine: prompts, decoding,
batches, captured graphs, greedy generation through the library's entry point, and the trace replay."""
import numpy as np
import pytest
import torch

import tilulorn_models as tm
from helpers import TraceRun, assert_logits
from plain import tilulorn_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
BOTH = ["float32", "bfloat16"]


def _rnd(dtype):
    return tm.bf16_round if dtype == "bfloat16" else (lambda a: np.asarray(a, dtype=np.float32))


def _f64(p):
    return {n: (t if t.dtype.kind == "i" else t.astype(np.float64)) for n, t in p.items()}


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
    given rows (and, for a feed-forward that looks at them, given token ids)."""

    def __init__(self, spec, params, dtype, feed_forward=False):
        from abacus_b200.cache import SequenceCache
        from abacus_b200.parts import FEED_FORWARDS, MIXERS, BuildContext, Workspace
        self.dtype, self.feed_forward = dtype, feed_forward
        self.part = (FEED_FORWARDS if feed_forward else MIXERS).build(spec)
        assert set(self.part.param_shapes()) == set(params), set(self.part.param_shapes()) ^ set(params)
        for n, shape in self.part.param_shapes().items():
            assert tuple(params[n].shape) == tuple(shape), (n, params[n].shape, shape)
        device = torch.device(DEV, torch.cuda.current_device())
        self.part.bind({n: torch.from_numpy(np.ascontiguousarray(t) if t.dtype.kind == "i" else np.ascontiguousarray(t, dtype=np.float32))
                        for n, t in params.items()}, BuildContext(device=device, dtype=DT[dtype]))
        self.ws = Workspace(device)
        self.cache = None
        if not feed_forward:
            self.cache = SequenceCache([self.part.cache_need()], [None], 64 * 64, DT[dtype], DEV)
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

    def close(self, slot):
        self.cache.close_slot(slot)

    def step(self, entries, tokens=None):
        """entries: [(slot or None, rows [n, d])] -> [out [n, d]] float32. tokens: the rows' token ids, entry by entry."""
        from abacus_b200.engine.batch import Sequence, StepBatch
        plans = getattr(self.part, "step_plans", lambda: [])()
        n = sum(len(h) for _, h in entries)
        seqs = []
        for i, (slot, h) in enumerate(entries):
            start = self.length.get(slot, 0)
            if self.cache is not None:
                self.cache.reserve(slot, start + len(h))
                self.length[slot] = start + len(h)
            seqs.append(Sequence(slot if slot is not None else i, list(tokens[i]) if tokens is not None else [0] * len(h), start, []))
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
    """The rows h of one sequence: whole, in portions down to two tokens and one (None: the part takes a sequence's
    several tokens only at its start), token by token, and in an unequal batch in slots that were used before."""
    T = len(h)
    slot = run.open()
    _close(run.step([(slot, h)])[0], want, dtype, f"{what}, whole")
    run.close(slot)
    if portions:
        slot, at, got = run.open(dirty=True), 0, []
        for size in portions:
            got.append(run.step([(slot, h[at:at + size])])[0])
            at += size
        assert at == T
        _close(np.concatenate(got), want, dtype, f"{what}, in portions")
        run.close(slot)
    slot = run.open(dirty=True)
    got = np.concatenate([run.step([(slot, h[t:t + 1])])[0] for t in range(40)])
    _close(got, want[:40], dtype, f"{what}, token by token")
    run.close(slot)
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
        run.close(s)


# ------------------------------------------------------------------ wkv
_WKV_SLOTS = {"mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w", "wr": "r", "wk": "k", "wv": "v",
              "wg": "g", "w1": "w1", "w2": "w2", "w0": "w0", "bonus": "u", "out_norm": "norm", "wo": "o"}


def _wkv(rng, d, H, K, rank, rnd, w0=(-5.0, 1.0)):
    p = {"mu." + s: rng.uniform(0, 1, d) for s in "rkvgw"}
    for s in "rkvg":
        p[s] = rng.standard_normal((H * K, d)) * 1.5 / np.sqrt(d)
    p.update(w1=rng.standard_normal((rank, d)) * 2 / np.sqrt(d), w2=rng.standard_normal((H * K, rank)) * 2 / np.sqrt(rank),
             w0=rng.uniform(w0[0], w0[1], H * K), u=rng.standard_normal((H, K)) * 0.5, norm=1 + rng.standard_normal(H * K) * 0.1,
             o=rng.standard_normal((d, H * K)) / np.sqrt(H * K))
    return {n: rnd(t) for n, t in p.items()}


def _wkv_run(p, d, H, K, rank, dtype):
    from abacus_b200.config.specs import WkvSpec
    return PartRun(WkvSpec(hidden=d, n_heads=H, key_dim=K, decay_rank=rank, norm_eps=1e-5),
                   {slot: p[short] for slot, short in _WKV_SLOTS.items()}, dtype)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,K,rank", [(2, 5, 3), (3, 16, 8), (1, 40, 6), (2, 64, 16), (2, 128, 5), (1, 200, 24)])
def test_wkv_every_way(dtype, H, K, rank):
    # (a width of 64: in bfloat16 a step of a few rows makes the five products in one launch; 40: each on its own)
    rng, rnd, d = np.random.default_rng(K), _rnd(dtype), 64 if K in (16, 64) else 40
    p = _wkv(rng, d, H, K, rank, rnd)
    h = rnd(rng.standard_normal((150, d)))
    want, _ = plain.wkv(h.astype(np.float64), {"heads": H, "dim": K}, _f64(p), 1e-5, None)
    _every_way(_wkv_run(p, d, H, K, rank, dtype), h, want, dtype, f"wkv {H} x {K}")


def test_wkv_keeps_a_token_over_a_long_decoding_and_forgets_with_decays_near_nothing():
    """Decays all but one: a loud early token is read back after 400 single-token steps (and the token before it is what
    the blends saw); decays all but nothing: only the token's own bonus term and the token before are left."""
    rng, d, H, K = np.random.default_rng(5), 24, 2, 16
    for w0, what in (((-12.0, -9.0), "lasting"), ((4.0, 5.0), "fading")):
        p = _wkv(rng, d, H, K, 4, _rnd("float32"), w0)
        h = rng.standard_normal((420, d)).astype(np.float32)
        h[3] *= 6.0
        want, _ = plain.wkv(h.astype(np.float64), {"heads": H, "dim": K}, _f64(p), 1e-5, None)
        other = h.copy()
        other[3] /= 6.0
        moved, _ = plain.wkv(other.astype(np.float64), {"heads": H, "dim": K}, _f64(p), 1e-5, None)
        assert (np.abs(want[-1] - moved[-1]).max() > 1e-2) == (what == "lasting")
        run = _wkv_run(p, d, H, K, 4, "float32")
        slot = run.open(dirty=True)
        got = [run.step([(slot, h[:20])])[0]] + [run.step([(slot, h[t:t + 1])])[0] for t in range(20, 420)]
        _close(np.concatenate(got), want, "float32", f"wkv {what}", f32=5e-4)


# ------------------------------------------------------------------ latent attention
_LATENT_SLOTS = {"wdq": "dq", "q_norm": "dq.norm", "wq": "uq", "wdown": "dkv", "down_norm": "dkv.norm", "wuk": "uk",
                 "wuv": "uv", "wg": "g", "wo": "o"}


def _latent(rng, d, m, rnd):
    H, K, R, V, rank, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
    p = {"dq": rng.standard_normal((qr, d)) / np.sqrt(d), "dq.norm": 1 + rng.standard_normal(qr) * 0.1,
         "uq": rng.standard_normal((H * (K + R), qr)) * 3 / np.sqrt(qr), "dkv": rng.standard_normal((rank + R, d)) * 1.5 / np.sqrt(d),
         "dkv.norm": 1 + rng.standard_normal(rank) * 0.1, "uk": rng.standard_normal((H * K, rank)) * 3 / np.sqrt(rank),
         "uv": rng.standard_normal((H * V, rank)) / np.sqrt(rank), "g": rng.standard_normal((H, d)) * 2 / np.sqrt(d),
         "o": rng.standard_normal((d, H * V)) / np.sqrt(H * V)}
    return {n: rnd(t) for n, t in p.items()}


def _latent_run(p, d, m, dtype):
    from abacus_b200.config.tilulorn import TilulornLatent
    from abacus_b200.config.specs import LatentAttentionSpec
    c = TilulornLatent.from_dict("", m)
    spec = LatentAttentionSpec(hidden=d, n_heads=c.heads, head_dim=c.dim, rot_dim=c.rot_dim, v_head_dim=c.vdim, rank=c.kv_rank,
                               scale=c.scale, norm_eps=1e-5, position=None if c.rot is None else c.rot.to_spec("half"),
                               q_rank=c.q_rank, head_gate=True)
    return PartRun(spec, {slot: p[short] for slot, short in _LATENT_SLOTS.items()}, dtype)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("sizes,rotation", [
    ((3, 16, 8, 24, 24, 20), tm.rot(10000.0, 8, 4.0, 64, 8.0, 1.0)),   # blended frequencies; sizes of whole vectors
    ((2, 10, 6, 7, 21, 9), tm.rot(100.0, 6)),                          # sizes that fit no vector; plain frequencies
    ((1, 12, 4, 12, 16, 16), None),                                     # no rotation at all
    ((4, 8, 16, 8, 32, 24), tm.rot(10000.0, 12, 3.0)),                  # part of the rotated part turns, slowed
    ((5, 32, 16, 40, 64, 48), tm.rot(50000.0, 16, 8.0, 1024, 16.0, 2.0)),
])
def test_latent_attention_with_query_latents_and_gated_heads_every_way(dtype, sizes, rotation):
    H, K, R, V, rank, qr = sizes
    rng, rnd, d = np.random.default_rng(K + R), _rnd(dtype), 48
    m = {"heads": H, "dim": K, "rot_dim": R, "vdim": V, "kv_rank": rank, "q_rank": qr, "scale": 0.25}
    if rotation is not None:
        m["rot"] = rotation
    p = _latent(rng, d, m, rnd)
    h = rnd(rng.standard_normal((150, d)))
    want, _ = plain.latent_attention(h.astype(np.float64), m, _f64(p), 1e-5, None)
    _every_way(_latent_run(p, d, m, dtype), h, want, dtype, f"latent attention {sizes}")


@pytest.mark.parametrize("dtype", BOTH)
def test_latent_attention_finds_one_loud_key_far_away_and_at_page_borders(dtype):
    """The rotated parts alone carry the scores (position 0's rotation is the identity, so a loud query and key match
    where their positions' rotations agree best: at the key's own position for slow frequencies). One key among hundreds
    is made loud through the down-projection's unrotated latent instead: a head's plain query part reads input columns
    that only the query row fills, its keys columns that only the key row fills."""
    rng, d = np.random.default_rng(3), 40
    m = {"heads": 2, "dim": 8, "rot_dim": 8, "vdim": 8, "kv_rank": 16, "q_rank": 8, "scale": 1.0, "rot": tm.rot(10000.0, 8, 4.0, 64, 8.0, 1.0)}
    p = _latent(rng, d, m, _rnd(dtype))
    # queries: latent = input columns 0..8 (through a unit norm weight); keys: latent columns 0..8 = input columns 8..16
    p["dq"] = np.eye(d)[:8].astype(np.float32)
    p["dq.norm"] = np.ones(8, np.float32)
    uq = np.zeros((2 * 16, 8), np.float32)
    uq[:8] = np.eye(8) * 4
    uq[16:24] = np.eye(8) * 4
    p["uq"] = uq
    dkv = rng.standard_normal((24, d)).astype(np.float32) / np.sqrt(d)  # (the other latents and the rotated part: ordinary)
    dkv[:8] = 0
    dkv[:8, 8:16] = np.eye(8)
    p["dkv"] = tm.bf16_round(dkv)
    p["dkv.norm"] = np.ones(16, np.float32)
    uk = np.zeros((16, 16), np.float32)
    uk[:8, :8] = np.eye(8)
    uk[8:, :8] = np.eye(8)
    p["uk"] = uk
    u = rng.standard_normal(8)
    u /= np.linalg.norm(u)
    T = 330
    run = _latent_run(p, d, m, dtype)
    for i, j in [(T - 1, 0), (T - 1, 1), (T - 1, 63), (T - 1, 64), (T - 1, 65), (200, 127), (200, 128), (129, 128), (T - 1, T - 2), (70, 70)]:
        h = rng.standard_normal((T, d)) * 0.3
        h[:, :16] *= 0.2
        h[i, :8] = 3.0 * u
        h[j, 8:16] = 5.0 * u
        h = _rnd(dtype)(h)
        want, _ = plain.latent_attention(h.astype(np.float64), m, _f64(p), 1e-5, None)
        quiet = h.copy()
        quiet[j, 8:16] = 0.0
        without, _ = plain.latent_attention(quiet.astype(np.float64), m, _f64(p), 1e-5, None)
        assert np.abs(want[i] - without[i]).max() > 0.2, "the loud key decides nothing: the test shows nothing"
        run.cache.views[0].kv.k.fill_(9.0)  # what former users left in the pages
        slot = run.open(dirty=True)
        _close(run.step([(slot, h[:i + 1])])[0], want[:i + 1], dtype, f"query {i}, loud key {j}, prompt")
        run.close(slot)
        slot, cut = run.open(dirty=True), max(1, i - 3 if j < i - 3 else j - 1)
        got = [run.step([(slot, h[:cut])])[0]] + [run.step([(slot, h[t:t + 1])])[0] for t in range(cut, i + 1)]
        _close(np.concatenate(got), want[:i + 1], dtype, f"query {i}, loud key {j}, decoded from {cut}")
        run.close(slot)


# ------------------------------------------------------------------ attention whose values are its keys
_WINDOW_SLOTS = {"wq": "q", "wk": "k", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink", "wg": "g", "wo": "o"}


def _window(rng, d, H, G, K, rnd):
    p = {"q": rng.standard_normal((H * K, d)) * 2 / np.sqrt(d), "k": rng.standard_normal((G * K, d)) * 2 / np.sqrt(d),
         "q.norm": 2 + rng.standard_normal(H * K) * 0.3, "k.norm": 2 + rng.standard_normal(G * K) * 0.3,
         "sink": rng.standard_normal(H) * 1.5, "g": rng.standard_normal((H, d)) * 2 / np.sqrt(d),
         "o": rng.standard_normal((d, H * K)) / np.sqrt(H * K)}
    return {n: rnd(t) for n, t in p.items()}


def _window_run(p, d, m, dtype):
    from abacus_b200.config.tilulorn import TilulornWindowed
    from abacus_b200.config.specs import AttentionSpec
    c = TilulornWindowed.from_dict("", m)
    spec = AttentionSpec(hidden=d, n_heads=c.heads, n_kv_heads=c.kv_heads, head_dim=c.dim, scale=c.scale, qk_norm_eps=1e-5,
                         position=None if c.rot is None else c.rot.to_spec("interleaved"), window=c.window, sink=True,
                         exact_weights=True, norm_over="projection", values="keys", head_gate=True)
    return PartRun(spec, {slot: p[short] for slot, short in _WINDOW_SLOTS.items()}, dtype)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("H,G,K,window,rotation", [
    (4, 2, 16, 40, tm.rot(5000.0, 8, 2.0)),       # half of each head turns, slowed
    (3, 3, 12, None, tm.rot(1000.0, 12)),         # every earlier key; a head that fits no vector
    (4, 2, 16, None, tm.rot(1000.0, 16, 4.0, 64, 8.0, 1.0)),   # every earlier key, heads the tensor-core kernels take
    (1, 1, 20, 9, None),                          # no rotation
    (6, 1, 8, 64, tm.rot(20000.0, 8, 8.0, 32, 4.0, 1.0)),   # a window of a page; blended frequencies; one key head
    (8, 2, 64, 130, tm.rot(30000.0, 64, 3.0)),
    (2, 2, 7, 5, tm.rot(300.0, 4)),
])
def test_attention_with_values_that_are_keys_a_window_and_a_sink_every_way(dtype, H, G, K, window, rotation):
    rng, rnd, d = np.random.default_rng(K), _rnd(dtype), 40
    m = {"heads": H, "kv_heads": G, "dim": K, "vdim": K, "scale": 0.3}
    if window is not None:
        m["mask"] = {"size": window}
    if rotation is not None:
        m["rot"] = rotation
    p = _window(rng, d, H, G, K, rnd)
    h = rnd(rng.standard_normal((150, d)))
    want, _ = plain.window_attention(h.astype(np.float64), m, _f64(p), 1e-5, None)
    # (the part takes several tokens of a windowed sequence only at its start: no portions)
    _every_way(_window_run(p, d, m, dtype), h, want, dtype, f"attention {H}/{G} x {K}, window {window}",
               portions=None if window is not None else (60, 2, 7, 1, 64, 16))


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("window", [5, 64, 80, 130])
def test_one_loud_key_just_inside_and_just_outside_the_window(window, dtype):
    """A key made loud for one query alone (q reads one part of the input row, k another; the norm over the whole row
    keeps directions): the oldest key the window still holds, the first it has dropped, keys on both sides of a page's
    border, the token's own; in a prompt and for tokens that come one by one over a ring of pages that has gone round."""
    rng, K, T = np.random.default_rng(window), 8, 300
    d = 2 * K + 4
    p = {"q": np.eye(d)[:K] * 1.0, "k": np.eye(d)[K:2 * K] * 1.0, "q.norm": np.ones(K), "k.norm": np.ones(K),
         "sink": np.array([0.5]), "g": np.zeros((1, d)), "o": np.eye(d)[:, :K]}
    p = {n: np.asarray(t, dtype=np.float32) for n, t in p.items()}
    m = {"heads": 1, "kv_heads": 1, "dim": K, "vdim": K, "scale": 6.0, "mask": {"size": window}}
    u = rng.standard_normal(K)
    u /= np.linalg.norm(u)
    run = _window_run(p, d, m, dtype)
    pairs = set()
    for i in (window - 1, window, 2 * window + 3, 192, T - 1):
        if window - 1 <= i < T:
            pairs |= {(i, i - window + 1), (i, i - window), (i, i), (i, i - 1), (i, max(i - window + 1, i // 64 * 64)),
                      (i, max(i - window + 1, i // 64 * 64 - 1))}
    for i, j in sorted((i, j) for i, j in pairs if j >= 0):
        h = rng.standard_normal((T, d)) * 0.3
        h[:, K:2 * K] -= np.outer(h[:, K:2 * K] @ u, u)  # (the norm levels the keys' sizes: the others point elsewhere)
        h[i, :K] = 4.0 * u
        h[j, K:2 * K] = 4.0 * u
        h = _rnd(dtype)(h)
        want, _ = plain.window_attention(h.astype(np.float64), m, _f64(p), 1e-5, None)
        seen = 0 <= i - j < window
        if j != i:  # the loud key's value (its projection, unnormed) decides the answer if and only if the window holds it
            assert (np.abs(want[i, :K] / 0.5 - h[j, K:2 * K]).max() < 0.1 * 4.0) == seen, (i, j)
        run.cache.views[0].kv.k.fill_(9.0), run.cache.views[0].kv.v.fill_(9.0)  # what former users left in the pages
        slot = run.open(dirty=True)
        _close(run.step([(slot, h[:i + 1])])[0], want[:i + 1], dtype, f"query {i}, loud key {j}, prompt")
        run.close(slot)
        if i - j not in (window - 1, window, 0):  # tokens one by one: for the keys at the window's far edge and the token's own
            continue
        slot, cut = run.open(dirty=True), max(1, min(i - 3, j - 1))
        got = [run.step([(slot, h[:cut])])[0]] + [run.step([(slot, h[t:t + 1])])[0] for t in range(cut, i + 1)]
        _close(np.concatenate(got), want[:i + 1], dtype, f"query {i}, loud key {j}, decoded from {cut}")
        run.close(slot)


def test_the_sink_takes_its_share_and_the_norm_spans_all_heads():
    """Against the plain function, which the CPU tests hold to closed forms: a sink so large that it takes nearly all the
    weight, one so small that it takes none, and a head whose projection is scaled (which the norm over the whole row
    hands on to the other heads)."""
    rng, d, H, G, K = np.random.default_rng(8), 32, 4, 2, 8
    m = {"heads": H, "kv_heads": G, "dim": K, "vdim": K, "scale": 0.4, "mask": {"size": 33}, "rot": tm.rot(100.0, 8, 2.0)}
    p = _window(rng, d, H, G, K, _rnd("float32"))
    p["sink"] = np.array([9.0, -30.0, 0.0, 2.0], np.float32)
    p["q"][:K] *= 5.0
    h = rng.standard_normal((100, d)).astype(np.float32)
    want, _ = plain.window_attention(h.astype(np.float64), m, _f64(p), 1e-5, None)
    run = _window_run(p, d, m, "float32")
    slot = run.open()
    _close(run.step([(slot, h)])[0], want, "float32", "sinks of every size")


# ------------------------------------------------------------------ experts by a table
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("E,top,d,ff", [(1, 1, 24, 8), (5, 2, 40, 24), (3, 3, 64, 16), (12, 1, 64, 64), (9, 4, 37, 9)])
def test_experts_picked_by_a_table(dtype, E, top, d, ff):
    from abacus_b200.config.specs import ExpertSpec, RoutedMLPSpec
    rng, rnd, vocab = np.random.default_rng(E), _rnd(dtype), 53
    w = {}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = rnd(rng.standard_normal((ff, d)) * 1.5 / np.sqrt(d)), rnd(rng.standard_normal((ff, d)) * 1.5 / np.sqrt(d))
        w[f"e{e}.down"] = rnd(rng.standard_normal((d, ff)) * 1.5 / np.sqrt(ff))
    w["table"] = np.stack([rng.permutation(E)[:top] for _ in range(vocab)]).astype(np.int32)
    spec = RoutedMLPSpec(hidden=d, experts=E, top=top, expert=ExpertSpec(ff, "silu_gated"), shared=None, score="table",
                         weight_on="output", vocab=vocab)
    params = {"table": w["table"]}
    for e in range(E):
        params.update({f"gate{e}": w[f"e{e}.gate"], f"up{e}": w[f"e{e}.up"], f"down{e}": w[f"e{e}.down"]})
    run = PartRun(spec, params, dtype, feed_forward=True)
    mlp = tm.experts(E, top, ff)
    for rows in (1, 9, 70, 300):  # few pairs: each row against its expert's matrices; many: sorted by expert
        h = rnd(rng.standard_normal((rows, d)))
        tokens = [int(t) for t in rng.integers(0, vocab, rows)]
        want = plain.table_experts(h.astype(np.float64), tokens, mlp, _f64(w))
        cut = rows // 3
        got = np.concatenate(run.step([(None, h[:cut]), (None, h[cut:])] if cut else [(None, h)],
                                      tokens=[tokens[:cut], tokens[cut:]] if cut else [tokens]))
        _close(got, want, dtype, f"{top} of {E} experts, {rows} rows")


def test_several_products_of_a_few_rows_in_one_launch():
    """Runs of output features that each read an input of their own (the last run shorter), against float64."""
    from abacus_b200.kernels import ops
    rng = np.random.default_rng(12)
    for rows, k, block, n in ((1, 64, 48, 48 * 4 + 8), (8, 320, 128, 128 * 4 + 16), (13, 1024, 1024, 4096 + 64)):
        runs = -(-n // block)
        x = tm.bf16_round(rng.standard_normal((runs, rows, k)))
        w = tm.bf16_round(rng.standard_normal((n, k)) / np.sqrt(k))
        want = np.concatenate([x[i].astype(np.float64) @ w[i * block:(i + 1) * block].astype(np.float64).T for i in range(runs)], axis=1)
        xd, wd = torch.from_numpy(x).to(DEV).to(torch.bfloat16), torch.from_numpy(w).to(DEV).to(torch.bfloat16)
        for out_dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 8e-3)):
            out = torch.full((rows, n), 7.0, dtype=out_dtype, device=DEV)
            ops.gemm_rows_planes(xd, wd, out, block, rows)
            torch.cuda.synchronize()
            assert np.abs(out.float().cpu().numpy() - want).max() <= tol * max(np.abs(want).max(), 1.0), (rows, k, block, n, out_dtype)


# ------------------------------------------------------------------ whole models through the engine
def _engine(tmp, name, dtype, raw=None, seed=0, tensors=None, **kw):
    from abacus_b200.engine import Engine, load_model
    folder, raw, tensors = tm.write_folder(tmp, name, seed=seed, raw=raw, tensors=tensors)
    return Engine(load_model(folder, dtype), max_tokens=64 * 24, **kw), raw, tensors, folder


def _oracle(raw, tensors, tokens):
    """(the plain model's logits in float64, the noise float32 itself shows on them)."""
    want = plain.PlainTilulorn(raw, tensors).forward(tokens)
    return want, float(np.abs(want - plain.PlainTilulorn(raw, tensors, real=np.float32).forward(tokens)).max())


class Bf16Count:
    """bfloat16 against float64: the distance of two roundings of one model, a few per cent of the logits' spread (the
    test models' queries and keys are large, so that a wrong key shows; rounding them moves the weights by per cents).
    Positions far off are counted, and few are allowed over a whole test."""

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


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "float32"), ("D", "float32"),
                                        ("A", "bfloat16"), ("C", "bfloat16"), ("D", "bfloat16")])
def test_prompts_decoding_batches_and_used_slots_against_the_plain_model(tmp_path, name, dtype):
    engine, raw, tensors, _ = _engine(tmp_path, name, dtype)
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


def test_portions_of_a_prompt_where_no_window_forbids_them(tmp_path):
    """Configuration B without its windowed layer's window: a prompt in portions down to two tokens and one."""
    raw = tm.config("B")
    del raw["layers"][4]["mixer"]["mask"]
    engine, raw, tensors, _ = _engine(tmp_path, "Bfull", "float32", raw=raw)
    rng = np.random.default_rng(5)
    tokens = [int(t) for t in rng.integers(0, raw["vocab"], 140)]
    want, noise = _oracle(raw, tensors, tokens)
    slot, got, at = engine.open(), [], 0
    for size in (60, 2, 7, 1, 64, 6):
        got.append(engine.step([(slot, tokens[at:at + size], list(range(size)))]).cpu().numpy())
        at += size
    engine.close(slot)
    assert at == len(tokens)
    assert_logits(np.concatenate(got), want, "float32", "B in portions", noise)


@pytest.mark.parametrize("name", ["A", "C"])
def test_token_by_token_from_the_first_token_and_long_decoding(tmp_path, name):
    engine, raw, tensors, _ = _engine(tmp_path, name, "float32")
    rng = np.random.default_rng(3)
    tokens = [int(t) for t in rng.integers(0, raw["vocab"], 220)]
    want, noise = _oracle(raw, tensors, tokens)
    slot = engine.open()
    got = np.concatenate([engine.step([(slot, [t], [0])]).cpu().numpy() for t in tokens])
    engine.close(slot)
    assert_logits(got, want, "float32", f"{name} token by token", noise)


def test_graphs_and_plain_launches_give_the_same_bits_and_states_survive_a_capture(tmp_path):
    from abacus_b200.engine import Engine
    engine, raw, tensors, _ = _engine(tmp_path, "A", "float32")
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
    want = np.concatenate([_oracle(raw, tensors, seqs[0])[0][4:5], _oracle(raw, tensors, seqs[1])[0][4:5]])
    assert_logits(outs[0][:2], want, "float32", "captured", 1e-4)


def test_greedy_generation_through_the_entry_point(tmp_path):
    from abacus_b200 import LM
    folder, raw, tensors = tm.write_folder(tmp_path, "D")
    model = LM(folder, dtype="float32", max_tokens=64 * 16)
    rng = np.random.default_rng(2)
    prompts = [[int(t) for t in rng.integers(0, raw["vocab"], n)] for n in (12, 3, 30)]
    outs = model.generate(prompts, max_new_tokens=20, temperature=0.0, stop_tokens=[])
    for p, out in zip(prompts, outs):
        assert len(out) == 20
        logits = plain.PlainTilulorn(raw, tensors).forward(p + out)
        for i, t in enumerate(out):  # each token is the plain model's choice, or within rounding of it
            row = logits[len(p) + i - 1]
            assert row[t] >= row.max() - 1e-3, f"token {i}: the engine chose {t}, the plain model {int(row.argmax())}"
    again = model.generate(prompts[::-1], max_new_tokens=20, temperature=0.0, stop_tokens=[], batch_size=2)
    assert again == outs[::-1]


def test_trace_replay_of_a_model_folder(tmp_path):
    folder, raw, tensors = tm.write_folder(tmp_path, "C")
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


@pytest.mark.parametrize("seed", range(10))
def test_random_configurations_against_the_plain_model(tmp_path, seed):
    rng = np.random.default_rng(100 + seed)
    raw = tm.random_config(rng)
    engine, raw, tensors, _ = _engine(tmp_path, f"fuzz{seed}", "float32", raw=raw, seed=seed)
    seqs = [[int(t) for t in rng.integers(0, raw["vocab"], n)] for n in (75, 2, 130)]
    cut = [70, 1, 66]
    oracle = [_oracle(raw, tensors, s) for s in seqs]
    slots = [engine.open() for _ in seqs]
    what = str([l["type"] for l in raw["layers"]]) + str(raw.get("loop"))
    got = engine.step([(slot, s[:c], list(range(c))) for slot, s, c in zip(slots, seqs, cut)]).cpu().numpy()
    at = 0
    for i, c in enumerate(cut):
        assert_logits(got[at:at + c], oracle[i][0][:c], "float32", f"{what} prompt {i}", oracle[i][1])
        at += c
    for step in range(2):
        live = [i for i, (s, c) in enumerate(zip(seqs, cut)) if c + step < len(s)]
        got = engine.step([(slots[i], [seqs[i][cut[i] + step]], [0]) for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            assert_logits(got[j:j + 1], oracle[i][0][cut[i] + step:cut[i] + step + 1], "float32", f"{what} decode {i}", oracle[i][1])
    engine.check_status()
