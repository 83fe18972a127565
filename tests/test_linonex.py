"""Linonex without a GPU: the configuration and its round trip, the tensor names, configurations that must be refused,
the run order of a loop, what the side-by-side mixer asks of the cache, and the plain implementation against closed
forms of its own mechanisms."""
import json

import numpy as np
import pytest

import linonex_models as lm
from plain import linonex_plain as plain


def _spec(raw):
    from abacus_b200.config.registry import architecture_of
    arch = architecture_of(raw)
    cfg = arch.parse_config(raw)
    return arch, cfg, cfg.to_spec()


@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_configuration_round_trip_and_tensor_names(name):
    raw = lm.config(name)
    arch, cfg, spec = _spec(raw)
    assert arch.name == "Linonex"
    again = arch.parse_config(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    expected, _ = arch.tensor_names(spec, None)
    tensors = lm.weights(raw)
    assert set(expected) == set(tensors)
    for n, shape in expected.items():
        assert tuple(shape) == tensors[n].shape, n
    assert "linonex" in arch.info(spec)


def test_the_run_order_of_a_loop_and_where_the_embedding_joins_again():
    _, cfg, spec = _spec(lm.config("P"))
    assert [(e.layer, e.rejoin) for e in spec.schedule] == [(0, False), (1, False), (0, True), (1, False), (0, True),
                                                            (1, False), (2, False), (3, False)]
    assert all(e.source is None for e in spec.schedule) and spec.frame_spec.keep
    assert [(l, again) for l, _, again in plain.run_order(lm.config("P"))] == [(e.layer, e.rejoin) for e in spec.schedule]
    _, _, spec = _spec(lm.config("Q"))
    assert [e.layer for e in spec.schedule] == [0, 1, 2] and not spec.frame_spec.keep
    raw = lm.config("R")
    raw["loop"] = {"start": 1, "stop": 3, "times": 2}
    _, _, spec = _spec(raw)
    assert [(e.layer, e.rejoin) for e in spec.schedule] == [(0, False), (1, False), (2, False), (1, True), (2, False)]
    raw["loop"] = {"start": 1, "stop": 2, "times": 1}  # once through is no loop
    assert [e.layer for e in _spec(raw)[2].schedule] == [0, 1, 2]


def _broken(change):
    raw = lm.config("P")
    change(raw)
    return raw


@pytest.mark.parametrize("change", [
    lambda r: r["layers"][0].update(type="attention"),
    lambda r: r["layers"][1]["mixer"].pop("gate_cap"),
    lambda r: r["layers"][0]["mixer"].pop("right"),
    lambda r: r["layers"][0]["mixer"]["left"].update(heads=3),            # 3 heads over 2 key heads
    lambda r: r["layers"][0]["mixer"]["right"].update(kv_heads=3),
    lambda r: r["layers"][0]["mixer"]["left"]["mask"].update(size=0),
    lambda r: r["layers"][0]["mixer"]["left"].update(softcap=-1.0),
    lambda r: r["layers"][1]["mlp"]["router"].update(top=7),              # six router outputs
    lambda r: r["layers"][1]["mlp"].update(kind="shared"),
    lambda r: r.update(loop={"start": 2, "stop": 5, "times": 2}),
    lambda r: r.pop("max_positions"),
    lambda r: r["norm"].pop("eps"),
])
def test_configurations_that_are_refused(change):
    from abacus_b200.config.registry import ConfigError
    with pytest.raises(ConfigError):
        _spec(_broken(change))


def test_what_two_mixers_side_by_side_ask_of_the_cache():
    from abacus_b200.parts import MIXERS
    _, _, spec = _spec(lm.config("P"))
    mixer = MIXERS.build(spec.layers[0].mixer)
    need = mixer.cache_need()
    assert (need.n_kv_heads, need.head_dim, need.v_head_dim, need.window) == (2, 16, 8, None)
    names = {name: shape for name, shape, _ in need.states}
    row = -(-(4 * 16 + 2 * 16 + 2 * 8) // 8) * 8
    assert names == {"left.conv_tail": (1, row), "right.delta": (4, 16, 8), "right.conv_tail": (2, 2 * 2 * 8 + 4 * 16)}
    shapes = mixer.param_shapes()
    assert shapes["left_out"] == shapes["right_out"] == (64,) and shapes["left.conv_k"] == (32, 2)
    assert shapes["right.wa"] == (4, 64) and shapes["right.decay_bias"] == (4,)
    assert mixer.capturable


# ------------------------------------------------------------------ the plain implementation against itself
def test_the_matrix_memory_against_its_sum_over_the_past():
    """Unrolled, the recurrence is a sum over the past with weights exp(i_j + f_(j+1) + ... + f_t - m_t), and m_t the
    largest exponent there is or that of the start (0 + f_1 + ... + f_t)."""
    rng = np.random.default_rng(0)
    d, m = 12, {"heads": 2, "dim": 5, "vdim": 3, "gate_cap": 6.0}
    T, H, K, V = 9, 2, 5, 3
    p = {n: rng.standard_normal(s) for n, s in (("q", (H * K, d)), ("k", (H * K, d)), ("v", (H * V, d)), ("g", (H * V, d)),
                                                ("i", (H, d)), ("f", (H, d)), ("i.b", (H,)), ("f.b", (H,)),
                                                ("norm", (H * V,)), ("o", (d, H * V)))}
    h = rng.standard_normal((T, d))
    got, _ = plain.matrix_memory(h, p, m, 1e-5, None)
    q = (h @ p["q"].T).reshape(T, H, K) * K ** -0.5
    k, v = (h @ p["k"].T).reshape(T, H, K), (h @ p["v"].T).reshape(T, H, V)
    gi = 6.0 * np.tanh((h @ p["i"].T + p["i.b"]) / 6.0)
    gf = plain.log_sigmoid(6.0 * np.tanh((h @ p["f"].T + p["f.b"]) / 6.0))
    o = np.zeros((T, H, V))
    for t in range(T):
        for a in range(H):
            e = np.array([gi[j, a] + gf[j + 1:t + 1, a].sum() for j in range(t + 1)])
            mx = max(e.max(), gf[:t + 1, a].sum())
            wgt = np.exp(e - mx)
            num = sum(wgt[j] * (k[j, a] @ q[t, a]) * v[j, a] for j in range(t + 1))
            den = max(abs(sum(wgt[j] * (k[j, a] @ q[t, a]) for j in range(t + 1))), np.exp(-mx)) + 1e-6
            o[t, a] = num / den
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + 1e-5)
    want = (o.reshape(T, H * V) * p["norm"] * plain.sigmoid(h @ p["g"].T)) @ p["o"].T
    np.testing.assert_allclose(got, want, rtol=1e-9, atol=1e-9)


def test_state_carried_in_portions_is_the_whole_sequence():
    raw = lm.config("P")
    tensors = lm.weights(raw, 3)
    rng = np.random.default_rng(1)
    tokens = [int(t) for t in rng.integers(0, raw["vocab"], 60)]
    whole, layers = plain.Plain(raw, tensors).feed(tokens)
    cut = plain.Plain(raw, tensors)
    parts = [cut.feed(tokens[a:b])[0] for a, b in ((0, 1), (1, 8), (8, 50), (50, 52), (52, 60))]
    np.testing.assert_allclose(np.concatenate(parts), whole, rtol=1e-9, atol=1e-9)
    assert layers.shape == (8, 60, raw["width"])


def test_an_expert_that_returns_its_input_and_the_correction_of_the_choice():
    rng = np.random.default_rng(2)
    d, ff = 8, 4
    mlp = {"router": {"experts": 2, "identity": 1, "top": 1, "scale": 3.0}, "expert": {"ff": ff}}
    p = {"router": np.zeros((3, d)), "correction": np.array([0.0, 0.0, 0.5])}
    for e in range(2):
        p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"] = (rng.standard_normal(s) for s in ((ff, d), (ff, d), (d, ff)))
    h = rng.standard_normal((5, d))
    # equal scores of 1/3; the correction picks the last output, which returns h; the weight is the score, not the key
    np.testing.assert_allclose(plain.routed_ff(h, p, mlp), h * (3.0 / 3.0), rtol=1e-12)
    p["correction"] = np.array([0.0, 0.1, 0.0])
    np.testing.assert_allclose(plain.routed_ff(h, p, mlp), plain.gated_ff(h, p["e1.gate"], p["e1.up"], p["e1.down"]),
                               rtol=1e-12)


def test_keys_outside_the_chunk_do_not_count():
    rng = np.random.default_rng(4)
    d, m = 6, {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 3, "mask": {"size": 5}, "softcap": 4.0, "scale": 0.5}
    p = {"q": rng.standard_normal((8, d)), "k": rng.standard_normal((4, d)), "v": rng.standard_normal((3, d)),
         "o": rng.standard_normal((d, 6))}
    for t, rows in (("q", 8), ("k", 4), ("v", 3)):
        p[t + ".conv"] = np.concatenate([np.zeros((rows, 1)), np.ones((rows, 1))], axis=1)  # the token's own input only
    h = rng.standard_normal((12, d))
    whole, _ = plain.chunked_attention(h, p, m, None)
    # positions 5..9 as a sequence of their own: without a convolution that reaches back they see the same keys
    alone, _ = plain.chunked_attention(h[5:10], p, m, None)
    np.testing.assert_allclose(whole[5:10], alone, rtol=1e-10, atol=1e-12)
    other = h.copy()
    other[4] += 1.0  # the last key of the chunk before
    moved, _ = plain.chunked_attention(other, p, m, None)
    np.testing.assert_allclose(moved[5:], whole[5:], rtol=1e-12)
    assert np.abs(moved[4] - whole[4]).max() > 1e-3
