"""Tilulorn without a GPU: the configuration, the tensor names, what is refused, the run order of passes, the tables of
scaled frequencies, and the plain implementation's mechanisms against closed forms."""
import json

import numpy as np
import pytest

import tilulorn_models as tm
from plain import tilulorn_plain as plain


def _config(raw, shapes=None):
    from abacus_b200.config.registry import architecture_of
    arch = architecture_of(raw)
    cfg = arch.parse_config(raw)
    return arch, (arch.complete_config(cfg, shapes) if shapes is not None else cfg)


@pytest.mark.parametrize("name", list(tm.CONFIGS))
def test_configuration_round_trip_and_tensor_names(name):
    raw = tm.config(name)
    tensors = tm.weights(raw)
    shapes = {n: tuple(t.shape) for n, t in tensors.items()}
    arch, cfg = _config(raw, shapes)
    assert arch.name == "Tilulorn"
    again = arch.complete_config(arch.parse_config(json.loads(json.dumps(cfg.to_dict()))), shapes)
    assert again == cfg
    expected, optional = arch.tensor_names(cfg.to_spec(), set(shapes))
    assert {n: tuple(s) for n, s in expected.items()} == shapes and not optional
    assert "tilulorn" in arch.info(cfg.to_spec())


def test_the_run_order_of_passes_and_where_the_stream_is_made_anew():
    raw = tm.config("A")
    _, cfg = _config(raw, {n: t.shape for n, t in tm.weights(raw).items()})
    assert cfg.run_order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    spec = cfg.to_spec()
    assert [(e.layer, e.inject) for e in spec.schedule] == cfg.run_order()
    assert all(e.source is None for e in spec.schedule) and spec.frame_spec.passes == 2
    assert plain.run_order(raw) == cfg.run_order()
    # a single pass still makes the stream anew; no loop: no such entry and no such tensors
    raw = tm.config("D")
    _, cfg = _config(raw, {n: t.shape for n, t in tm.weights(raw).items()})
    assert cfg.run_order() == [(0, None), (1, 0), (2, None)]
    raw = tm.config("B")
    _, cfg = _config(raw, {n: t.shape for n, t in tm.weights(raw).items()})
    assert all(e.inject is None for e in cfg.to_spec().schedule) and cfg.to_spec().frame_spec.passes == 0
    expected, _ = _config(raw)[0].tensor_names(cfg.to_spec(), None)
    assert "loop.in" not in expected and "loop.step" not in expected


@pytest.mark.parametrize("change,message", [
    (lambda r: r["layers"][0].update(type="mamba"), "type"),
    (lambda r: r["layers"][2]["mixer"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][2]["mixer"].update(vdim=8), "vdim"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=7), "even"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=10), "at most"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=6), "more than"),
    (lambda r: r["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda r: r["loop"].update(stop=9), "loop"),
    (lambda r: r["loop"].update(times=0), "times"),
    (lambda r: r["norm"].pop("eps"), "eps"),
    (lambda r: r["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
])
def test_configurations_that_are_refused(change, message):
    from abacus_b200.config.registry import ConfigError
    raw = tm.config("A")
    change(raw)
    with pytest.raises(ConfigError, match=message):
        _config(raw)


def test_the_decays_inner_size_comes_from_the_tensors():
    from abacus_b200.config.registry import ConfigError
    raw = tm.config("A")
    arch, cfg = _config(raw)
    with pytest.raises(ConfigError, match="inner size"):
        cfg.to_spec()
    with pytest.raises(ConfigError, match="l0.mix.w1"):
        arch.complete_config(cfg, {})
    done = arch.complete_config(cfg, {"l0.mix.w1": (5, 64), "l3.mix.w1": (11, 64)})
    assert [l.mixer.decay_rank for l in done.layers if l.type == "wkv"] == [5, 11]


@pytest.mark.parametrize("rot", [tm.rot(10000.0, 16), tm.rot(30000.0, 64, 3.0), tm.rot(50000.0, 16, 8.0, 1024, 16.0, 2.0),
                                 tm.rot(500.0, 8, 2.0, 16, 2.0, 0.5), tm.rot(1e6, 32, 8.0, 4096, 32.0, 1.0)])
def test_the_tables_of_scaled_frequencies(rot):
    """The position part's tables against the frequencies written out here: plain, all slowed by a factor, and blended
    pair by pair between slowed and plain with cosines and sines enlarged."""
    import torch
    from abacus_b200.config.tilulorn import TilulornRotation
    from abacus_b200.parts import POSITIONS
    part = POSITIONS.build(TilulornRotation.from_dict("rot.", rot, rot["dims"]).to_spec("half"))
    cos, sin = part.tables(300, torch.device("cpu"))
    f, mag = plain.frequencies(rot)
    angle = np.arange(300)[:, None] * f[None, :]
    np.testing.assert_allclose(cos.numpy(), np.cos(angle) * mag, atol=2e-7 * mag)
    np.testing.assert_allclose(sin.numpy(), np.sin(angle) * mag, atol=2e-7 * mag)
    i = np.arange(rot["dims"] // 2)
    base = rot["base"] ** (-2.0 * i / rot["dims"])
    sc = rot.get("scaling")
    if sc is None:
        assert mag == 1.0 and np.allclose(f, base)
    elif "original" not in sc:
        assert mag == 1.0 and np.allclose(f, base / sc["factor"])
    else:
        assert mag == pytest.approx(0.1 * np.log(sc["factor"]) + 1.0)
        assert np.all(f <= base * (1 + 1e-12)) and np.all(f >= base / sc["factor"] * (1 - 1e-12))
        # a pair that makes more than `fast` turns over the original context keeps its frequency; one that makes fewer
        # than `slow` is slowed whole
        turns = sc["original"] * base / (2 * np.pi)
        assert np.allclose(f[turns > sc["fast"] * rot["base"] ** (2.0 / rot["dims"])], base[turns > sc["fast"] * rot["base"] ** (2.0 / rot["dims"])])
        assert np.allclose(f[turns < sc["slow"] / rot["base"] ** (2.0 / rot["dims"])], (base / sc["factor"])[turns < sc["slow"] / rot["base"] ** (2.0 / rot["dims"])])


def test_the_plain_wkv_against_its_sum_over_the_past():
    """o_t = sum_{s<t} (r_t . (prod_{s<j<t} w_j) k_s) v_s + (r_t . u k_t) v_t, and a state carried in portions."""
    rng = np.random.default_rng(0)
    d, H, K, T = 12, 2, 3, 9
    m = {"heads": H, "dim": K}
    w = {"mu." + s: rng.uniform(0, 1, d) for s in "rkvgw"}
    w.update({s: rng.standard_normal((H * K, d)) for s in "rkvg"})
    w.update(w1=rng.standard_normal((4, d)), w2=rng.standard_normal((H * K, 4)), w0=rng.uniform(-3, 0, H * K),
             u=rng.standard_normal((H, K)), norm=np.ones(H * K), o=np.eye(H * K))
    h = rng.standard_normal((T, d))
    out, state = plain.wkv(h, m, w, 1e-6, None)
    shifted = np.concatenate([np.zeros((1, d)), h[:-1]])
    mix = {s: h + (shifted - h) * w["mu." + s] for s in "rkvgw"}
    r, k, v = ((mix[s] @ w[s].T).reshape(T, H, K) for s in "rkv")
    dec = np.exp(-np.exp(np.tanh(mix["w"] @ w["w1"].T) @ w["w2"].T + w["w0"])).reshape(T, H, K)
    o = np.zeros((T, H, K))
    for t in range(T):
        for s in range(t):
            o[t] += np.einsum("hk,hk,hv->hv", r[t], np.prod(dec[s + 1:t], axis=0) * k[s], v[s])
        o[t] += np.einsum("hk,hk,hv->hv", r[t], w["u"] * k[t], v[t])
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + 1e-6)
    gate = mix["g"] @ w["g"].T
    np.testing.assert_allclose(out, o.reshape(T, -1) * gate / (1 + np.exp(-gate)), rtol=1e-9, atol=1e-9)
    a, st = plain.wkv(h[:4], m, w, 1e-6, None)
    b, st = plain.wkv(h[4:5], m, w, 1e-6, st)
    c, st = plain.wkv(h[5:], m, w, 1e-6, st)
    np.testing.assert_allclose(np.concatenate([a, b, c]), out, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(st[1], state[1], rtol=1e-12)


def test_the_plain_window_the_sink_and_values_that_are_keys():
    rng = np.random.default_rng(1)
    d, H, G, K, T = 10, 2, 1, 4, 12
    m = {"heads": H, "kv_heads": G, "dim": K, "scale": 0.5, "mask": {"size": 3}}
    w = {"q": rng.standard_normal((H * K, d)), "k": rng.standard_normal((G * K, d)), "q.norm": np.ones(H * K),
         "k.norm": np.ones(G * K), "sink": np.array([-50.0, 2.0]), "g": np.zeros((H, d)), "o": np.eye(H * K)}
    h = rng.standard_normal((T, d))
    out, _ = plain.window_attention(h, m, w, 1e-6, None)
    values = h @ w["k"].T
    # the first token sees itself alone: head 0 (no sink to speak of) returns its value, the key as projected, halved by
    # the gate; head 1 shares the weight with its sink
    np.testing.assert_allclose(out[0, :K], 0.5 * values[0], rtol=1e-9)
    assert np.all(np.abs(out[0, K:]) < np.abs(0.5 * values[0]) - 1e-9) or np.allclose(values[0], 0)
    # a token far back does not count: changing it leaves later outputs alone, changing one inside the window does not
    other = h.copy()
    other[5] += 1.0
    moved, _ = plain.window_attention(other, m, w, 1e-6, None)
    assert np.allclose(moved[8:], out[8:]) and not np.allclose(moved[7], out[7])
    # q and k are normed over all heads at once: scaling one head's rows of Wq changes the other head's scores
    w2 = dict(w, q=w["q"] * np.repeat([3.0, 1.0], K)[:, None])
    scaled, _ = plain.window_attention(h, m, w2, 1e-6, None)
    assert not np.allclose(scaled[5, K:], out[5, K:])


def test_the_plain_latent_form_against_keys_in_full_size_and_experts_by_table():
    rng = np.random.default_rng(2)
    d, T = 16, 7
    m = {"heads": 2, "dim": 4, "rot_dim": 4, "vdim": 3, "kv_rank": 5, "q_rank": 6, "scale": 0.4, "rot": tm.rot(100.0, 4, 2.0, 8, 4.0, 1.0)}
    w = {"dq": rng.standard_normal((6, d)), "dq.norm": np.ones(6), "uq": rng.standard_normal((16, 6)),
         "dkv": rng.standard_normal((9, d)), "dkv.norm": np.ones(5), "uk": rng.standard_normal((8, 5)),
         "uv": rng.standard_normal((6, 5)), "g": rng.standard_normal((2, d)), "o": np.eye(6)}
    h = rng.standard_normal((T, d))
    out, state = plain.latent_attention(h, m, w, 1e-6, None)
    a, st = plain.latent_attention(h[:3], m, w, 1e-6, None)
    b, st = plain.latent_attention(h[3:], m, w, 1e-6, st)
    np.testing.assert_allclose(np.concatenate([a, b]), out, rtol=1e-10, atol=1e-12)
    # the first token's output is its own value, gated
    c = plain.rms_norm((h @ w["dkv"].T)[:1, :5], np.ones(5), 1e-6)
    gate = 1 / (1 + np.exp(-(h[:1] @ w["g"].T)))
    np.testing.assert_allclose(out[0], ((c @ w["uv"].T).reshape(2, 3) * gate.reshape(2, 1)).reshape(-1), rtol=1e-9)
    # experts by table: a token's output depends on its id alone, through the table
    mlp = tm.experts(3, 2, 4)
    ew = {f"e{e}.{s}": rng.standard_normal((4, d) if s != "down" else (d, 4)) for e in range(3) for s in ("gate", "up", "down")}
    ew["table"] = np.array([[0, 1], [2, 0], [1, 2]])
    x = rng.standard_normal((3, d))
    got = plain.table_experts(np.stack([x[0], x[0], x[0]]), [0, 1, 2], mlp, ew)
    def one(e):
        z = ew[f"e{e}.gate"] @ x[0]
        return ew[f"e{e}.down"] @ (z / (1 + np.exp(-z)) * (ew[f"e{e}.up"] @ x[0]))
    np.testing.assert_allclose(got, [(one(0) + one(1)) / 2, (one(2) + one(0)) / 2, (one(1) + one(2)) / 2], rtol=1e-10)
