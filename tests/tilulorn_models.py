"""Small Tilulorn models for the tests: configurations that differ in every size and option, and random weights made
here (numpy, bfloat16-representable), written as a model folder."""
import json
import os

import numpy as np
import torch


def bf16_round(a):
    """float32 values rounded to the nearest bfloat16 (ties to even), kept as float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).reshape(a.shape)


def rot(base, dims, factor=None, original=None, fast=None, slow=None):
    r = {"base": base, "dims": dims}
    if factor is not None:
        r["scaling"] = {"factor": factor}
        if original is not None:
            r["scaling"].update(original=original, fast=fast, slow=slow)
    return r


def latent_layer(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rotation, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}
    if rotation is not None:
        m["rot"] = rotation
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def window_layer(heads, kv_heads, dim, scale, window, rotation, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rotation is not None:
        m["rot"] = rotation
    return {"type": "attention", "mixer": m, "mlp": mlp}


def wkv_layer(heads, dim, mlp=None):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


def experts(n, top, ff):
    return {"kind": "moe", "router": {"experts": n, "top": top}, "expert": {"ff": ff}}


# A: a wkv layer first; layers 1 and 2 gone through twice; blended frequencies over the whole rotated part of the latent
#    layer, slowed frequencies over half of each head of the windowed layer; a window of 40 (inside a page); grouped
#    heads; two of five experts, all three of three, none.
# B: what the options leave out: no loop, no window, no scaling of the frequencies, no rotation at all in one latent
#    layer, as many key heads as query heads, a single head, one expert of one; sizes that fit no vector (heads of 10
#    with 6 rotated, values of 7, 21 latents, 9 query latents, a wkv head of 5 channels, a width of 44).
# C: the loop is the whole model, three passes; windows of exactly a page and of 130; slowed frequencies in the latent
#    layer and blended ones in the windowed layer; a rotation over part of the latent's rotated part; a wkv head of 128
#    channels; one key head for six query heads.
CONFIGS = {
    "A": {"architecture": "Tilulorn", "vocab": 131, "width": 64, "norm": {"eps": 1e-5},
          "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [wkv_layer(2, 16, experts(5, 2, 24)),
                     latent_layer(3, 16, 8, 24, 24, 20, 0.2, rot(10000.0, 8, 4.0, 64, 8.0, 1.0), experts(3, 3, 16)),
                     window_layer(4, 2, 16, 0.3, 40, rot(5000.0, 8, 2.0)),
                     wkv_layer(3, 8, experts(4, 1, 12))]},
    "B": {"architecture": "Tilulorn", "vocab": 97, "width": 44, "norm": {"eps": 1e-6},
          "layers": [latent_layer(2, 10, 6, 7, 21, 9, 0.25, rot(100.0, 6), experts(1, 1, 10)),
                     window_layer(3, 3, 12, 0.28, None, rot(1000.0, 12)),
                     wkv_layer(1, 5),
                     latent_layer(1, 12, 4, 12, 16, 16, 0.3, None, experts(6, 4, 8)),
                     window_layer(1, 1, 20, 0.2, 9, None, experts(2, 2, 20))]},
    "C": {"architecture": "Tilulorn", "vocab": 77, "width": 48, "norm": {"eps": 1e-5},
          "loop": {"start": 0, "stop": 3, "times": 3},
          "layers": [window_layer(6, 1, 8, 0.35, 64, rot(20000.0, 8, 8.0, 32, 4.0, 1.0), experts(7, 3, 12)),
                     latent_layer(4, 8, 16, 8, 32, 24, 0.2, rot(10000.0, 12, 3.0)),
                     wkv_layer(1, 128, experts(2, 1, 16))]},
    "D": {"architecture": "Tilulorn", "vocab": 61, "width": 40, "norm": {"eps": 1e-5},
          "loop": {"start": 1, "stop": 2, "times": 1},
          "layers": [window_layer(2, 2, 16, 0.25, 130, rot(10000.0, 16), experts(3, 2, 8)),
                     wkv_layer(2, 40),
                     latent_layer(5, 8, 8, 16, 40, 8, 0.3, rot(500.0, 8, 2.0, 16, 2.0, 0.5), experts(9, 1, 12))]},
}


def config(name):
    return json.loads(json.dumps(CONFIGS[name]))


def weights(raw, seed=0):
    """{tensor name: float32 array of bfloat16-representable values, or an integer table} for a configuration (a dict).
    Matrices are scaled by their input size so that activations stay of order one; queries and keys are made large so that
    scores are a few units wide and a lost or extra key shows; decays are spread so that states both fade and last."""
    rng = np.random.default_rng(seed)
    d, vocab = raw["width"], raw["vocab"]
    w = {}

    def mat(n_out, n_in, gain=1.0):
        return rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in)

    def vec(n, mean=1.0, spread=0.1):
        return mean + rng.standard_normal(n) * spread
    w["embed"] = rng.standard_normal((vocab, d))
    if raw.get("loop"):
        w["loop.in"] = np.concatenate([mat(d, d, 0.8), mat(d, d, 0.6)], axis=1) * np.sqrt(2.0)
        w["loop.step"] = rng.standard_normal((raw["loop"]["times"], d)) * 0.3
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = vec(d)
        q = p + "mix."
        if layer["type"] == "latent_attention":
            H, K, R, V, rank, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w[q + "dq"], w[q + "dq.norm"], w[q + "uq"] = mat(qr, d), vec(qr), mat(H * (K + R), qr, 3.0)
            w[q + "dkv"], w[q + "dkv.norm"] = mat(rank + R, d, 1.5), vec(rank)
            w[q + "uk"], w[q + "uv"] = mat(H * K, rank, 3.0), mat(H * V, rank, 1.5)
            w[q + "g"], w[q + "o"] = mat(H, d, 2.0), mat(d, H * V, 2.0)
        elif layer["type"] == "attention":
            H, G, K = m["heads"], m["kv_heads"], m["dim"]
            w[q + "q"], w[q + "k"] = mat(H * K, d, 2.0), mat(G * K, d, 2.0)
            w[q + "q.norm"], w[q + "k.norm"] = vec(H * K, 2.0, 0.3), vec(G * K, 2.0, 0.3)
            w[q + "sink"] = rng.standard_normal(H) * 1.5
            w[q + "g"], w[q + "o"] = mat(H, d, 2.0), mat(d, H * K, 2.0)
        else:
            H, K = m["heads"], m["dim"]
            rank = int(rng.choice([3, 6, 8, 16]))  # the inner size of the decay's pair of matrices: only their shapes say it
            for s in "rkvgw":
                w[q + "mu." + s] = rng.uniform(0.0, 1.0, d)
            for s, gain in (("r", 1.5), ("k", 1.5), ("v", 1.5), ("g", 2.0)):
                w[q + s] = mat(H * K, d, gain)
            w[q + "w1"], w[q + "w2"] = mat(rank, d, 2.0), mat(H * K, rank, 2.0)
            w[q + "w0"] = rng.uniform(-5.0, 1.0, H * K)
            w[q + "u"] = rng.standard_normal((H, K)) * 0.5
            w[q + "norm"], w[q + "o"] = vec(H * K), mat(d, H * K, 2.0)
        mlp = layer["mlp"]
        if mlp is not None:
            w[p + "norm2"] = vec(d)
            E, top, ff = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
            for e in range(E):
                w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"] = mat(ff, d, 1.5), mat(ff, d, 1.5)
                w[p + f"mlp.e{e}.down"] = mat(d, ff, 1.5)
            w[p + "mlp.table"] = np.stack([rng.permutation(E)[:top] for _ in range(vocab)]).astype(np.int32)
    w["final.norm"] = vec(d)
    w["head"] = mat(vocab, d, 2.0)
    return {n: (t if t.dtype.kind == "i" else bf16_round(t)) for n, t in w.items()}


def write_folder(tmp, name, seed=0, raw=None, tensors=None):
    """config.json and model.safetensors of configuration `name` (or of `raw`) under tmp -> (folder, config, tensors)."""
    from abacus_b200.weights.safetensors_io import save_tensors
    raw = raw if raw is not None else config(name)
    tensors = tensors if tensors is not None else weights(raw, seed)
    folder = os.path.join(str(tmp), f"tilulorn{name}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    save_tensors(os.path.join(folder, "model.safetensors"),
                 {n: torch.from_numpy(np.ascontiguousarray(t)) if t.dtype.kind == "i"
                  else torch.from_numpy(np.ascontiguousarray(t)).to(torch.bfloat16) for n, t in tensors.items()})
    return folder, raw, tensors


def random_config(rng):
    """A random configuration: two to five layers of the three mixers, experts or no feed-forward, with or without a
    loop, every kind of frequency scaling, sizes that fit and that do not fit the vector kernels."""
    def rotation(dims):
        kind = int(rng.integers(0, 4))
        base = float(rng.choice([100.0, 10000.0, 50000.0]))
        if kind == 0:
            return None
        if kind == 1:
            return rot(base, dims)
        if kind == 2:
            return rot(base, dims, float(rng.choice([1.5, 2.0, 8.0])))
        return rot(base, dims, float(rng.choice([2.0, 4.0])), int(rng.choice([16, 64, 2048])), float(rng.choice([8.0, 32.0])), 1.0)
    width = int(rng.choice([24, 40, 64, 72]))
    n_layers = int(rng.integers(2, 6))
    layers = []
    for _ in range(n_layers):
        mlp = None
        if rng.random() < 0.75:
            n = int(rng.choice([1, 2, 3, 5, 9]))
            mlp = experts(n, int(rng.integers(1, min(n, 4) + 1)), int(rng.choice([8, 12, 20])))
        kind = int(rng.integers(0, 3))
        if kind == 0:
            rd = int(rng.choice([2, 4, 8, 16]))
            layers.append(latent_layer(int(rng.choice([1, 2, 3, 5])), int(rng.choice([4, 8, 10, 16, 32])), rd,
                                       int(rng.choice([3, 8, 16, 24])), int(rng.choice([8, 21, 32, 40])),
                                       int(rng.choice([5, 8, 16, 24])), float(rng.choice([0.15, 0.3])),
                                       rotation(int(rng.choice([d for d in (2, 4, 8, 16) if d <= rd]))), mlp))
        elif kind == 1:
            G = int(rng.choice([1, 2, 3]))
            K = int(rng.choice([4, 8, 12, 16, 32]))
            layers.append(window_layer(G * int(rng.choice([1, 2, 4])), G, K, float(rng.choice([0.2, 0.35])),
                                       None if rng.random() < 0.25 else int(rng.choice([1, 5, 33, 64, 100])),
                                       rotation(int(rng.choice([d for d in (2, 4, 8, 12, 16, 32) if d <= K]))), mlp))
        else:
            layers.append(wkv_layer(int(rng.choice([1, 2, 3])), int(rng.choice([1, 5, 16, 24, 40, 100])), mlp))
    raw = {"architecture": "Tilulorn", "vocab": int(rng.choice([50, 131])), "width": width,
           "norm": {"eps": float(rng.choice([1e-6, 1e-5]))}, "layers": layers}
    if rng.random() < 0.7:
        start = int(rng.integers(0, n_layers))
        raw["loop"] = {"start": start, "stop": int(rng.integers(start + 1, n_layers + 1)), "times": int(rng.integers(1, 4))}
    return raw
