"""Small Linonex models for the tests: configurations that differ in every size and option, and random weights made
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


def memory_layer(heads, dim, vdim, cap, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def left(heads, kv_heads, dim, vdim, scale, conv=0, chunk=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if softcap is not None:
        m["softcap"] = softcap
    return m


def right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel_layer(l, r, mlp=None):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def experts(n, identity, top, scale, ff):
    return {"kind": "moe", "router": {"experts": n, "identity": identity, "top": top, "scale": scale}, "expert": {"ff": ff}}


# P: a parallel layer first, and the first two layers gone through three times (the loop starts at layer 0): grouped
#    heads on both sides, values smaller than keys on the left and larger on the right, two and three taps, chunks of 48
#    positions (no multiple or divisor of a page); a memory layer with values larger than keys, three of six router
#    outputs chosen, one of them an expert that returns its input; a memory layer with sizes that fit no vector and no
#    feed-forward; a parallel layer with chunks of 7, four taps, one key head for both delta heads, one expert of three.
# Q: what the options leave out: attention without convolution, chunks or a cap; no loop; every router output chosen, two
#    of three returning their input; a single head everywhere in the last layer; a scale of 1 on the experts' weights.
# R: the loop is the whole model; chunks of exactly a page and of 130; a memory head of 200 key channels with 133
#    values; a delta head of 128 key channels; five taps.
CONFIGS = {
    "P": {"architecture": "Linonex", "vocab": 131, "width": 64, "norm": {"eps": 1e-5}, "max_positions": 512,
          "loop": {"start": 0, "stop": 2, "times": 3},
          "layers": [parallel_layer(left(4, 2, 16, 8, 0.25, 2, 48, 20.0), right(4, 2, 8, 16, 3), dense(96)),
                     memory_layer(2, 24, 40, 15.0, experts(5, 1, 3, 2.0, 24)),
                     memory_layer(3, 5, 3, 8.0),
                     parallel_layer(left(3, 3, 10, 7, 0.3, 4, 7, 5.0), right(2, 1, 20, 6, 2), experts(3, 0, 1, 0.5, 12))]},
    "Q": {"architecture": "Linonex", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "max_positions": 300,
          "layers": [memory_layer(1, 16, 16, 10.0, experts(1, 2, 3, 1.0, 8)),
                     parallel_layer(left(6, 1, 8, 8, 0.35), right(3, 3, 16, 8, 4), dense(40)),
                     parallel_layer(left(1, 1, 24, 12, 0.2, 3, None, 9.0), right(1, 1, 12, 24, 2))]},
    "R": {"architecture": "Linonex", "vocab": 77, "width": 40, "norm": {"eps": 1e-5}, "max_positions": 400,
          "loop": {"start": 0, "stop": 3, "times": 2},
          "layers": [parallel_layer(left(2, 1, 32, 16, 0.18, 5, 64, 12.0), right(2, 2, 128, 8, 5), experts(8, 3, 4, 1.5, 16)),
                     memory_layer(1, 200, 133, 6.0, dense(24)),
                     parallel_layer(left(2, 2, 8, 24, 0.4, 2, 130, 50.0), right(4, 2, 8, 8, 3))]},
}


def config(name):
    return json.loads(json.dumps(CONFIGS[name]))


def weights(raw, seed=0):
    """{tensor name: float32 array of bfloat16-representable values} for a configuration (a dict). Matrices are scaled by
    their input size so that activations stay of order one; queries and keys are made large so that scores are a few
    units wide and a lost or extra key shows; gates and decays are spread so that states both fade and last."""
    rng = np.random.default_rng(seed)
    d = raw["width"]
    w = {}

    def mat(n_out, n_in, gain=1.0):
        return rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in)

    def vec(n, mean=1.0, spread=0.1):
        return mean + rng.standard_normal(n) * spread
    w["embed"] = rng.standard_normal((raw["vocab"], d))
    w["pos"] = rng.standard_normal((raw["max_positions"], d)) * 0.5
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = vec(d)
        if layer["type"] == "mlstm":
            H, K, V = m["heads"], m["dim"], m["vdim"]
            for t, rows, gain in (("q", H * K, 2.0), ("k", H * K, 2.0), ("v", H * V, 1.5), ("g", H * V, 1.5)):
                w[p + "mix." + t] = mat(rows, d, gain)
            w[p + "mix.i"], w[p + "mix.f"] = mat(H, d, 3.0), mat(H, d, 3.0)
            w[p + "mix.i.b"], w[p + "mix.f.b"] = vec(H, 0.0, 1.0), vec(H, 2.0, 1.5)
            w[p + "mix.norm"] = vec(H * V)
            w[p + "mix.o"] = mat(d, H * V, 2.0)
        else:
            a, r = m["left"], m["right"]
            q = p + "mix.left."
            H, G, K, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = mat(H * K, d, 3.0), mat(G * K, d, 3.0), mat(G * V, d, 1.5)
            if a.get("conv"):
                for t, rows in (("q", H * K), ("k", G * K), ("v", G * V)):
                    w[q + t + ".conv"] = rng.standard_normal((rows, a["conv"])) * 0.6
            w[q + "o"], w[q + "out"] = mat(d, H * V, 2.0), vec(d)
            q = p + "mix.right."
            H, G, K, V = r["heads"], r["kv_heads"], r["dim"], r["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = mat(G * K, d, 2.0), mat(G * K, d, 2.0), mat(H * V, d, 1.5)
            for t, rows in (("q", G * K), ("k", G * K), ("v", H * V)):
                w[q + t + ".conv"] = rng.standard_normal((rows, r["conv"])) * 0.6
            w[q + "b"], w[q + "a"] = mat(H, d, 2.0), mat(H, d, 2.0)
            w[q + "A_log"], w[q + "dt_bias"] = vec(H, -1.0, 1.0), vec(H, 0.0, 1.0)
            w[q + "g"], w[q + "norm"] = mat(H * V, d, 1.5), vec(V)
            w[q + "o"], w[q + "out"] = mat(d, H * V, 2.0), vec(d)
        mlp = layer["mlp"]
        if mlp is not None:
            w[p + "norm2"] = vec(d)
            if mlp["kind"] == "dense":
                w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(mlp["ff"], d), mat(mlp["ff"], d), mat(d, mlp["ff"], 2.0)
            else:
                n_out = mlp["router"]["experts"] + mlp["router"].get("identity", 0)
                w[p + "mlp.router"] = mat(n_out, d, 3.0)
                w[p + "mlp.correction"] = rng.standard_normal(n_out) * 0.2
                for e in range(mlp["router"]["experts"]):
                    ff = mlp["expert"]["ff"]
                    w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"] = mat(ff, d, 1.5), mat(ff, d, 1.5)
                    w[p + f"mlp.e{e}.down"] = mat(d, ff, 1.5)
    w["final.norm"] = vec(d)
    w["head"] = mat(raw["vocab"], d, 2.0)
    return {n: bf16_round(t) for n, t in w.items()}


def write_folder(tmp, name, seed=0, raw=None, tensors=None):
    """config.json and model.safetensors of configuration `name` (or of `raw`) under tmp -> (folder, config, tensors)."""
    from abacus_b200.weights.safetensors_io import save_tensors
    raw = raw if raw is not None else config(name)
    tensors = tensors if tensors is not None else weights(raw, seed)
    folder = os.path.join(str(tmp), f"linonex{name}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    save_tensors(os.path.join(folder, "model.safetensors"),
                 {n: torch.from_numpy(np.ascontiguousarray(t)).to(torch.bfloat16) for n, t in tensors.items()})
    return folder, raw, tensors


def random_config(rng):
    """A random configuration: two to four layers of either mixer, every kind of feed-forward or none, with or without a
    loop, sizes that fit and that do not fit the vector kernels."""
    width = int(rng.choice([24, 40, 64, 72]))
    n_layers = int(rng.integers(2, 5))
    layers = []
    for _ in range(n_layers):
        r = rng.random()
        if r < 0.25:
            mlp = None
        elif r < 0.5:
            mlp = dense(int(rng.choice([16, 24, 40])))
        else:
            n, ident = int(rng.choice([1, 2, 3, 5, 9])), int(rng.choice([0, 1, 2]))
            mlp = experts(n, ident, int(rng.integers(1, min(n + ident, 4) + 1)), float(rng.choice([0.5, 1.0, 2.5])),
                          int(rng.choice([8, 12, 20])))
        if rng.random() < 0.5:
            layers.append(memory_layer(int(rng.choice([1, 2, 3, 5])), int(rng.choice([1, 5, 16, 24, 40, 100])),
                                       int(rng.choice([1, 3, 8, 20, 33])), float(rng.choice([4.0, 10.0, 15.0])), mlp))
        else:
            G = int(rng.choice([1, 2, 3]))
            a = left(G * int(rng.choice([1, 2, 4])), G, int(rng.choice([4, 8, 12, 16, 32])), int(rng.choice([3, 8, 16, 24])),
                     float(rng.choice([0.2, 0.35])), int(rng.choice([0, 2, 3, 4])),
                     None if rng.random() < 0.2 else int(rng.choice([1, 5, 33, 64, 100])),
                     None if rng.random() < 0.2 else float(rng.choice([3.0, 15.0, 50.0])))
            G = int(rng.choice([1, 2]))
            b = right(G * int(rng.choice([1, 2, 3])), G, int(rng.choice([4, 8, 20, 32, 72])), int(rng.choice([3, 8, 16, 40])),
                      int(rng.choice([1, 2, 4])))
            layers.append(parallel_layer(a, b, mlp))
    raw = {"architecture": "Linonex", "vocab": int(rng.choice([50, 131])), "width": width,
           "norm": {"eps": float(rng.choice([1e-6, 1e-5]))}, "max_positions": 256, "layers": layers}
    if rng.random() < 0.7:
        start = int(rng.integers(0, n_layers))
        raw["loop"] = {"start": start, "stop": int(rng.integers(start + 1, n_layers + 1)), "times": int(rng.integers(2, 4))}
    return raw
