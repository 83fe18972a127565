"""Plain, slow implementation of the Tilulorn decoder, for comparison only.

numpy (float64) only, one function per mechanism, no code shared with the package under test (its own file reader).
Every function that keeps something between tokens takes and returns it as `state` (None at the start), so the same
functions serve whole prompts, portions and tokens that come one by one.

Notation: T tokens, d width, H heads, K key size, V value size.
  norm(x; w)  = x / sqrt(mean(x^2) + eps) * w
  frame:      x_0 = E[token];   logits = Wout norm(x; w_final)
  layer:      x += mixer(norm(x; w1));   x += ff(norm(x; w2))            (ff may be absent)
  loop:       layers [a, b) run n times in a row, pass t = 0 .. n - 1; before every pass x = Win [x; x_0] + step[t]
  rotation:   the pair (u, v) at position p and frequency f becomes (u cos pf - v sin pf, v cos pf + u sin pf);
              f_i = base^(-2i / dims); "half" pairs element i with i + dims / 2, "interleaved" 2i with 2i + 1;
              linear scaling divides f_i by `factor`; YaRN blends f_i / factor and f_i by a ramp over i and
              multiplies cosine and sine by 0.1 ln(factor) + 1
  latent attention: cq = norm(Wdq h; wq');  q = Wuq cq, per head [K plain | R rotated];  Wdkv h = [z | r];
              c = norm(z; wc');  k_h = [Wuk_h c | rot(r)];  v_h = Wuv_h c;  s_ij = scale q_i . k_j, j <= i;  softmax;
              o_h *= sigmoid(Wg h)_h;  out = Wo o
  attention:  q = Wq h, k = Wk h, v = k (as projected);  q and k each normed over their whole row (all heads at once),
              then rotated;  s_ij = scale q_i . k_j for 0 <= i - j < window;  the softmax's denominator also holds
              e^(sink_h);  o_h *= sigmoid(Wg h)_h;  out = Wo o
  wkv:        h' the token before (zeros at the start);  m_s = h + (h' - h) mu_s for s in r, k, v, g, w;
              r, k, v = W. m_.;  gate = silu(Wg m_g);  w = exp(-exp(W2 tanh(W1 m_w) + w0));
              per head S [K, V]:  o = (S + diag(u) k v^T)^T r;  S <- diag(w) S + k v^T
              out = Wo (wn * [o_h / rms(o_h)]_h * gate)
  experts:    token id -> `top` experts by a table, each with weight 1 / top;  expert: Wdown (silu(Wgate h) * (Wup h))
"""
import json
import math
import struct

import numpy as np


def read_safetensors(path):
    """name -> float64 array (bfloat16 widened exactly) or int array."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = raw[8 + n + a:8 + n + b]
        if info["dtype"] == "BF16":
            arr = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif info["dtype"] == "I32":
            arr = np.frombuffer(buf, dtype="<i4").astype(np.int64)
        elif info["dtype"] == "I64":
            arr = np.frombuffer(buf, dtype="<i8").astype(np.int64)
        else:
            raise ValueError(f"dtype {info['dtype']} of {name}")
        out[name] = arr.reshape(info["shape"])
    return out


def rms_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def frequencies(rot):
    """(frequency per pair [dims / 2], the factor on cosine and sine) of a rotation's description."""
    dims, base = rot["dims"], float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor = float(scaling["factor"])
    if "original" not in scaling:  # linear
        return f / factor, 1.0
    def where(turns):
        return dims * math.log(scaling["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(scaling["fast"])), 0)
    hi = min(math.ceil(where(scaling["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot, pairing):
    """x [T, ..., size]: the first rot["dims"] elements of the last axis rotated, the rest as they are."""
    dims = rot["dims"]
    f, mag = frequencies(rot)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = (np.cos(angle) * mag).reshape(shape).astype(x.dtype), (np.sin(angle) * mag).reshape(shape).astype(x.dtype)
    out = x.copy()
    if pairing == "half":
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2], out[..., dims // 2:dims] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = u * c - v * s, v * c + u * s
    return out


def softmax_rows(scores, visible, sink=None):
    """scores [H, T, S], visible [T, S] bool; sink [H] or None: one more term e^sink in every denominator."""
    s = np.where(visible[None], scores, -np.inf)
    top = s.max(axis=-1, keepdims=True)
    if sink is not None:
        top = np.maximum(top, sink[:, None, None])
    e = np.exp(s - top)
    den = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink[:, None, None] - top)
    return e / den


def latent_attention(h, m, w, eps, state):
    """h [T, d]; m: the mixer's sizes; w: its tensors by short name; state: (latents [S, rank], rotated parts [S, R])."""
    H, K, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    past = 0 if state is None else state[0].shape[0]
    positions = np.arange(past, past + T)
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, H, K + R)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    r, q_rot = down[:, rank:], q[:, :, K:]
    if m.get("rot"):
        r, q_rot = rotate(r, positions, m["rot"], "half"), rotate(q_rot, positions, m["rot"], "half")
    if state is not None:
        c, r = np.concatenate([state[0], c]), np.concatenate([state[1], r])
    k = (c @ w["uk"].T).reshape(-1, H, K)
    v = (c @ w["uv"].T).reshape(-1, H, V)
    scores = (np.einsum("thk,shk->hts", q[:, :, :K], k) + np.einsum("thr,sr->hts", q_rot, r)) * m["scale"]
    visible = np.arange(past + T)[None, :] <= positions[:, None]
    p = softmax_rows(scores, visible)
    o = np.einsum("hts,shv->thv", p, v) * sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * V) @ w["o"].T, (c, r)


def window_attention(h, m, w, eps, state):
    """state: (keys [S, G, K] normed and rotated, values [S, G, K] as projected)."""
    H, G, K = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    past = 0 if state is None else state[0].shape[0]
    positions = np.arange(past, past + T)
    q_raw, k_raw = h @ w["q"].T, h @ w["k"].T
    v = k_raw.reshape(T, G, K)
    q = rms_norm(q_raw, w["q.norm"], eps).reshape(T, H, K)
    k = rms_norm(k_raw, w["k.norm"], eps).reshape(T, G, K)
    if m.get("rot"):
        q, k = rotate(q, positions, m["rot"], "interleaved"), rotate(k, positions, m["rot"], "interleaved")
    if state is not None:
        k, v = np.concatenate([state[0], k]), np.concatenate([state[1], v])
    per = H // G
    kh, vh = np.repeat(k, per, axis=1), np.repeat(v, per, axis=1)
    scores = np.einsum("thk,shk->hts", q, kh) * m["scale"]
    back = positions[:, None] - np.arange(past + T)[None, :]
    visible = back >= 0
    if m.get("mask"):
        visible &= back < m["mask"]["size"]
    p = softmax_rows(scores, visible, w["sink"] if "sink" in w else None)
    o = np.einsum("hts,shv->thv", p, vh) * sigmoid(h @ w["g"].T)[:, :, None]
    return o.reshape(T, H * K) @ w["o"].T, (k, v)


def wkv(h, m, w, eps, state):
    """state: (the token before [d], S [H, K, K])."""
    H, K = m["heads"], m["dim"]
    T, d = h.shape
    before, S = (np.zeros(d, h.dtype), np.zeros((H, K, K), h.dtype)) if state is None else (state[0], state[1].copy())
    shifted = np.concatenate([before[None], h[:-1]])
    mix = {s: h + (shifted - h) * w["mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w["r"].T).reshape(T, H, K)
    k = (mix["k"] @ w["k"].T).reshape(T, H, K)
    v = (mix["v"] @ w["v"].T).reshape(T, H, K)
    gate = silu(mix["g"] @ w["g"].T)
    decay = np.exp(-np.exp(np.tanh(mix["w"] @ w["w1"].T) @ w["w2"].T + w["w0"])).reshape(T, H, K)
    o = np.zeros((T, H, K), h.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hk,hkv->hv", r[t], S + w["u"][:, :, None] * kv)
        S = decay[t][:, :, None] * S + kv
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps)
    return (o.reshape(T, H * K) * w["norm"] * gate) @ w["o"].T, (h[-1].copy(), S)


def table_experts(h, tokens, mlp, w):
    """Each token's experts by its id; weight 1 / top each."""
    top = mlp["router"]["top"]
    out = np.zeros_like(h)
    for t, token in enumerate(tokens):
        for e in w["table"][token]:
            g, u, dn = w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"]
            out[t] += (dn @ (silu(g @ h[t]) * (u @ h[t]))) / top
    return out


MIXERS = {"latent_attention": latent_attention, "attention": window_attention, "wkv": wkv}


def run_order(config):
    """[(layer, pass number if a pass starts right before it else None)]."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(l, None) for l in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(l, None) for l in range(a)]
    for t in range(times):
        order += [(l, t if l == a else None) for l in range(a, b)]
    return order + [(l, None) for l in range(b, n)]


def part(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


class PlainTilulorn:
    def __init__(self, config, weights, real=np.float64):
        """real: the type everything is computed in (float32: to see what float32 itself loses on an input)."""
        self.config = config
        self.w = {n: (t if t.dtype.kind == "i" else t.astype(real)) for n, t in weights.items()}
        self.eps = config["norm"]["eps"]
        self.order = run_order(config)

    @classmethod
    def from_folder(cls, folder):
        with open(f"{folder}/config.json") as f:
            config = json.load(f)
        return cls(config, read_safetensors(f"{folder}/model.safetensors"))

    def new_state(self):
        return [None] * len(self.order)

    def forward(self, tokens, state=None, streams=None):
        """tokens: the sequence's next tokens; state: what new_state() or an earlier call left (changed in place).
        Returns logits [T, vocab]. streams: a list that gets the residual stream after every layer run."""
        state = self.new_state() if state is None else state
        w, eps = self.w, self.eps
        x0 = w["embed"][np.asarray(tokens)]
        x = x0.copy()
        for run, (l, starts_pass) in enumerate(self.order):
            if starts_pass is not None:
                x = np.concatenate([x, x0], axis=1) @ w["loop.in"].T + w["loop.step"][starts_pass]
            layer, p = self.config["layers"][l], f"l{l}."
            y, state[run] = MIXERS[layer["type"]](rms_norm(x, w[p + "norm1"], eps), layer["mixer"], part(w, p + "mix."), eps, state[run])
            x = x + y
            if layer.get("mlp"):
                x = x + table_experts(rms_norm(x, w[p + "norm2"], eps), tokens, layer["mlp"], part(w, p + "mlp."))
            if streams is not None:
                streams.append(x.copy())
        return rms_norm(x, w["final.norm"], eps) @ w["head"].T
