"""Plain, slow implementation of the Linonex decoder, for comparison only.

numpy only, one function per mechanism, no code shared with the package under test (its own file reader). A sequence
is walked token by token where a mechanism is recurrent, so the same functions serve whole prompts and tokens that come
one by one: every function that keeps something between tokens takes and returns it as `state` (None at the start).

Notation: T tokens, d width, H heads, K key size, V value size.
  norm(x; w)  = x / sqrt(mean(x^2) + eps) * w
  frame:      x_0 = E[token] + P[position];   logits = Wout norm(x; w_final)
  layer:      x += mixer(norm(x; w1));   x += ff(norm(x; w2))            (ff may be absent)
  loop:       layers [a, b) run n times in a row; before every pass after the first, x += x_0
  matrix memory ("mlstm"), per head, C [K, V], n [K], m a scalar (all zero at the start):
              i = c tanh((wi . h + bi) / c);   f = logsigmoid(c tanh((wf . h + bf) / c))
              m' = max(f + m, i);   C' = e^(f + m - m') C + e^(i - m') k v^T;   n' = e^(f + m - m') n + e^(i - m') k
              o = C'^T q / (max(|n' . q|, e^(-m')) + 1e-6),   q = K^(-1/2) Wq h
              out = Wo (w * [o_h / rms(o_h)]_h * sigmoid(Wg h))
  side by side ("parallel"): out = (norm(A(h); wa) + norm(B(h); wb)) / 2, with
    A, chunked attention: q, k, v = conv(W. h);  s_ij = cap tanh(scale q_i . k_j / cap) for j <= i in i's chunk of
              `size` positions;  softmax over those j;  Wo on the heads
    B, gated delta rule: q, k, v = silu(conv(W. h));  q, k unit vectors, q times K^(-1/2);  b = sigmoid(wb . h);
              g = exp(-e^A softplus(wa . h + dt));   S <- g S;  u = b (v - S^T k);  S <- S + k u^T;  o = S^T q
              out = Wo (w * o_h / rms(o_h) * silu(Wg h))
    conv:     y_t = sum_j c[:, j] u_(t - taps + 1 + j), zeros before the sequence's start
  experts:    z = R h;  s = softmax(z);  chosen: the `top` largest of s + correction;  weight s_e * scale;
              the last `identity` router outputs stand for experts that return h itself
"""
import json
import struct

import numpy as np


def read_safetensors(path):
    """name -> float32 array (bfloat16 widened exactly) or int32 array."""
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
            arr = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4").copy()
        elif info["dtype"] == "I32":
            arr = np.frombuffer(buf, dtype="<i4").copy()
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


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def softplus(z):
    return np.logaddexp(0.0, z)


def causal_conv(u, w, state):
    """u [T, C], w [C, taps]; state: the last taps - 1 inputs [taps - 1, C] (None: zeros). -> (y, state)."""
    taps = w.shape[1]
    if state is None:
        state = np.zeros((taps - 1, u.shape[1]), dtype=u.dtype)
    full = np.concatenate([state, u], axis=0)
    y = np.zeros_like(u)
    for j in range(taps):
        y += full[j:j + u.shape[0]] * w[:, j]
    return y, full[full.shape[0] - (taps - 1):]


def matrix_memory(h, p, m, eps, state):
    """The mixer "mlstm". h [T, d]; p: its tensors by short name; m: its sizes."""
    H, K, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    T = h.shape[0]
    q = (h @ p["q"].T).reshape(T, H, K) * K ** -0.5
    k = (h @ p["k"].T).reshape(T, H, K)
    v = (h @ p["v"].T).reshape(T, H, V)
    gi = cap * np.tanh((h @ p["i"].T + p["i.b"]) / cap)
    gf = log_sigmoid(cap * np.tanh((h @ p["f"].T + p["f.b"]) / cap))
    if state is None:
        state = (np.zeros((H, K, V), h.dtype), np.zeros((H, K), h.dtype), np.zeros(H, h.dtype))
    C, n, mx = (a.copy() for a in state)
    o = np.zeros((T, H, V), h.dtype)
    for t in range(T):
        m_new = np.maximum(gf[t] + mx, gi[t])
        keep, write = np.exp(gf[t] + mx - m_new), np.exp(gi[t] - m_new)
        C = keep[:, None, None] * C + write[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + write[:, None] * k[t]
        mx = m_new
        num = np.einsum("hkv,hk->hv", C, q[t])
        den = np.maximum(np.abs(np.einsum("hk,hk->h", n, q[t])), np.exp(-mx)) + 1e-6
        o[t] = num / den[:, None]
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps)
    y = o.reshape(T, H * V) * p["norm"] * sigmoid(h @ p["g"].T)
    return y @ p["o"].T, (C, n, mx)


def chunked_attention(h, p, m, state):
    """The left side of "parallel". state: (conv tails of q, k, v; keys; values; tokens seen)."""
    H, G, K, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = m["mask"]["size"] if m.get("mask") else None   # no mask: every earlier key is seen
    cap, scale = m.get("softcap"), m["scale"]               # no cap: scores as they are
    T = h.shape[0]
    tails, keys, values, seen = state if state is not None else ((None, None, None), None, None, 0)
    q, k, v = h @ p["q"].T, h @ p["k"].T, h @ p["v"].T
    tq = tk = tv = None
    if "q.conv" in p:                                       # no taps: the projections as they are
        q, tq = causal_conv(q, p["q.conv"], tails[0])
        k, tk = causal_conv(k, p["k.conv"], tails[1])
        v, tv = causal_conv(v, p["v.conv"], tails[2])
    k, v = k.reshape(T, G, K), v.reshape(T, G, V)
    keys = k if keys is None else np.concatenate([keys, k], axis=0)
    values = v if values is None else np.concatenate([values, v], axis=0)
    q = q.reshape(T, H, K)
    out = np.zeros((T, H, V), h.dtype)
    for t in range(T):
        i = seen + t
        first = (i // size) * size if size else 0
        for a in range(H):
            g = a // (H // G)
            s = keys[first:i + 1, g] @ q[t, a] * scale
            if cap:
                s = cap * np.tanh(s / cap)
            w = np.exp(s - s.max())
            out[t, a] = (w / w.sum()) @ values[first:i + 1, g]
    return out.reshape(T, H * V) @ p["o"].T, ((tq, tk, tv), keys, values, seen + T)


def scalar_delta_rule(h, p, m, eps, state):
    """The right side of "parallel": the gated delta rule with one decay per head."""
    H, G, K, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    tails, S = state if state is not None else ((None, None, None), np.zeros((H, K, V), h.dtype))
    q, tq = causal_conv(h @ p["q"].T, p["q.conv"], tails[0])
    k, tk = causal_conv(h @ p["k"].T, p["k.conv"], tails[1])
    v, tv = causal_conv(h @ p["v"].T, p["v.conv"], tails[2])
    q, k, v = silu(q).reshape(T, G, K), silu(k).reshape(T, G, K), silu(v).reshape(T, H, V)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * K ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ p["b"].T)
    decay = np.exp(-np.exp(p["A_log"]) * softplus(h @ p["a"].T + p["dt_bias"]))
    S = S.copy()
    o = np.zeros((T, H, V), h.dtype)
    for t in range(T):
        for a in range(H):
            g = a // (H // G)
            S[a] *= decay[t, a]
            u = beta[t, a] * (v[t, a] - S[a].T @ k[t, g])
            S[a] += np.outer(k[t, g], u)
            o[t, a] = S[a].T @ q[t, g]
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps) * p["norm"]
    y = o.reshape(T, H * V) * silu(h @ p["g"].T)
    return y @ p["o"].T, ((tq, tk, tv), S)


def side_by_side(h, p, m, eps, state):
    """The mixer "parallel": both sides read h; their outputs are normed over the width and averaged."""
    left = {n[5:]: t for n, t in p.items() if n.startswith("left.")}
    right = {n[6:]: t for n, t in p.items() if n.startswith("right.")}
    sl, sr = state if state is not None else (None, None)
    a, sl = chunked_attention(h, left, m["left"], sl)
    b, sr = scalar_delta_rule(h, right, m["right"], eps, sr)
    return 0.5 * (rms_norm(a, left["out"], eps) + rms_norm(b, right["out"], eps)), (sl, sr)


def gated_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def routed_ff(h, p, mlp):
    r = mlp["router"]
    n_real, top, scale, ident = r["experts"], r["top"], r.get("scale", 1.0), r.get("identity", 0)
    z = h @ p["router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=-1, keepdims=True)
    assert s.shape[1] == n_real + ident
    choice = s + p["correction"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in np.argsort(-choice[t], kind="stable")[:top]:
            w = s[t, e] * scale
            if e >= n_real:
                out[t] += w * h[t]
            else:
                out[t] += w * gated_ff(h[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    return out


def feed_forward(h, p, mlp):
    if mlp["kind"] == "dense":
        return gated_ff(h, p["gate"], p["up"], p["down"])
    return routed_ff(h, p, mlp)


def run_order(config):
    """[(layer, pass of the loop, first of its pass)] in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(l, 0, False) for l in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(l, 0, False) for l in range(a)]
    for k in range(times):
        order += [(l, k, l == a and k > 0) for l in range(a, b)]
    return order + [(l, 0, False) for l in range(b, n)]


class Plain:
    """A sequence's model: feed(tokens) runs the next tokens and returns (logits [T, vocab], the stream after every
    layer run [runs, T, d])."""

    def __init__(self, config, tensors, real=np.float64):
        self.config, self.real = config, real
        self.w = {n: (t.astype(real) if t.dtype.kind == "f" else t) for n, t in tensors.items()}
        self.eps = config["norm"]["eps"]
        self.order = run_order(config)
        self.states = [None] * len(self.order)
        self.seen = 0

    def part(self, prefix):
        return {n[len(prefix):]: t for n, t in self.w.items() if n.startswith(prefix)}

    def feed(self, tokens):
        w, eps = self.w, self.eps
        tokens = np.asarray(tokens)
        T = len(tokens)
        x = w["embed"][tokens] + w["pos"][self.seen:self.seen + T]
        x0 = x.copy()
        after = []
        for run, (l, _, again) in enumerate(self.order):
            layer = self.config["layers"][l]
            if again:
                x = x + x0
            h = rms_norm(x, w[f"l{l}.norm1"], eps)
            mix = self.part(f"l{l}.mix.")
            if layer["type"] == "mlstm":
                y, self.states[run] = matrix_memory(h, mix, layer["mixer"], eps, self.states[run])
            elif layer["type"] == "parallel":
                y, self.states[run] = side_by_side(h, mix, layer["mixer"], eps, self.states[run])
            else:
                raise ValueError(layer["type"])
            x = x + y
            if layer.get("mlp") is not None:
                x = x + feed_forward(rms_norm(x, w[f"l{l}.norm2"], eps), self.part(f"l{l}.mlp."), layer["mlp"])
            after.append(x.copy())
        self.seen += T
        logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
        return logits, np.stack(after)
