"""A plain, slow implementation of the Fimudra decoder in NumPy float64: one function per
mechanism, whole sequences at once, no cache, token-by-token recurrences. It shares no code
with the library and is the oracle of the library's tests.

The design: token embedding times a constant; ``streams`` copies of the residual that every
sublayer reads a weighted sum of and writes back into through a small mixing matrix
(hyper-connections); layer norms without bias; two kinds of mixer: ``wkv`` (token-shifted
projections, a decay per key channel from a low-rank product, a matrix state per head with a
bonus for the current token) and ``parallel`` (grouped-query attention with a sink in the
softmax, partly rotated heads and Llama-3.1 frequency scaling, beside a matrix memory with
exponential gates and a running maximum); a feed-forward of routed experts with identity
experts, a correction on the choice only and a shared expert; a layer may use another layer's
weights; the head is the embedding table.

``weights``: a dict name -> float64 array. ``config``: the dict of config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np


# ---------------------------------------------------------------------------- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis, no bias."""
    mu = np.mean(x, axis=-1, keepdims=True)
    var = np.mean((x - mu) ** 2, axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


# ---------------------------------------------------------------------------- positions
def rotary_frequencies(rot: Dict) -> np.ndarray:
    """dims/2 angular frequencies base^(-2i/dims); with ``scaling`` the long wavelengths are
    slowed by ``factor``, the short ones kept and those between blended linearly in
    original/wavelength."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high = float(sc["factor"]), float(sc["low"]), float(sc["high"])
    original = float(sc["original"])
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            out[i] = fi
        elif wavelength > original / low:
            out[i] = fi / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate(x, positions, freqs, dims):
    """x [T, heads, dim]: value i of the first ``dims`` turns with value i + dims/2."""
    half = dims // 2
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]      # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


# ---------------------------------------------------------------------------- mixers
def sink_attention(h, W, p: Dict, pre: str, positions) -> np.ndarray:
    """Causal grouped-query attention whose softmax denominator also holds exp(sink) per head."""
    T = h.shape[0]
    H, G, dim, vdim = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
    q = (h @ W[pre + "q"].T).reshape(T, H, dim)
    k = (h @ W[pre + "k"].T).reshape(T, G, dim)
    v = (h @ W[pre + "v"].T).reshape(T, G, vdim)
    rot = p.get("rot")
    if rot and int(rot["dims"]) > 0:
        f = rotary_frequencies(rot)
        q, k = rotate(q, positions, f, int(rot["dims"])), rotate(k, positions, f, int(rot["dims"]))
    sink = W[pre + "sink"]
    out = np.zeros((T, H, vdim))
    per = H // G
    for hd in range(H):
        g = hd // per
        for t in range(T):
            s = (k[:t + 1, g] @ q[t, hd]) * float(p["scale"])
            m = max(s.max(), sink[hd])
            e = np.exp(s - m)
            out[t, hd] = (e @ v[:t + 1, g]) / (e.sum() + math.exp(sink[hd] - m))
    return out.reshape(T, H * vdim) @ W[pre + "o"].T


def matrix_memory(h, W, p: Dict, pre: str, eps: float) -> np.ndarray:
    """The matrix memory with exponential input gate, sigmoid forget gate (both in logarithms,
    softly capped) and a running maximum that starts at 0."""
    T = h.shape[0]
    H, dim, vdim, cap = int(p["heads"]), int(p["dim"]), int(p["vdim"]), float(p["gate_cap"])
    q = (h @ W[pre + "q"].T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ W[pre + "k"].T).reshape(T, H, dim)
    v = (h @ W[pre + "v"].T).reshape(T, H, vdim)
    gi = cap * np.tanh((h @ W[pre + "i"].T + W[pre + "i.b"]) / cap)                 # [T, H]
    gf = log_sigmoid(cap * np.tanh((h @ W[pre + "f"].T + W[pre + "f.b"]) / cap))
    out = np.zeros((T, H, vdim))
    for hd in range(H):
        S, n, m = np.zeros((dim, vdim)), np.zeros(dim), 0.0
        for t in range(T):
            m_new = max(gf[t, hd] + m, gi[t, hd])
            a, b = math.exp(gf[t, hd] + m - m_new), math.exp(gi[t, hd] - m_new)
            S = a * S + b * np.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            m = m_new
            out[t, hd] = (S.T @ q[t, hd]) / (max(abs(n @ q[t, hd]), math.exp(-m)) + 1e-6)
    out = unit_rms(out, eps).reshape(T, H * vdim) * W[pre + "norm"]
    out = out * sigmoid(h @ W[pre + "g"].T)
    return out @ W[pre + "o"].T


def parallel_mixer(h, W, p: Dict, pre: str, eps: float, positions) -> np.ndarray:
    left = sink_attention(h, W, p["left"], pre + "left.", positions)
    right = matrix_memory(h, W, p["right"], pre + "right.", eps)
    return float(p["left_scale"]) * left + float(p["right_scale"]) * right


def wkv_mixer(h, W, p: Dict, pre: str, eps: float) -> np.ndarray:
    """Token-shifted time mixing with a decaying matrix state per head."""
    T = h.shape[0]
    H, dim = int(p["heads"]), int(p["dim"])
    prev = np.vstack([np.zeros((1, h.shape[1])), h[:-1]])
    mix = {s: h + (prev - h) * W[pre + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ W[pre + "r"].T).reshape(T, H, dim)
    k = (mix["k"] @ W[pre + "k"].T).reshape(T, H, dim)
    v = (mix["v"] @ W[pre + "v"].T).reshape(T, H, dim)
    gate = silu(mix["g"] @ W[pre + "g"].T)
    lw = np.tanh(mix["w"] @ W[pre + "w1"].T) @ W[pre + "w2"].T + W[pre + "w0"]
    w = np.exp(-np.exp(lw)).reshape(T, H, dim)
    u = W[pre + "u"].reshape(H, dim)
    out = np.zeros((T, H, dim))
    for hd in range(H):
        S = np.zeros((dim, dim))
        for t in range(T):
            kv = np.outer(k[t, hd], v[t, hd])
            out[t, hd] = (S + u[hd][:, None] * kv).T @ r[t, hd]
            S = w[t, hd][:, None] * S + kv
    out = unit_rms(out, eps).reshape(T, H * dim) * W[pre + "norm"] * gate
    return out @ W[pre + "o"].T


# ---------------------------------------------------------------------------- feed-forward
def clamped_expert(h, W, pre: str, limit: float) -> np.ndarray:
    g = np.minimum(h @ W[pre + "gate"].T, limit)
    u = np.clip(h @ W[pre + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[pre + "down"].T


def route(h, W, mlp: Dict, pre: str):
    """(chosen experts [T, top], their weights [T, top], the margin between the last chosen and
    the best not chosen choice score [T])."""
    r = mlp["router"]
    top = int(r["top"])
    z = h @ W[pre + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(axis=-1, keepdims=True)
    choice = s + W[pre + "correction"]
    if int(r.get("identity") or 0) + int(r["experts"]) != choice.shape[1]:
        raise ValueError("the router's outputs are not experts + identity")
    order = np.argsort(-choice, axis=-1, kind="stable")
    ids = order[:, :top]
    w = np.take_along_axis(s, ids, axis=-1) * float(r.get("scale", 1.0))
    ranked = np.take_along_axis(choice, order, axis=-1)
    margin = (ranked[:, top - 1] - ranked[:, top]) if choice.shape[1] > top else \
        np.full(h.shape[0], np.inf)
    return ids, w, margin


class Routing:
    """What a test wants to know of the routers' choices, or to settle about them.

    ``margins[(layer, t)]``: how far the last chosen choice score of token t in layer ``layer``
    lies above the first one left out, in units of the root mean square of the token's
    scores. ``forced[(layer, t)]``: the experts that another implementation chose there; they
    replace the plain choice where the two differ and the margin is below ``close`` (a
    computation in 16 bits may fall on either side of such a call); where the margin is larger
    the difference is an error."""

    def __init__(self, forced=None, close: float = 0.12):
        self.forced = forced or {}
        self.close = close
        self.margins: Dict = {}
        self.replaced: List = []

    def choose(self, layer, ids, w, margin, weights):
        ids, w = ids.copy(), w.copy()
        for t in range(ids.shape[0]):
            self.margins[(layer, t)] = float(margin[t])
            theirs = self.forced.get((layer, t))
            if theirs is not None and set(int(e) for e in theirs) != set(ids[t].tolist()):
                if margin[t] >= self.close:
                    raise AssertionError(
                        f"layer {layer}, token {t}: experts {sorted(theirs)} were chosen, "
                        f"{sorted(ids[t].tolist())} expected, at a margin of {margin[t]:.3g}")
                ids[t] = [int(e) for e in theirs]
                w[t] = weights[t, ids[t]]
                self.replaced.append((layer, t))
        return ids, w


def routed_feed_forward(h, W, mlp: Dict, pre: str, routing=None, tag=None) -> np.ndarray:
    """``routing``: None or a ``Routing``, which may settle close calls otherwise."""
    r = mlp["router"]
    real = int(r["experts"])
    ids, w, margin = route(h, W, mlp, pre)
    if routing is not None:
        z = h @ W[pre + "router"].T
        z = z - z.max(axis=-1, keepdims=True)
        s = np.exp(z) / np.exp(z).sum(axis=-1, keepdims=True)
        rms = np.sqrt(np.mean(s * s, axis=-1))
        ids, w = routing.choose(tag, ids, w, margin / rms, s * float(r.get("scale", 1.0)))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(ids[t], w[t]):
            if e >= real:                                   # an identity expert
                out[t] += we * h[t]
            else:
                out[t] += we * clamped_expert(h[t:t + 1], W, f"{pre}e{int(e)}.",
                                              float(mlp["expert"]["limit"]))[0]
    if mlp.get("shared"):
        out += clamped_expert(h, W, pre + "shared.", float(mlp["shared"]["limit"]))
    return out


# ---------------------------------------------------------------------------- the model
def weight_layer(config: Dict, i: int) -> int:
    """The layer whose tensors layer i uses."""
    seen = set()
    while config["layers"][i].get("weights_of") is not None and i not in seen:
        seen.add(i)
        i = int(config["layers"][i]["weights_of"])
    return i


def forward(config: Dict, W: Dict[str, np.ndarray], ids: List[int],
            states: Optional[List[np.ndarray]] = None, routing=None) -> np.ndarray:
    """Logits [T, vocab] of one sequence from its first token. ``states``: a list that receives
    the residual (the sum of the streams) after every layer."""
    eps = float(config["norm"]["eps"])
    T = len(ids)
    positions = np.arange(T)
    x0 = W["embed"][np.asarray(ids)] * float(config.get("embedding", {}).get("scale", 1.0))
    streams = config.get("streams")
    xs = [x0.copy() for _ in range(int(streams))] if streams else [x0.copy()]
    for i, layer in enumerate(config["layers"]):
        pre = f"l{weight_layer(config, i)}."

        def mixer(h, layer=layer, pre=pre):
            if layer["type"] == "wkv":
                return wkv_mixer(h, W, layer["mixer"], pre + "mix.", eps)
            if layer["type"] == "parallel":
                return parallel_mixer(h, W, layer["mixer"], pre + "mix.", eps, positions)
            raise ValueError(layer["type"])

        def ff(h, layer=layer, pre=pre, i=i):
            return routed_feed_forward(h, W, layer["mlp"], pre + "mlp.", routing, i)

        subs = [(1, mixer)] + ([(2, ff)] if layer.get("mlp") else [])
        for q, fn in subs:
            if streams:
                a, o, mx = W[f"{pre}hc{q}.in"], W[f"{pre}hc{q}.out"], W[f"{pre}hc{q}.mix"]
                u = sum(a[s] * xs[s] for s in range(len(xs)))
                y = fn(layer_norm(u, W[f"{pre}norm{q}"], eps))
                xs = [sum(mx[s, t] * xs[s] for s in range(len(xs))) + o[t] * y
                      for t in range(len(xs))]
            else:
                xs[0] = xs[0] + fn(layer_norm(xs[0], W[f"{pre}norm{q}"], eps))
        if states is not None:
            states.append(sum(xs))
    x = layer_norm(sum(xs), W["final.norm"], eps)
    return x @ W["embed"].T
