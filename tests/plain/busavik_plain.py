"""A plain, slow implementation of the Busavik decoder in NumPy float64: one function per
mechanism, whole sequences at once, no cache. It shares no code with the library and is the
oracle of the library's tests.

The design: token embedding; layers ``x += mixer(norm1(x)); x += ff(norm2(x))`` whose norms
are Dynamic Tanh; the mixer is latent attention (queries and keys/values through low-rank
latents, one rotated key part shared by all heads, YaRN-scaled rotary positions, an output
gate); the feed-forward is a dense gated GELU with biases or a mixture of experts with a
gated shared expert; a run of layers may be looped with the same weights; final norm, head,
logit scale.

``weights``: a dict name -> float64 array. ``config``: the dict of config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np


# ---------------------------------------------------------------------------- small functions
def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def dynamic_tanh(x, w, b, alpha):
    """tanh(alpha x) w + b: no mean, no variance."""
    return np.tanh(alpha * x) * w + b


# ---------------------------------------------------------------------------- positions
def yarn_frequencies(rot: Dict) -> (np.ndarray, float):
    """The dims/2 angular frequencies of a YaRN-scaled rotary encoding and the factor that
    multiplies both cosine and sine. Without ``scaling`` the plain frequencies and 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(v, positions, freqs, amplitude):
    """v [T, ..., n]: the first 2*len(freqs) values of the last axis rotate, value i paired
    with value i + len(freqs); the rest pass unchanged. positions [T]."""
    half = len(freqs)
    out = np.array(v, dtype=np.float64, copy=True)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]      # [T, half]
    shape = (v.shape[0],) + (1,) * (v.ndim - 2) + (half,)
    cos, sin = (np.cos(ang) * amplitude).reshape(shape), (np.sin(ang) * amplitude).reshape(shape)
    u, w = v[..., :half], v[..., half:2 * half]
    out[..., :half] = u * cos - w * sin
    out[..., half:2 * half] = w * cos + u * sin
    return out


# ---------------------------------------------------------------------------- the mixer
def latent_attention(h, m: Dict, W: Dict[str, np.ndarray], prefix: str, eps: float,
                     positions=None):
    """h [T, width] of one sequence. Keys and values are formed head by head from the latent
    (the form that caches nothing cleverly): k_h = [W_uk,h c ; rotated shared part],
    v_h = W_uv,h c."""
    T = h.shape[0]
    H, dim, rd, vd, kvr = (int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]),
                           int(m["kv_rank"]))
    pos = np.arange(T) if positions is None else np.asarray(positions)
    freqs, amp = yarn_frequencies(m["rot"])
    cq = rms_norm(h @ W[prefix + "dq"].T, W[prefix + "dq.norm"], eps)
    q = (cq @ W[prefix + "uq"].T).reshape(T, H, dim + rd)
    q_plain, q_rot = q[..., :dim], rotate_half(q[..., dim:], pos, freqs, amp)
    dkv = h @ W[prefix + "dkv"].T
    c = rms_norm(dkv[:, :kvr], W[prefix + "dkv.norm"], eps)
    k_rot = rotate_half(dkv[:, kvr:], pos, freqs, amp)                         # [T, rd], shared
    k_plain = (c @ W[prefix + "uk"].T).reshape(T, H, dim)
    v = (c @ W[prefix + "uv"].T).reshape(T, H, vd)
    scores = (np.einsum("ihd,jhd->hij", q_plain, k_plain)
              + np.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    visible = pos[None, :] <= pos[:, None]
    scores = np.where(visible[None], scores, -np.inf)
    scores -= scores.max(axis=-1, keepdims=True)
    p = np.exp(scores)
    p /= p.sum(axis=-1, keepdims=True)
    heads = np.einsum("hij,jhd->ihd", p, v).reshape(T, H * vd)
    heads = heads * sigmoid(h @ W[prefix + "g"].T)
    return heads @ W[prefix + "o"].T


# ---------------------------------------------------------------------------- feed-forwards
def dense_ff(h, W, prefix: str):
    g = h @ W[prefix + "gate"].T + W[prefix + "gate.b"]
    u = h @ W[prefix + "up"].T + W[prefix + "up.b"]
    return (gelu_tanh(g) * u) @ W[prefix + "down"].T + W[prefix + "down.b"]


def expert_ff(h, W, prefix: str):
    return (silu(h @ W[prefix + "gate"].T) * (h @ W[prefix + "up"].T)) @ W[prefix + "down"].T


def route(z, top: int):
    """z [T, experts] -> chosen [T, top] (largest logits first, the lower index on a tie) and
    their weights, the softmax over the chosen logits only."""
    order = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, order, axis=-1)
    e = np.exp(zc - zc.max(axis=-1, keepdims=True))
    return order, e / e.sum(axis=-1, keepdims=True)


class Routing:
    """What a test wants to know of the routers' choices, or to settle about them.

    ``margins[(run, t)]``: how far the last chosen logit of token t in layer run ``run`` lies
    above the first one left out, in units of the root mean square of the token's logits
    (their scale; their spread around the mean says nothing when there are two or three). ``forced[(run, t)]``: experts that another implementation chose there; they
    replace the plain choice where the two differ and the margin is below ``close`` (a
    computation in 16 bits may fall on either side of such a call), and where the margin is
    larger the difference is an error."""

    def __init__(self, forced=None, close: float = 0.03):
        self.forced = forced or {}
        self.close = close
        self.margins: Dict = {}
        self.replaced: List = []


def moe_ff(h, mlp: Dict, W, prefix: str, routing: Optional[Routing] = None, run: int = 0):
    top = int(mlp["router"]["top"])
    z = h @ W[prefix + "router"].T
    chosen, weight = route(z, top)
    if routing is not None:
        for t in range(h.shape[0]):
            zs = np.sort(z[t])[::-1]
            scale = max(float(np.sqrt(np.mean(z[t] ** 2))), 1e-30)
            margin = (zs[top - 1] - zs[top]) / scale if top < len(zs) else np.inf
            routing.margins[(run, t)] = float(margin)
            theirs = routing.forced.get((run, t))
            if theirs is not None and set(int(e) for e in theirs) != set(chosen[t].tolist()):
                if margin >= routing.close:
                    raise AssertionError(f"run {run}, token {t}: experts {sorted(theirs)} were "
                                         f"chosen, {sorted(chosen[t].tolist())} expected, at a "
                                         f"margin of {margin:.3g}")
                order = sorted((int(e) for e in theirs), key=lambda e: (-z[t, e], e))
                chosen[t] = order
                zc = z[t, order]
                e = np.exp(zc - zc.max())
                weight[t] = e / e.sum()
                routing.replaced.append((run, t))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(chosen[t, k])
            out[t] += weight[t, k] * expert_ff(h[t:t + 1], W, f"{prefix}e{e}.")[0]
    if mlp.get("shared"):
        gate = sigmoid(h @ W[prefix + "shared.sg"].T)                          # [T, 1]
        out += gate * expert_ff(h, W, prefix + "shared.")
    return out


def feed_forward(h, mlp: Optional[Dict], W, prefix: str, routing=None, run: int = 0):
    if mlp is None:
        return np.zeros_like(h)
    if mlp.get("kind", "dense") == "dense":
        return dense_ff(h, W, prefix)
    return moe_ff(h, mlp, W, prefix, routing, run)


# ---------------------------------------------------------------------------- the model
def layer_order(config: Dict) -> List[int]:
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def norm_of(x, W, name: str):
    return dynamic_tanh(x, W[name], W[name + ".b"], float(W[name + ".alpha"]))


def forward(config: Dict, W: Dict[str, np.ndarray], tokens, states: Optional[list] = None,
            routing: Optional[Routing] = None):
    """Logits [T, vocab] of one sequence from position 0. ``states``: a list that receives the
    residual after every layer run. ``routing``: see ``Routing``; a run is counted by its
    place in the order of layer runs."""
    eps = float(config["norm"]["eps"])
    x = W["embed"][np.asarray(tokens)]
    for run, i in enumerate(layer_order(config)):
        layer = config["layers"][i]
        p = f"l{i}."
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        x = x + latent_attention(norm_of(x, W, p + "norm1"), layer["mixer"], W, p + "mix.", eps)
        if layer.get("mlp") is not None:
            x = x + feed_forward(norm_of(x, W, p + "norm2"), layer["mlp"], W, p + "mlp.",
                                 routing, run)
        if states is not None:
            states.append(x.copy())
    return norm_of(x, W, "final.norm") @ W["head"].T * float(config["logit_scale"])
