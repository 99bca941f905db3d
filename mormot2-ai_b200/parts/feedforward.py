"""Feed-forwards without routing.

``gated_mlp``: x += W_d (act(W_g h + b_g) * (W_u h + b_u)) + b_d with ``activation`` "silu" or
"gelu_tanh" and optional biases; gate and up are one product, the activation kernel adds the
biases (and leaves b_d in the residual rows that the last product then accumulates onto).
``none``: a layer without a feed-forward.

SwiGLU feed-forward: x += (silu(h·Wgᵀ) · (h·Wuᵀ)) · Wdᵀ, no bias
(``decoder.pas:2865-2899``, ``backend.cpu.pas:1827-1833`` of the reference). Gate and up are
one product whose epilogue applies the activation: their rows are laid out alternately (gate
of output 0, up of output 0, gate of output 1, ...), a pure re-layout done once at load."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..errors import ConfigError
from .base import FEED_FORWARDS, Part, TensorNeed
from .linear import Linear


class SwiGluFfn(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.names = {k: prefix + v for k, v in p["names"].items()}

    def tensors(self) -> List[TensorNeed]:
        n = self.names
        return [TensorNeed(n["gate"], (self.inter, self.hidden)),
                TensorNeed(n["up"], (self.inter, self.hidden)),
                TensorNeed(n["down"], (self.hidden, self.inter))]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        n = self.names
        g, u = weights[n["gate"]], weights[n["up"]]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        pairs = torch.stack([g, u], dim=1).reshape(2 * self.inter, self.hidden)
        self.gate_up = Linear(pairs, rt, swiglu=True)
        if getattr(rt, "consume_weights", False):   # the originals go once they are interleaved
            del g, u
            weights.pop(n["gate"], None)
            weights.pop(n["up"], None)
        self.down = Linear(weights[n["down"]], rt)

    def forward(self, h, x, step):
        """Adds the feed-forward's output into x, or returns it as ``Pending`` split sums for
        the next norm to add."""
        from .linear import Pending
        act = self.gate_up(h)
        out = self.down(act, add_into=x, defer=True)
        return out if isinstance(out, Pending) else None


class GatedMlp(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        if p["activation"] not in K.ACTIVATIONS:
            raise ConfigError(f"activation \"{p['activation']}\" is not known "
                              f"(known: {', '.join(sorted(K.ACTIVATIONS))})")
        self.act = K.ACTIVATIONS[p["activation"]]
        self.bias = bool(p.get("bias", False))
        self.names = {k: prefix + v for k, v in p["names"].items()}

    def tensors(self) -> List[TensorNeed]:
        n = self.names
        out = [TensorNeed(n["gate"], (self.inter, self.hidden)),
               TensorNeed(n["up"], (self.inter, self.hidden)),
               TensorNeed(n["down"], (self.hidden, self.inter))]
        if self.bias:
            out += [TensorNeed(n["gate_bias"], (self.inter,), "bias"),
                    TensorNeed(n["up_bias"], (self.inter,), "bias"),
                    TensorNeed(n["down_bias"], (self.hidden,), "bias")]
        return out

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        n = self.names
        g, u = weights[n["gate"]], weights[n["up"]]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.gate_up = Linear(torch.cat([g, u], dim=0), rt)      # gate rows, then up rows
        if getattr(rt, "consume_weights", False):
            del g, u
            weights.pop(n["gate"], None)
            weights.pop(n["up"], None)
        self.down = Linear(weights[n["down"]], rt)
        self.biases = None
        if self.bias:
            b = [weights[n["gate_bias"]], weights[n["up_bias"]], weights[n["down_bias"]]]
            if len({t.dtype for t in b}) > 1:
                b = [t.float() for t in b]
            self.biases = b

    def forward(self, h, x, step):
        from .linear import Pending
        gu = self.gate_up(h)
        act = torch.empty((h.shape[0], self.inter), dtype=self.rt.dtype, device=h.device)
        if self.biases is not None:
            K.gated_act(gu, act, self.act, self.biases[0], self.biases[1], x, self.biases[2])
        else:
            K.gated_act(gu, act, self.act)
        out = self.down(act, add_into=x, defer=True)
        return out if isinstance(out, Pending) else None


class NoFeedForward(Part):
    capturable = True

    def forward(self, h, x, step):
        return None


FEED_FORWARDS.register("swiglu", SwiGluFfn)
FEED_FORWARDS.register("gated_mlp", GatedMlp)
FEED_FORWARDS.register("none", NoFeedForward)
