"""A feed-forward of routed experts, entirely on the device (``csrc/moe.cu``).

    z = W_router h (float32)          the ``top`` largest logits choose a token's experts
    w = softmax over the chosen logits only
    x += sum_k w_k · expert_k(h) + sigmoid(w_sg · h) · shared(h)
    expert(h) = W_d (act(W_g h) * (W_u h)), no biases; the shared expert (optional) has the
    same form with a size of its own and runs for every token.

The router and the shared expert's gate are one product with float32 results. The (token, k)
assignments are listed expert by expert by a kernel, the experts' two products run over
those lists in tiles (rows gathered for the first, results scattered back to the
assignment's own row by the second), and one kernel adds everything into the residual in a
fixed order. Nothing is read back to the host, so a decode pass stays a CUDA graph.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..errors import ConfigError
from .base import FEED_FORWARDS, Part, TensorNeed
from .linear import Linear, Pending


def _sums(result):
    """A product's float32 result [T, N], or its pending split sums as [parts, T, N]."""
    return result.partial if isinstance(result, Pending) else result


class RoutedExperts(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.experts, self.top = int(p["experts"]), int(p["top"])
        self.inter = int(p["intermediate_size"])
        self.shared_size = int(p.get("shared_size", 0))
        if not 0 < self.top <= min(self.experts, 32):
            raise ConfigError(f"{self.top} of {self.experts} experts per token")
        if p.get("weights", "softmax_of_chosen") != "softmax_of_chosen":
            raise ConfigError(f"expert weights \"{p['weights']}\" are not known "
                              "(known: softmax_of_chosen)")
        if p.get("activation", "silu") not in K.ACTIVATIONS:
            raise ConfigError(f"activation \"{p['activation']}\" is not known")
        self.act = K.ACTIVATIONS[p.get("activation", "silu")]
        names = p["names"]
        self.n_router = prefix + names["router"]
        self.n_expert = [prefix + names["expert"].format(e) for e in range(self.experts)]
        self.n_shared = prefix + names["shared"]
        self.n_shared_gate = prefix + names["shared_gate"]
        self.leaf = {k: names[k] for k in ("gate", "up", "down")}
        # for tests and debugging: called with (part, step, chosen experts [T, top] on the
        # device) in every forward; while it is set the part is not captured into graphs
        self.probe = None

    def libraries(self, rt) -> List[str]:
        return ["moe"]

    def tensors(self) -> List[TensorNeed]:
        l = self.leaf
        out = [TensorNeed(self.n_router, (self.experts, self.hidden))]
        for e in self.n_expert:
            out += [TensorNeed(e + l["gate"], (self.inter, self.hidden)),
                    TensorNeed(e + l["up"], (self.inter, self.hidden)),
                    TensorNeed(e + l["down"], (self.hidden, self.inter))]
        if self.shared_size:
            s = self.n_shared
            out += [TensorNeed(s + l["gate"], (self.shared_size, self.hidden)),
                    TensorNeed(s + l["up"], (self.shared_size, self.hidden)),
                    TensorNeed(s + l["down"], (self.hidden, self.shared_size)),
                    TensorNeed(self.n_shared_gate, (1, self.hidden))]
        return out

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        l = self.leaf
        consume = getattr(rt, "consume_weights", False)
        take = (lambda name: weights.pop(name)) if consume else (lambda name: weights[name])
        router = [take(self.n_router)]
        if self.shared_size:
            router.append(take(self.n_shared_gate))
        if len({w.dtype for w in router}) > 1:
            router = [w.float() for w in router]
        self.router = Linear(torch.cat(router, dim=0), rt)      # the gate's row behind the experts'
        ws = [take(e + l[k]) for e in self.n_expert for k in ("gate", "up", "down")]
        kind = ws[0].dtype if len({w.dtype for w in ws}) == 1 else torch.float32
        dev = ws[0].device
        # all experts' weights in two tensors: [E, 2 ff, hidden] (gate rows, then up rows) and
        # [E, hidden, ff]
        self.w_up = torch.empty((self.experts, 2 * self.inter, self.hidden), dtype=kind, device=dev)
        self.w_down = torch.empty((self.experts, self.hidden, self.inter), dtype=kind, device=dev)
        for e in range(self.experts):
            self.w_up[e, :self.inter].copy_(ws[3 * e])
            self.w_up[e, self.inter:].copy_(ws[3 * e + 1])
            self.w_down[e].copy_(ws[3 * e + 2])
            ws[3 * e] = ws[3 * e + 1] = ws[3 * e + 2] = None
        self.shared_up = self.shared_down = None
        if self.shared_size:
            g, u = take(self.n_shared + l["gate"]), take(self.n_shared + l["up"])
            if g.dtype != u.dtype:
                g, u = g.float(), u.float()
            # SiLU: gate and up rows alternate and the product's epilogue applies the activation
            # (as the SwiGLU feed-forward does); another activation: gate rows, then up rows,
            # and the activation kernel after the product
            self.shared_fused = self.act == K.ACT_SILU
            if self.shared_fused:
                both = torch.stack([g, u], dim=1).reshape(2 * self.shared_size, self.hidden)
            else:
                both = torch.cat([g, u], dim=0)
            self.shared_up = Linear(both, rt, swiglu=self.shared_fused)
            self.shared_down = Linear(weights[self.n_shared + l["down"]], rt)

    def forward(self, h, x, step):
        T, dev = h.shape[0], h.device
        E, top = self.experts, self.top
        A = T * top
        # [T, E (+ 1)] float32, or the split sums of the product, which the router adds up
        z = _sums(self.router(h, out_dtype=torch.float32, defer=True))
        ids = torch.empty((T, top), dtype=torch.int32, device=dev)
        w = torch.empty((T, top), dtype=torch.float32, device=dev)
        sg = torch.empty((T,), dtype=torch.float32, device=dev) if self.shared_size else None
        # rows per tile of an expert's list: 128 where the tensor-core kernel runs (bfloat16; 8
        # for a decode step of at most 8 tokens, the form that reads weights into registers),
        # else 64, or 16 while an expert has few rows, so that few multiply-adds are wasted
        fast = self.rt.fast_kernels and self.w_up.dtype == torch.bfloat16 and self.hidden % 8 == 0 \
            and self.inter % 8 == 0
        bm = 128 if fast else (64 if A > 16 * E else 16)
        if fast and T <= 8 and self.hidden % 32 == 0 and self.inter % 32 == 0:
            bm = 8      # a decode step: no expert has more rows, its weights stream once
        max_tiles = (A + bm - 1) // bm + E
        plan = torch.empty((2 + E + A + 2 * max_tiles,), dtype=torch.int32, device=dev)
        if T <= 64:          # the router's choice and the lists in one kernel
            K.moe_route_plan(z, E, top, E, ids, w, sg, bm, max_tiles, plan)
        else:
            K.moe_route(z, E, top, E, ids, w, sg)
            K.moe_plan(ids, E, bm, max_tiles, plan)
        if self.probe is not None:
            self.probe(self, step, ids)
        act = torch.empty((A, self.inter), dtype=self.rt.dtype, device=dev)
        K.moe_gemm(h, self.w_up, act, plan, A, max_tiles, bm, top, True, self.act)
        y = torch.empty((A, self.hidden), dtype=torch.float32, device=dev)
        K.moe_gemm(act, self.w_down, y, plan, A, max_tiles, bm, top, False, self.act, w)
        shared = None
        if self.shared_size:
            if self.shared_fused:
                sa = self.shared_up(h)
            else:
                gu = self.shared_up(h)
                sa = torch.empty((T, self.shared_size), dtype=self.rt.dtype, device=dev)
                K.gated_act(gu, sa, self.act)
            shared = _sums(self.shared_down(sa, out_dtype=torch.float32, defer=True))
        K.moe_combine(x, y, top, shared, sg)
        return None


FEED_FORWARDS.register("routed_experts", RoutedExperts)
