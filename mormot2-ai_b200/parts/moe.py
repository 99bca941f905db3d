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

Options that a design may name. ``weights = "softmax_of_all"``: s = softmax(z) over every
router output; the choice goes by s + ``correction`` (a stored vector), the weights are the
chosen s times ``route_scale``, not renormalized. ``identity`` = n: the last n router outputs
are identity experts without tensors, whose output is the input h times the weight.
``activation = "clamped_swish"`` with ``limit``: g = min(W_g h, limit),
u = clamp(W_u h, −limit, limit), g · sigmoid(1.702 g) · (u + 1) (the shared expert has a
``shared_limit`` of its own). ``shared_gate = False``: the shared expert is added as it is.
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
        if not 0 < self.top <= min(self.experts + int(p.get("identity", 0)), 32):
            raise ConfigError(f"{self.top} of {self.experts} experts per token")
        modes = {"softmax_of_chosen": K.ROUTE_SOFTMAX_OF_CHOSEN,
                 "softmax_of_all": K.ROUTE_SOFTMAX_OF_ALL}
        if p.get("weights", "softmax_of_chosen") not in modes:
            raise ConfigError(f"expert weights \"{p['weights']}\" are not known "
                              f"(known: {', '.join(sorted(modes))})")
        self.mode = modes[p.get("weights", "softmax_of_chosen")]
        self.identity = int(p.get("identity", 0))
        self.routed = self.experts + self.identity      # what the router chooses among
        self.route_scale = float(p.get("route_scale", 1.0))
        self.limit = float(p.get("limit", 0.0))
        self.shared_limit = float(p.get("shared_limit", self.limit))
        self.shared_gate = bool(p.get("shared_gate", True))
        if self.mode == K.ROUTE_SOFTMAX_OF_ALL and (self.routed > 256 or self.shared_gate
                                                    and int(p.get("shared_size", 0))):
            raise ConfigError("scores over all router outputs: at most 256 outputs, and a "
                              "shared expert without a gate")
        if self.identity and self.mode != K.ROUTE_SOFTMAX_OF_ALL:
            raise ConfigError("identity experts come with scores over all router outputs")
        if self.top > self.routed:
            raise ConfigError(f"{self.top} of {self.routed} experts per token")
        if p.get("activation", "silu") not in K.ACTIVATIONS:
            raise ConfigError(f"activation \"{p['activation']}\" is not known")
        self.act = K.ACTIVATIONS[p.get("activation", "silu")]
        names = p["names"]
        self.n_router = prefix + names["router"]
        self.n_expert = [prefix + names["expert"].format(e) for e in range(self.experts)]
        self.n_shared = prefix + names["shared"]
        self.n_shared_gate = prefix + names.get("shared_gate", "")
        self.n_correction = prefix + names["correction"] if "correction" in names else None
        self.leaf = {k: names[k] for k in ("gate", "up", "down")}
        # for tests and debugging: called with (part, step, chosen experts [T, top] on the
        # device) in every forward; while it is set the part is not captured into graphs
        self.probe = None

    def libraries(self, rt) -> List[str]:
        return ["moe"]

    can_store = True      # forward(..., store=True) writes its output into x instead of adding

    def tensors(self) -> List[TensorNeed]:
        l = self.leaf
        out = [TensorNeed(self.n_router, (self.routed, self.hidden))]
        if self.n_correction:
            out.append(TensorNeed(self.n_correction, (self.routed,), "bias"))
        for e in self.n_expert:
            out += [TensorNeed(e + l["gate"], (self.inter, self.hidden)),
                    TensorNeed(e + l["up"], (self.inter, self.hidden)),
                    TensorNeed(e + l["down"], (self.hidden, self.inter))]
        if self.shared_size:
            s = self.n_shared
            out += [TensorNeed(s + l["gate"], (self.shared_size, self.hidden)),
                    TensorNeed(s + l["up"], (self.shared_size, self.hidden)),
                    TensorNeed(s + l["down"], (self.hidden, self.shared_size))]
            if self.shared_gate:
                out.append(TensorNeed(self.n_shared_gate, (1, self.hidden)))
        return out

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        l = self.leaf
        consume = getattr(rt, "consume_weights", False)
        take = (lambda name: weights.pop(name)) if consume else (lambda name: weights[name])
        router = [take(self.n_router)]
        if self.shared_size and self.shared_gate:
            router.append(take(self.n_shared_gate))
        self.correction = (weights[self.n_correction].to(torch.float32).contiguous()
                           if self.n_correction else None)
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

    def forward(self, h, x, step, store: bool = False):
        T, dev = h.shape[0], h.device
        E, top = self.experts, self.top
        A = T * top
        # [T, E (+ 1)] float32, or the split sums of the product, which the router adds up
        z = _sums(self.router(h, out_dtype=torch.float32, defer=True))
        ids = torch.empty((T, top), dtype=torch.int32, device=dev)
        w = torch.empty((T, top), dtype=torch.float32, device=dev)
        sg = (torch.empty((T,), dtype=torch.float32, device=dev)
              if self.shared_size and self.shared_gate else None)
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
        R = self.routed
        if T <= 64:          # the router's choice and the lists in one kernel
            K.moe_route_plan(z, E, top, R, ids, w, sg, bm, max_tiles, plan, self.mode,
                             self.correction, self.route_scale, R)
        else:
            K.moe_route(z, R, top, R, ids, w, sg, self.mode, self.correction, self.route_scale)
            K.moe_plan(ids, E, bm, max_tiles, plan)
        if self.probe is not None:
            self.probe(self, step, ids)
        act = torch.empty((A, self.inter), dtype=self.rt.dtype, device=dev)
        K.moe_gemm(h, self.w_up, act, plan, A, max_tiles, bm, top, True, self.act,
                   limit=self.limit)
        y = torch.empty((A, self.hidden), dtype=torch.float32, device=dev)
        K.moe_gemm(act, self.w_down, y, plan, A, max_tiles, bm, top, False, self.act, w)
        shared = None
        if self.shared_size:
            if self.shared_fused:
                sa = self.shared_up(h)
            else:
                gu = self.shared_up(h)
                sa = torch.empty((T, self.shared_size), dtype=self.rt.dtype, device=dev)
                K.gated_act(gu, sa, self.act, limit=self.shared_limit)
            shared = _sums(self.shared_down(sa, out_dtype=torch.float32, defer=True))
        if self.identity:
            K.moe_combine(x, y, top, shared, sg, ids, w, E, h, store=store)
        else:
            K.moe_combine(x, y, top, shared, sg, store=store)
        return None


FEED_FORWARDS.register("routed_experts", RoutedExperts)
