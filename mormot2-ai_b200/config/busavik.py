"""The typed configuration of the Busavik decoder, read from its own config.json keys.

config.json: ``architecture`` = "Busavik", ``vocab``, ``width``, ``norm.eps``,
``logit_scale``, ``layers`` (a list; each entry has ``type``, the mixer's sizes in ``mixer``
and its feed-forward in ``mlp`` or null) and optionally ``loop`` (``start``, ``stop``,
``times``: layers start .. stop-1 run that many times in a row with the same weights, each
pass with a cache line of its own). Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``,
``l<i>.norm2``, ``l<i>.mlp.*``, ``final.norm``, ``head``.

Every layer is a pre-norm residual block whose norms are Dynamic Tanh. Mixer
``latent_attention``: queries and keys/values through low-rank latents, a rotated key part
shared by all heads, YaRN-scaled rotary positions, an output gate. Feed-forward ``dense``: a
gated GELU (tanh form) with biases; ``moe``: routed SiLU experts, the weights a softmax over
the chosen logits, plus a shared expert behind a sigmoid gate.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, Run

MAX_POSITIONS = 1 << 20      # the design names no limit; the cache's size is the real one


def _int(doc: Dict[str, Any], key: str, source: str, lo: int = 1, hi: int = 1 << 24) -> int:
    if key not in doc:
        raise ConfigError(f"{source} has no \"{key}\"")
    v = doc[key]
    if isinstance(v, float) and v == int(v):
        v = int(v)
    if isinstance(v, bool) or not isinstance(v, int) or not lo <= v <= hi:
        raise ConfigError(f"{source}: \"{key}\" is {v!r} (an integer from {lo} to {hi})")
    return v


def _num(doc: Dict[str, Any], key: str, source: str) -> float:
    if key not in doc:
        raise ConfigError(f"{source} has no \"{key}\"")
    v = doc[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"{source}: \"{key}\" is {v!r}, not a number")
    return float(v)


def _dict(doc: Dict[str, Any], key: str, source: str) -> Dict[str, Any]:
    v = doc.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{source}: \"{key}\" is missing or no object")
    return v


@dataclass(frozen=True)
class BusavikConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[Dict[str, Any], ...]          # as in config.json, checked
    loop: Optional[Tuple[int, int, int]] = None  # start, stop, times
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Busavik"
    MODEL_TYPE = "busavik"

    # the names that generic tools print
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return MAX_POSITIONS

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, doc: Dict[str, Any], source: str = "config") -> "BusavikConfig":
        if not isinstance(doc, dict):
            raise ConfigError(f"{source} is no JSON object")
        if doc.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError(f"{source}: architecture \"{doc.get('architecture')}\" is not "
                              f"{cls.ARCHITECTURE}")
        layers = doc.get("layers")
        if not isinstance(layers, list) or not 0 < len(layers) <= 1024:
            raise ConfigError(f"{source}: \"layers\" is missing, empty or too long")
        width = _int(doc, "width", source, hi=1 << 16)
        for i, layer in enumerate(layers):
            cls._check_layer(layer, f"{source}: layer {i}")
        loop = None
        if doc.get("loop") is not None:
            lp = _dict(doc, "loop", source)
            start = _int(lp, "start", source + " loop", lo=0, hi=len(layers))
            stop = _int(lp, "stop", source + " loop", lo=0, hi=len(layers))
            times = _int(lp, "times", source + " loop", lo=1, hi=1024)
            if stop < start:
                raise ConfigError(f"{source}: a loop from layer {start} to {stop}")
            loop = (start, stop, times)
        return cls(vocab=_int(doc, "vocab", source, hi=1 << 22), width=width,
                   norm_eps=_num(_dict(doc, "norm", source), "eps", source + " norm"),
                   logit_scale=_num(doc, "logit_scale", source) if "logit_scale" in doc else 1.0,
                   layers=tuple(layers), loop=loop)

    @staticmethod
    def _check_layer(layer: Any, source: str) -> None:
        if not isinstance(layer, dict):
            raise ConfigError(f"{source} is no object")
        if layer.get("type") != "latent_attention":
            raise ConfigError(f"{source}: mixer type \"{layer.get('type')}\" is not known "
                              "(known: latent_attention)")
        m = _dict(layer, "mixer", source)
        for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
            _int(m, key, source + " mixer", hi=1 << 16)
        _num(m, "scale", source + " mixer")
        rot = _dict(m, "rot", source + " mixer")
        dims = _int(rot, "dims", source + " rot", hi=1 << 16)
        if dims % 2 or dims > m["rot_dim"]:
            raise ConfigError(f"{source}: {dims} rotating values of a part of {m['rot_dim']}")
        if _num(rot, "base", source + " rot") <= 1:
            raise ConfigError(f"{source}: a rotary base of {rot['base']}")
        if rot.get("scaling") is not None:
            sc = _dict(rot, "scaling", source + " rot")
            for key in ("factor", "original", "fast", "slow"):
                if _num(sc, key, source + " rot.scaling") <= 0:
                    raise ConfigError(f"{source}: rot.scaling.{key} is {sc[key]!r}")
        mlp = layer.get("mlp")
        if mlp is None:
            return
        if not isinstance(mlp, dict):
            raise ConfigError(f"{source}: \"mlp\" is no object")
        kind = mlp.get("kind", "dense")
        if kind == "dense":
            _int(mlp, "ff", source + " mlp", hi=1 << 20)
        elif kind == "moe":
            _int(_dict(mlp, "expert", source + " mlp"), "ff", source + " mlp.expert", hi=1 << 20)
            r = _dict(mlp, "router", source + " mlp")
            experts = _int(r, "experts", source + " mlp.router", hi=4096)
            _int(r, "top", source + " mlp.router", hi=min(experts, 32))
            if mlp.get("shared") is not None:
                _int(_dict(mlp, "shared", source + " mlp"), "ff", source + " mlp.shared",
                     hi=1 << 20)
        else:
            raise ConfigError(f"{source}: feed-forward kind \"{kind}\" is not known "
                              "(known: dense, moe)")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        doc: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.norm_eps},
                               "logit_scale": self.logit_scale, "layers": list(self.layers)}
        if self.loop is not None:
            doc["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return doc

    # ------------------------------------------------------------------ the model as data
    def order(self) -> List[int]:
        """The layers in the order they run (a looped layer once per pass)."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_model_spec(self) -> ModelSpec:
        c = self
        positions: Dict[str, PartSpec] = {}
        layers = []
        for i, layer in enumerate(c.layers):
            m, mlp = layer["mixer"], layer.get("mlp")
            rot = m["rot"]
            pos_name = f"rot{i}"
            params = {"theta": float(rot["base"]), "rot_dim": int(rot["dims"])}
            if rot.get("scaling"):
                sc = rot["scaling"]
                params.update(factor=float(sc["factor"]), original=float(sc["original"]),
                              fast=float(sc["fast"]), slow=float(sc["slow"]))
            # layers with the same constants share one encoding
            for name, spec in positions.items():
                if spec.params == params:
                    pos_name = name
                    break
            else:
                positions[pos_name] = PartSpec("rope_yarn" if rot.get("scaling") else "rope_half",
                                               params)
            norm = lambda name: PartSpec("dynamic_tanh", {"name": name, "size": c.width})
            mixer = PartSpec("latent_attention", {
                "hidden_size": c.width, "heads": int(m["heads"]), "dim": int(m["dim"]),
                "rot_dim": int(m["rot_dim"]), "vdim": int(m["vdim"]),
                "kv_rank": int(m["kv_rank"]), "q_rank": int(m["q_rank"]),
                "scale": float(m["scale"]), "latent_norm_eps": c.norm_eps, "gate": True,
                "position": pos_name,
                "names": {"dq": "mix.dq", "dq_norm": "mix.dq.norm", "uq": "mix.uq",
                          "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm", "uk": "mix.uk",
                          "uv": "mix.uv", "g": "mix.g", "o": "mix.o"}})
            norms = {"mixer": norm("norm1")}
            if mlp is None:
                ff = PartSpec("none")
            elif mlp.get("kind", "dense") == "dense":
                ff = PartSpec("gated_mlp", {
                    "hidden_size": c.width, "intermediate_size": int(mlp["ff"]),
                    "activation": "gelu_tanh", "bias": True,
                    "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down",
                              "gate_bias": "mlp.gate.b", "up_bias": "mlp.up.b",
                              "down_bias": "mlp.down.b"}})
            else:
                shared = mlp.get("shared")
                ff = PartSpec("routed_experts", {
                    "hidden_size": c.width, "experts": int(mlp["router"]["experts"]),
                    "top": int(mlp["router"]["top"]),
                    "intermediate_size": int(mlp["expert"]["ff"]),
                    "shared_size": int(shared["ff"]) if shared else 0,
                    "activation": "silu", "weights": "softmax_of_chosen",
                    "names": {"router": "mlp.router", "expert": "mlp.e{}.",
                              "shared": "mlp.shared.", "shared_gate": "mlp.shared.sg",
                              "gate": "gate", "up": "up", "down": "down"}})
            if mlp is not None:
                norms["feed_forward"] = norm("norm2")
            else:
                # a layer without a feed-forward may still store its second norm: tolerated, unused
                norms["spare"] = PartSpec("dynamic_tanh", {"name": "norm2", "size": c.width,
                                                           "optional": True})
            layers.append(LayerSpec(block=PartSpec("prenorm_residual"), mixer=mixer,
                                    feed_forward=ff, norms=norms, prefix=f"l{i}."))
        schedule = tuple(Run(layer=l, cache_line=n, writes_cache=True)
                         for n, l in enumerate(c.order()))
        return ModelSpec(
            architecture=c.ARCHITECTURE, vocab_size=c.vocab, hidden_size=c.width,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": c.vocab,
                                                   "hidden_size": c.width}),
            positions=positions, layers=tuple(layers), schedule=schedule,
            final_norm=PartSpec("dynamic_tanh", {"name": "final.norm", "size": c.width}),
            head=PartSpec("lm_head", {"name": "head", "tied": False, "tied_to": "embed",
                                      "vocab_size": c.vocab, "hidden_size": c.width,
                                      "scale": c.logit_scale}))
