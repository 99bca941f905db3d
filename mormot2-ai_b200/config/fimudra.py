"""The typed configuration of the Fimudra decoder, read from its own config.json keys.

config.json: ``architecture`` = "Fimudra", ``vocab``, ``width``, ``norm.eps``,
``embedding.scale``, ``streams`` (the residual streams of the hyper-connections; absent: one
plain residual) and ``layers``, a list whose entries have ``type`` ("wkv" or "parallel"), the
mixer's sizes in ``mixer``, the feed-forward in ``mlp`` (or null) and optionally
``weights_of``: j, which makes the layer use layer j's tensors with a cache and a state of its
own. Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``l<i>.hc1.*``, ``l<i>.hc2.*``, ``final.norm``; the head is the embedding table.

Mixer ``wkv``: ``heads``, ``dim`` (and, for a random model only, ``decay_rank``: the low rank
of the decay's product, which a stored model gives by its tensors' shapes). Mixer
``parallel``: ``left`` (attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``rot`` with ``base``, ``dims`` and optionally ``scaling``: ``factor``, ``low``, ``high``,
``original``), ``right`` (matrix memory: ``heads``, ``dim``, ``vdim``, ``gate_cap``),
``left_scale``, ``right_scale``. Feed-forward ``moe``: ``expert`` (``ff``, ``limit``),
``router`` (``experts``, ``top``, ``identity``, ``scale``), ``shared`` (``ff``, ``limit``) or
none.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import ConfigError
from .busavik import MAX_POSITIONS, _dict, _int, _num
from .spec import LayerSpec, ModelSpec, PartSpec, Run


@dataclass(frozen=True)
class FimudraConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    streams: int                                  # 0: one plain residual
    layers: Tuple[Dict[str, Any], ...]            # as in config.json, checked
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Fimudra"
    MODEL_TYPE = "fimudra"

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
    def from_dict(cls, doc: Dict[str, Any], source: str = "config") -> "FimudraConfig":
        if not isinstance(doc, dict):
            raise ConfigError(f"{source} is no JSON object")
        if doc.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError(f"{source}: architecture \"{doc.get('architecture')}\" is not "
                              f"{cls.ARCHITECTURE}")
        layers = doc.get("layers")
        if not isinstance(layers, list) or not 0 < len(layers) <= 1024:
            raise ConfigError(f"{source}: \"layers\" is missing, empty or too long")
        for i, layer in enumerate(layers):
            cls._check_layer(layer, i, len(layers), f"{source}: layer {i}")
        scale = 1.0
        if doc.get("embedding") is not None:
            scale = _num(_dict(doc, "embedding", source), "scale", source + " embedding")
        streams = _int(doc, "streams", source, hi=8) if doc.get("streams") is not None else 0
        c = cls(vocab=_int(doc, "vocab", source, hi=1 << 22),
                width=_int(doc, "width", source, hi=1 << 16),
                norm_eps=_num(_dict(doc, "norm", source), "eps", source + " norm"),
                embedding_scale=scale, streams=streams, layers=tuple(layers))
        for i in range(len(layers)):
            j = c.weight_layer(i)
            if j != i and (layers[j]["type"] != layers[i]["type"]
                           or layers[j]["mixer"] != layers[i]["mixer"]
                           or layers[j].get("mlp") != layers[i].get("mlp")):
                raise ConfigError(f"{source}: layer {i} uses the weights of layer {j}, whose "
                                  "entry differs")
        return c

    @staticmethod
    def _check_layer(layer: Any, i: int, n: int, source: str) -> None:
        if not isinstance(layer, dict):
            raise ConfigError(f"{source} is no object")
        kind = layer.get("type")
        m = _dict(layer, "mixer", source)
        if kind == "wkv":
            _int(m, "heads", source + " mixer", hi=1 << 12)
            _int(m, "dim", source + " mixer", hi=1 << 12)
            if m.get("decay_rank") is not None:
                _int(m, "decay_rank", source + " mixer", hi=1 << 12)
        elif kind == "parallel":
            left, right = _dict(m, "left", source + " mixer"), _dict(m, "right", source + " mixer")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _int(left, key, source + " mixer.left", hi=1 << 12)
            if left["heads"] % left["kv_heads"]:
                raise ConfigError(f"{source}: {left['heads']} heads on {left['kv_heads']} "
                                  "key/value heads")
            _num(left, "scale", source + " mixer.left")
            if left.get("rot") is not None:
                rot = _dict(left, "rot", source + " mixer.left")
                dims = _int(rot, "dims", source + " rot", lo=0, hi=1 << 12)
                if dims % 2 or dims > left["dim"]:
                    raise ConfigError(f"{source}: {dims} rotating values of a head of "
                                      f"{left['dim']}")
                if dims and _num(rot, "base", source + " rot") <= 0:
                    raise ConfigError(f"{source}: a rotary base of {rot['base']}")
                if rot.get("scaling") is not None:
                    sc = _dict(rot, "scaling", source + " rot")
                    for key in ("factor", "low", "high", "original"):
                        if _num(sc, key, source + " rot.scaling") <= 0:
                            raise ConfigError(f"{source}: rot.scaling.{key} is {sc[key]!r}")
            for key in ("heads", "dim", "vdim"):
                _int(right, key, source + " mixer.right", hi=1 << 12)
            if _num(right, "gate_cap", source + " mixer.right") <= 0:
                raise ConfigError(f"{source}: a gate cap of {right['gate_cap']}")
            _num(m, "left_scale", source + " mixer")
            _num(m, "right_scale", source + " mixer")
        else:
            raise ConfigError(f"{source}: mixer type \"{kind}\" is not known "
                              "(known: parallel, wkv)")
        if layer.get("weights_of") is not None:
            j = _int(layer, "weights_of", source, lo=0, hi=n - 1)
            if j == i:
                raise ConfigError(f"{source} uses its own weights")
        mlp = layer.get("mlp")
        if mlp is None:
            return
        if not isinstance(mlp, dict) or mlp.get("kind", "moe") != "moe":
            raise ConfigError(f"{source}: feed-forward kind \"{mlp.get('kind') if isinstance(mlp, dict) else mlp}\" "
                              "is not known (known: moe)")
        e = _dict(mlp, "expert", source + " mlp")
        _int(e, "ff", source + " mlp.expert", hi=1 << 20)
        _num(e, "limit", source + " mlp.expert")
        r = _dict(mlp, "router", source + " mlp")
        experts = _int(r, "experts", source + " mlp.router", hi=256)
        identity = _int(r, "identity", source + " mlp.router", lo=0, hi=256) \
            if r.get("identity") is not None else 0
        if experts + identity > 256:
            raise ConfigError(f"{source}: {experts} + {identity} router outputs (at most 256)")
        _int(r, "top", source + " mlp.router", hi=min(experts + identity, 32))
        if r.get("scale") is not None:
            _num(r, "scale", source + " mlp.router")
        if mlp.get("shared") is not None:
            sh = _dict(mlp, "shared", source + " mlp")
            _int(sh, "ff", source + " mlp.shared", hi=1 << 20)
            _num(sh, "limit", source + " mlp.shared")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        doc: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.norm_eps},
                               "embedding": {"scale": self.embedding_scale},
                               "layers": list(self.layers)}
        if self.streams:
            doc["streams"] = self.streams
        return doc

    # ------------------------------------------------------------------ the model as data
    def weight_layer(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself, unless ``weights_of`` says otherwise)."""
        seen = set()
        while self.layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError(f"the layers' weights_of run in a circle at layer {i}")
            seen.add(i)
            i = int(self.layers[i]["weights_of"])
        return i

    def _positions(self, rot: Optional[Dict[str, Any]], positions: Dict[str, PartSpec]) -> str:
        """The name of the encoding with these constants (layers with equal ones share it)."""
        if not rot or not int(rot["dims"]):
            spec = PartSpec("none", {})
        else:
            sc = rot.get("scaling") or {"factor": 1.0, "low": 1.0, "high": 1.0, "original": 1.0}
            spec = PartSpec("rope_scaled_bands", {
                "theta": float(rot["base"]), "rot_dim": int(rot["dims"]),
                "factor": float(sc["factor"]), "low": float(sc["low"]),
                "high": float(sc["high"]), "original": float(sc["original"])})
        for name, have in positions.items():
            if have == spec:
                return name
        name = f"rot{len(positions)}"
        positions[name] = spec
        return name

    def to_model_spec(self) -> ModelSpec:
        c = self
        positions: Dict[str, PartSpec] = {}
        layers: List[LayerSpec] = []
        index_of: Dict[int, int] = {}      # config layer that owns tensors -> index in `layers`
        for i, layer in enumerate(c.layers):
            if c.weight_layer(i) != i:
                continue
            m, mlp = layer["mixer"], layer.get("mlp")
            if layer["type"] == "wkv":
                mixer = PartSpec("wkv", {
                    "hidden_size": c.width, "heads": int(m["heads"]), "dim": int(m["dim"]),
                    "eps": c.norm_eps, "decay_rank": m.get("decay_rank"),
                    "names": {"mu_r": "mix.mu.r", "mu_k": "mix.mu.k", "mu_v": "mix.mu.v",
                              "mu_g": "mix.mu.g", "mu_w": "mix.mu.w", "r": "mix.r", "k": "mix.k",
                              "v": "mix.v", "g": "mix.g", "w1": "mix.w1", "w2": "mix.w2",
                              "w0": "mix.w0", "u": "mix.u", "norm": "mix.norm", "o": "mix.o"}})
            else:
                left, right = m["left"], m["right"]
                attention = PartSpec("gqa_attention", {
                    "hidden_size": c.width, "heads": int(left["heads"]),
                    "kv_heads": int(left["kv_heads"]), "head_dim": int(left["dim"]),
                    "v_dim": int(left["vdim"]), "scale": float(left["scale"]),
                    "position": c._positions(left.get("rot"), positions),
                    "names": {"q": "mix.left.q", "k": "mix.left.k", "v": "mix.left.v",
                              "o": "mix.left.o", "sink": "mix.left.sink"}})
                memory = PartSpec("mlstm", {
                    "hidden_size": c.width, "heads": int(right["heads"]),
                    "dim": int(right["dim"]), "vdim": int(right["vdim"]),
                    "gate_cap": float(right["gate_cap"]), "eps": c.norm_eps,
                    "names": {"q": "mix.right.q", "k": "mix.right.k", "v": "mix.right.v",
                              "g": "mix.right.g", "o": "mix.right.o", "norm": "mix.right.norm",
                              "i": "mix.right.i", "f": "mix.right.f", "i_bias": "mix.right.i.b",
                              "f_bias": "mix.right.f.b"}})
                mixer = PartSpec("side_by_side", {"branches": [
                    {"mixer": attention, "scale": float(m["left_scale"])},
                    {"mixer": memory, "scale": float(m["right_scale"])}]})
            norm = lambda name: PartSpec("layernorm", {"name": name, "size": c.width,
                                                       "eps": c.norm_eps})
            norms = {"mixer": norm("norm1")}
            if mlp is None:
                ff = PartSpec("none")
            else:
                shared, r = mlp.get("shared"), mlp["router"]
                ff = PartSpec("routed_experts", {
                    "hidden_size": c.width, "experts": int(r["experts"]), "top": int(r["top"]),
                    "identity": int(r.get("identity") or 0),
                    "route_scale": float(r.get("scale", 1.0)),
                    "intermediate_size": int(mlp["expert"]["ff"]),
                    "limit": float(mlp["expert"]["limit"]),
                    "shared_size": int(shared["ff"]) if shared else 0,
                    "shared_limit": float(shared["limit"]) if shared else 0.0,
                    "shared_gate": False, "activation": "clamped_swish",
                    "weights": "softmax_of_all",
                    "names": {"router": "mlp.router", "correction": "mlp.correction",
                              "expert": "mlp.e{}.", "shared": "mlp.shared.",
                              "gate": "gate", "up": "up", "down": "down"}})
                norms["feed_forward"] = norm("norm2")
            if c.streams:
                names = {"mixer": {"in": "hc1.in", "out": "hc1.out", "mix": "hc1.mix"}}
                if mlp is not None:
                    names["feed_forward"] = {"in": "hc2.in", "out": "hc2.out", "mix": "hc2.mix"}
                block = PartSpec("hyper_connections", {"streams": c.streams, "names": names})
            else:
                block = PartSpec("prenorm_residual")
            index_of[i] = len(layers)
            layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ff, norms=norms,
                                    prefix=f"l{i}."))
        # every entry of the order has a cache line (keys and values, state, or both) of its own
        schedule = tuple(Run(layer=index_of[c.weight_layer(i)], cache_line=i, writes_cache=True)
                         for i in range(len(c.layers)))
        return ModelSpec(
            architecture=c.ARCHITECTURE, vocab_size=c.vocab, hidden_size=c.width,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": c.vocab,
                                                   "hidden_size": c.width,
                                                   "scale": c.embedding_scale}),
            positions=positions, layers=tuple(layers), schedule=schedule,
            final_norm=PartSpec("layernorm", {"name": "final.norm", "size": c.width,
                                              "eps": c.norm_eps}),
            head=PartSpec("lm_head", {"name": "head", "tied": True, "tied_to": "embed",
                                      "vocab_size": c.vocab, "hidden_size": c.width}),
            streams=c.streams)
