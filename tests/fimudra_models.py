"""Small Fimudra configurations for the tests, their random model folders and the plain
implementation's view of them.

U: three residual streams; a parallel layer whose attention has value rows of another size
   than its keys, a head only partly rotated and scaled frequencies, beside a matrix memory
   with other sizes again; a decaying-state layer; a layer that uses the first layer's
   weights; a layer without a feed-forward; identity experts, three experts of seven.
V: no streams (one plain residual), no embedding scale; attention without rotation and with
   as many key/value heads as heads; one expert per token, no shared expert, no identity
   expert; sizes that are not multiples of four.
W: one stream; sizes that the tensor-core kernels take (heads of 64 values, multiples of 32);
   full rotation without scaling; a decaying-state layer that is used twice.
"""
import json
import os

import numpy as np


def _left(heads, kv, dim, vdim, scale, rot=None):
    d = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        d["rot"] = rot
    return d


def _moe(ff, limit, experts, top, identity=None, scale=None, shared=None):
    r = {"experts": experts, "top": top}
    if identity is not None:
        r["identity"] = identity
    if scale is not None:
        r["scale"] = scale
    doc = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}
    if shared:
        doc["shared"] = {"ff": shared[0], "limit": shared[1]}
    return doc


def _u():
    par = {"type": "parallel", "mixer": {
        "left": _left(4, 2, 24, 40, 0.2, {"base": 1e4, "dims": 16, "scaling": {
            "factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}),
        "right": {"heads": 3, "dim": 20, "vdim": 12, "gate_cap": 8.0},
        "left_scale": 0.7, "right_scale": 0.6},
        "mlp": _moe(36, 2.0, 6, 3, identity=1, scale=1.2, shared=(28, 1.0))}
    return {"architecture": "Fimudra", "vocab": 199, "width": 80, "norm": {"eps": 1e-5},
            "embedding": {"scale": 3.0}, "streams": 3,
            "layers": [par,
                       {"type": "wkv", "mixer": {"heads": 5, "dim": 12, "decay_rank": 6},
                        "mlp": _moe(20, 0.7, 4, 1, identity=0, scale=2.0)},
                       dict(par, weights_of=0),
                       {"type": "wkv", "mixer": {"heads": 2, "dim": 36, "decay_rank": 10},
                        "mlp": None}]}


def _v():
    return {"architecture": "Fimudra", "vocab": 130, "width": 50, "norm": {"eps": 1e-6},
            "layers": [
                {"type": "wkv", "mixer": {"heads": 3, "dim": 7, "decay_rank": 5},
                 "mlp": _moe(18, 1.5, 3, 1)},
                {"type": "parallel", "mixer": {
                    "left": _left(3, 3, 10, 6, 0.31),
                    "right": {"heads": 1, "dim": 9, "vdim": 22, "gate_cap": 15.0},
                    "left_scale": 1.0, "right_scale": 1.0},
                 "mlp": _moe(10, 3.0, 5, 2, identity=2, shared=(14, 0.5))},
                {"type": "parallel", "mixer": {
                    "left": _left(2, 1, 6, 14, 0.4, {"base": 300.0, "dims": 6}),
                    "right": {"heads": 2, "dim": 5, "vdim": 5, "gate_cap": 4.0},
                    "left_scale": 0.3, "right_scale": 1.4},
                 "mlp": None}]}


def _w():
    wkv = {"type": "wkv", "mixer": {"heads": 2, "dim": 64, "decay_rank": 16},
           "mlp": _moe(64, 1.0, 8, 2, identity=0, scale=1.0, shared=(96, 2.0))}
    return {"architecture": "Fimudra", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
            "embedding": {"scale": 8.0}, "streams": 1,
            "layers": [wkv,
                       {"type": "parallel", "mixer": {
                           "left": _left(4, 1, 64, 64, 0.125, {"base": 5e5, "dims": 64}),
                           "right": {"heads": 2, "dim": 32, "vdim": 64, "gate_cap": 10.0},
                           "left_scale": 0.9, "right_scale": 0.4},
                        "mlp": _moe(32, 1.2, 16, 4, identity=3, scale=2.5)},
                       dict(wkv, weights_of=0)]}


SMALL = {"U": _u, "V": _v, "W": _w}

# name -> (seed, std of matrices, prompt lengths of the whole-prompt tests, decode steps)
HOW = {"U": (21, 0.12, [1, 9, 64, 150], 9), "V": (22, 0.1, [2, 63, 65, 131], 7),
       "W": (23, 0.09, [5, 128, 200], 6)}


def small_doc(name):
    return SMALL[name]()


class SmallModel:
    def __init__(self, name, folder):
        from mormot2_ai_b200 import FimudraConfig, write_random_model
        from tests.plain import fimudra_plain as plain
        from tests.plain.qwen3_plain import read_safetensors
        self.name, self.doc = name, small_doc(name)
        self.seed, std, self.prompt_lens, self.decode_steps = HOW[name]
        self.config = FimudraConfig.from_dict(self.doc)
        self.folder = write_random_model(folder, self.config, self.seed, std=std, norm_std=0.2)
        with open(os.path.join(folder, "config.json")) as f:
            self.plain_config = json.load(f)
        self.weights = {k: np.asarray(v, dtype=np.float64)
                        for k, v in read_safetensors(os.path.join(folder, "model.safetensors")).items()}
        self.plain = plain

    def tokens(self, n, seed=0):
        rng = np.random.default_rng(1000 * self.seed + seed)
        return rng.integers(0, self.doc["vocab"], n).tolist()

    def reference(self, ids, states=None, routing=None):
        return self.plain.forward(self.plain_config, self.weights, ids, states, routing)
