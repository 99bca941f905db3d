"""Small Busavik configurations for the tests, their random model folders and the plain
implementation's view of them.

P: two layers looped twice and one after them; a dense and a routed feed-forward; YaRN; sizes
   that are no powers of two and all differ from one another.
Q: no loop; a layer without a feed-forward; one expert chosen of three and no shared expert
   in one layer, three of five with a shared expert in another; a rotary encoding without
   scaling; fewer rotating values than the rotated part holds; sizes that are not multiples
   of four (the kernels' scalar paths).
R: sizes that the tensor-core kernels take (multiples of 16), a loop over the last layers
   only, eight heads, four of sixteen experts.
"""
import json
import os

import numpy as np


def _mixer(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, dims=None, scaling=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
            "q_rank": q_rank, "scale": scale, "rot": rot}


def _moe(ff, experts, top, shared):
    doc = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        doc["shared"] = {"ff": shared}
    return doc


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


SMALL = {
    "P": lambda: {
        "architecture": "Busavik", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
        "logit_scale": 0.7, "loop": {"start": 0, "stop": 2, "times": 2},
        "layers": [
            _layer(_mixer(3, 20, 12, 28, 40, 24, 0.21, 1e4, scaling=(4.0, 64, 8.0, 2.0)),
                   {"kind": "dense", "ff": 100}),
            _layer(_mixer(3, 20, 12, 28, 40, 24, 0.21, 1e4, scaling=(4.0, 64, 8.0, 2.0)),
                   _moe(36, 6, 2, 52)),
            _layer(_mixer(5, 8, 16, 12, 24, 32, 0.3, 5e5, scaling=(16.0, 48, 16.0, 1.0)),
                   {"kind": "dense", "ff": 44}),
        ]},
    "Q": lambda: {
        "architecture": "Busavik", "vocab": 130, "width": 50, "norm": {"eps": 1e-6},
        "logit_scale": 1.0,
        "layers": [
            _layer(_mixer(2, 7, 10, 9, 13, 11, 0.4, 777.0, dims=6), _moe(18, 3, 1, 0)),
            _layer(_mixer(1, 14, 6, 5, 22, 19, 0.25, 1e4, scaling=(2.0, 16, 4.0, 1.0)), None),
            _layer(_mixer(4, 6, 2, 6, 9, 7, 0.5, 50.0), _moe(10, 5, 3, 14)),
        ]},
    "R": lambda: {
        "architecture": "Busavik", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
        "logit_scale": 2.0, "loop": {"start": 1, "stop": 3, "times": 3},
        "layers": [
            _layer(_mixer(8, 16, 16, 32, 48, 64, 0.18, 2e5, scaling=(6.0, 96, 24.0, 1.5)),
                   {"kind": "dense", "ff": 192}),
            _layer(_mixer(8, 16, 16, 32, 48, 64, 0.18, 2e5, scaling=(6.0, 96, 24.0, 1.5)),
                   _moe(64, 16, 4, 96)),
            _layer(_mixer(4, 32, 32, 16, 80, 48, 0.125, 1e4, scaling=(2.0, 32, 8.0, 2.0)),
                   {"kind": "dense", "ff": 160}),
        ]},
}

# name -> (seed, std of matrices, prompt lengths of the whole-prompt tests, decode steps)
HOW = {"P": (11, 0.12, [1, 9, 64, 150], 9), "Q": (12, 0.2, [2, 63, 65, 131], 7),
       "R": (13, 0.09, [5, 128, 200], 6)}


def small_doc(name):
    return SMALL[name]()


class SmallModel:
    def __init__(self, name, folder):
        from mormot2_ai_b200 import BusavikConfig, write_random_model
        from tests.plain import busavik_plain as plain
        from tests.plain.qwen3_plain import read_safetensors
        self.name, self.doc = name, small_doc(name)
        self.seed, std, self.prompt_lens, self.decode_steps = HOW[name]
        self.config = BusavikConfig.from_dict(self.doc)
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
