"""The Busavik family without a GPU: its config.json keys, the order of looped layers, the
model as data, the tensors it binds, YaRN frequencies against the plain implementation, and
the plain implementation against itself (latent attention in its two algebraic forms)."""
import copy
import json
import math

import numpy as np
import pytest

from mormot2_ai_b200 import BusavikConfig, ConfigError, DecoderModel
from mormot2_ai_b200.config.registry import family_of
from mormot2_ai_b200.parts.position import yarn_inverse_frequencies
from tests.busavik_models import SMALL, small_doc
from tests.plain import busavik_plain as plain


def test_registry_finds_the_family_by_its_architecture_key():
    doc = small_doc("P")
    assert family_of(doc) is BusavikConfig
    with pytest.raises(ConfigError, match="not known"):
        family_of({"architecture": "Nobody"})


@pytest.mark.parametrize("name", sorted(SMALL))
def test_round_trip_and_order(name):
    doc = small_doc(name)
    cfg = BusavikConfig.from_dict(doc)
    assert BusavikConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    assert cfg.order() == plain.layer_order(doc)
    spec = cfg.to_model_spec()
    assert [r.layer for r in spec.schedule] == cfg.order()
    # every run has a cache line of its own
    assert sorted(r.cache_line for r in spec.schedule) == list(range(len(cfg.order())))
    model = DecoderModel(spec)
    for line, need in model.line_needs.items():
        m = doc["layers"][spec.schedule[line].layer]["mixer"]
        assert (need.kv_heads, need.head_dim, need.planes) == (1, m["kv_rank"] + m["rot_dim"], 1)


def test_tensor_names_and_shapes():
    doc = small_doc("Q")
    model = DecoderModel(BusavikConfig.from_dict(doc).to_model_spec())
    needs = {n.name: tuple(n.shape) for n in model.tensors()}
    w, m0 = doc["width"], doc["layers"][0]["mixer"]
    assert needs["embed"] == (doc["vocab"], w) and needs["head"] == (doc["vocab"], w)
    assert needs["final.norm"] == (w,) and needs["final.norm.b"] == (w,)
    assert needs["final.norm.alpha"] == ()
    assert needs["l0.mix.dkv"] == (m0["kv_rank"] + m0["rot_dim"], w)
    assert needs["l0.mix.uq"] == (m0["heads"] * (m0["dim"] + m0["rot_dim"]), m0["q_rank"])
    assert needs["l0.mix.uk"] == (m0["heads"] * m0["dim"], m0["kv_rank"])
    assert needs["l0.mix.uv"] == (m0["heads"] * m0["vdim"], m0["kv_rank"])
    assert needs["l0.mix.g"] == (m0["heads"] * m0["vdim"], w)
    for i, layer in enumerate(doc["layers"]):
        mlp = layer["mlp"]
        if mlp is None:
            assert not any(k.startswith(f"l{i}.mlp") for k in needs)
            spare = [n for n in model.tensors() if n.name.startswith(f"l{i}.norm2")]
            assert spare and all(n.optional for n in spare)    # tolerated when stored, never needed
        elif mlp["kind"] == "dense":
            assert needs[f"l{i}.mlp.gate.b"] == (mlp["ff"],)
            assert needs[f"l{i}.mlp.down.b"] == (w,)
        else:
            e = mlp["router"]["experts"]
            assert needs[f"l{i}.mlp.router"] == (e, w)
            assert needs[f"l{i}.mlp.e{e - 1}.down"] == (w, mlp["expert"]["ff"])
            assert f"l{i}.mlp.e{e}.down" not in needs
            if mlp.get("shared"):
                assert needs[f"l{i}.mlp.shared.sg"] == (1, w)
            else:
                assert f"l{i}.mlp.shared.sg" not in needs


def test_refusals():
    good = small_doc("P")
    for change, match in [
        (lambda d: d.pop("vocab"), "vocab"),
        (lambda d: d["layers"][0].update(type="conv"), "not known"),
        (lambda d: d["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
        (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=3), "rotating"),
        (lambda d: d["layers"][1]["mlp"].update(kind="maxout"), "not known"),
        (lambda d: d.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
        (lambda d: d["layers"][1]["mlp"]["router"].update(top=99), "top"),
    ]:
        doc = copy.deepcopy(good)
        change(doc)
        with pytest.raises(ConfigError, match=match):
            BusavikConfig.from_dict(doc)


def test_yarn_frequencies_match_the_plain_ones():
    for rot in ({"dims": 16, "base": 10000.0,
                 "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}},
                {"dims": 24, "base": 5e5,
                 "scaling": {"factor": 16.0, "original": 4096, "fast": 32.0, "slow": 1.0}}):
        want, amp = plain.yarn_frequencies(rot)
        sc = rot["scaling"]
        got = yarn_inverse_frequencies(rot["base"], rot["dims"], sc["factor"], sc["original"],
                                       sc["fast"], sc["slow"])
        assert np.allclose(got, want, rtol=1e-6, atol=0)
        assert amp == pytest.approx(0.1 * math.log(sc["factor"]) + 1.0)
        # pairs that turn fast keep their frequency, slow ones are stretched by the factor
        plain_f = rot["base"] ** (-2.0 * np.arange(rot["dims"] // 2) / rot["dims"])
        assert want[0] == pytest.approx(plain_f[0])
        assert want[-1] == pytest.approx(plain_f[-1] / sc["factor"])
        assert np.all(want <= plain_f * (1 + 1e-12)) and np.all(want >= plain_f / sc["factor"] * (1 - 1e-12))


def test_plain_latent_attention_in_the_cached_form():
    """The oracle forms keys and values head by head. The library keeps only the latent and
    the shared rotated part; the same numbers must come out when the query is carried into the
    latent space instead (restated here in NumPy)."""
    rng = np.random.default_rng(5)
    m = {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 7, "q_rank": 9, "scale": 0.3,
         "rot": {"dims": 4, "base": 100.0,
                 "scaling": {"factor": 2.0, "original": 8, "fast": 4.0, "slow": 1.0}}}
    width, T, eps = 10, 12, 1e-5
    H, dim, rd, vd, kvr, qr = 3, 6, 4, 5, 7, 9
    W = {"dq": rng.normal(size=(qr, width)), "dq.norm": rng.normal(size=qr) + 1,
         "uq": rng.normal(size=(H * (dim + rd), qr)), "dkv": rng.normal(size=(kvr + rd, width)),
         "dkv.norm": rng.normal(size=kvr) + 1, "uk": rng.normal(size=(H * dim, kvr)),
         "uv": rng.normal(size=(H * vd, kvr)), "g": rng.normal(size=(H * vd, width)),
         "o": rng.normal(size=(width, H * vd))}
    h = rng.normal(size=(T, width))
    want = plain.latent_attention(h, m, W, "", eps)
    freqs, amp = plain.yarn_frequencies(m["rot"])
    pos = np.arange(T)
    cq = plain.rms_norm(h @ W["dq"].T, W["dq.norm"], eps)
    q = (cq @ W["uq"].T).reshape(T, H, dim + rd)
    dkv = h @ W["dkv"].T
    row = np.concatenate([plain.rms_norm(dkv[:, :kvr], W["dkv.norm"], eps),
                          plain.rotate_half(dkv[:, kvr:], pos, freqs, amp)], axis=1)   # the cache
    uk, uv = W["uk"].reshape(H, dim, kvr), W["uv"].reshape(H, vd, kvr)
    ql = np.concatenate([np.einsum("thd,hdr->thr", q[..., :dim], uk),
                         plain.rotate_half(q[..., dim:], pos, freqs, amp)], axis=-1)
    out = np.zeros((T, H, vd))
    for t in range(T):
        s = ql[t] @ row[:t + 1].T * m["scale"]                     # [H, t + 1]
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        out[t] = np.einsum("hr,hvr->hv", p @ row[:t + 1, :kvr], uv)
    got = (out.reshape(T, H * vd) * plain.sigmoid(h @ W["g"].T)) @ W["o"].T
    assert np.allclose(got, want, rtol=1e-9, atol=1e-9)


def test_plain_routing():
    z = np.array([[0.1, 2.0, 2.0, -1.0], [3.0, 1.0, 0.0, 3.5]])
    chosen, weight = plain.route(z, 2)
    assert chosen.tolist() == [[1, 2], [3, 0]]               # the lower index on a tie
    assert np.allclose(weight[0], [0.5, 0.5])
    assert np.allclose(weight[1], np.exp([0.0, -0.5]) / np.exp([0.0, -0.5]).sum())
