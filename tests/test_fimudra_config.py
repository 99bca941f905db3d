"""The Fimudra family without a GPU: the registry, the model as data (layers that share
weights, cache lines and state of their own), tensor names and shapes, refusals, the scaled
rotary frequencies against the plain implementation's, and the plain implementation's own
consistency (a sequence fed whole against the recurrences restated step by step)."""
import json

import numpy as np
import pytest

from mormot2_ai_b200 import ConfigError, DecoderModel, FimudraConfig, architectures
from mormot2_ai_b200.config.registry import family_of
from mormot2_ai_b200.parts.position import banded_inverse_frequencies
from tests.fimudra_models import SMALL, small_doc
from tests.plain import fimudra_plain as plain


def test_registry_and_round_trip():
    assert "Fimudra" in architectures()
    for name in SMALL:
        doc = small_doc(name)
        assert family_of(doc) is FimudraConfig
        c = FimudraConfig.from_dict(doc)
        again = FimudraConfig.from_dict(json.loads(json.dumps(c.to_dict())))
        assert again == c
        assert c.vocab_size == doc["vocab"] and c.hidden_size == doc["width"]
        assert c.num_hidden_layers == len(doc["layers"])


def test_layers_that_share_weights_have_lines_of_their_own():
    c = FimudraConfig.from_dict(small_doc("U"))
    spec = c.to_model_spec()
    assert spec.streams == 3
    assert len(spec.layers) == 3 and len(spec.schedule) == 4        # layer 2 uses layer 0's
    assert [r.layer for r in spec.schedule] == [0, 1, 0, 2]
    assert [r.cache_line for r in spec.schedule] == [0, 1, 2, 3]
    model = DecoderModel(spec)
    names = {t.name for t in model.tensors()}
    assert not any(n.startswith("l2.") for n in names)
    assert {"l0.hc1.mix", "l0.hc2.in", "l3.hc1.out", "l0.mix.left.sink", "l1.mix.mu.w",
            "l0.mlp.correction", "final.norm", "embed"} <= names
    assert "l3.hc2.in" not in names and "l3.norm2" not in names     # no feed-forward there
    assert "l1.mlp.shared.gate" not in names
    shapes = {t.name: t.shape for t in model.tensors()}
    assert shapes["l0.mlp.router"] == (7, 80) and shapes["l0.mlp.correction"] == (7,)
    assert shapes["l0.mix.left.v"] == (2 * 40, 80) and shapes["l0.mix.left.o"] == (80, 4 * 40)
    assert shapes["l1.mix.w1"] == (6, 80) and shapes["l1.mix.u"] == (5, 12)
    assert shapes["l0.mix.right.i"] == (3, 80) and shapes["l0.mix.right.norm"] == (36,)
    # attention lines with value rows of their own size; state for every line
    assert model.line_needs[0].v_dim == 40 and model.line_needs[0].head_dim == 24
    assert set(model.line_needs) == {0, 2} and set(model.state_needs) == {0, 1, 2, 3}
    assert model.state_needs[0].shape == (3 * (20 * 12 + 20 + 1),)
    assert model.state_needs[1].shape == (80 + 5 * 12 * 12,)


def test_a_model_without_streams_is_a_plain_residual():
    spec = FimudraConfig.from_dict(small_doc("V")).to_model_spec()
    assert spec.streams == 0
    assert all(l.block.kind == "prenorm_residual" for l in spec.layers)
    assert spec.embedding.params["scale"] == 1.0
    names = {t.name for t in DecoderModel(spec).tensors()}
    assert not any(".hc" in n for n in names)
    # the decay's rank is a size that a stored model's tensors give
    doc = small_doc("V")
    del doc["layers"][0]["mixer"]["decay_rank"]
    shapes = {t.name: t.shape for t in DecoderModel(FimudraConfig.from_dict(doc).to_model_spec()).tensors()}
    assert shapes["l0.mix.w1"] == (-1, 50) and shapes["l0.mix.w2"] == (21, -1)


@pytest.mark.parametrize("change,match", [
    (lambda d: d["layers"][0].update(type="conv"), "mixer type"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3), "key/value heads"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=26), "rotating"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][2].update(weights_of=2), "own weights"),
    (lambda d: d["layers"][2].update(weights_of=1), "differs"),
    (lambda d: d.update(streams=9), "streams"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(gate_cap=0.0), "gate cap"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "feed-forward kind"),
])
def test_refusals(change, match):
    doc = small_doc("U")
    change(doc)
    with pytest.raises(ConfigError, match=match):
        FimudraConfig.from_dict(doc).to_model_spec()


@pytest.mark.parametrize("rot", [
    {"base": 1e4, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}},
    {"base": 5e5, "dims": 128, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}},
    {"base": 300.0, "dims": 6, "scaling": {"factor": 2.0, "low": 0.5, "high": 3.0, "original": 16}},
])
def test_scaled_frequencies(rot):
    sc = rot["scaling"]
    got = banded_inverse_frequencies(rot["base"], rot["dims"], sc["factor"], sc["low"], sc["high"],
                                     sc["original"])
    want = plain.rotary_frequencies(rot)
    assert np.allclose(got, want, rtol=1e-6, atol=0)
    plain_f = plain.rotary_frequencies({"base": rot["base"], "dims": rot["dims"]})
    kept, slowed = np.isclose(want, plain_f), np.isclose(want, plain_f / sc["factor"])
    assert kept.any() or slowed.any() or rot["dims"] < 8    # the bands of the rule occur
    assert not np.allclose(want, plain_f)
    # without scaling the same part gives the plain frequencies
    assert np.allclose(banded_inverse_frequencies(rot["base"], rot["dims"], 1.0, 1.0, 1.0, 1.0),
                       plain_f, rtol=1e-6, atol=0)


def test_the_plain_recurrences_do_not_depend_on_where_a_sequence_is_cut():
    """The oracle's own check: the logits of a prefix equal the first logits of the whole."""
    rng = np.random.default_rng(0)
    doc = small_doc("U")
    from mormot2_ai_b200.engine.model import DecoderModel as Model
    needs = Model(FimudraConfig.from_dict(doc).to_model_spec()).tensors()
    W = {}
    for n in needs:
        W[n.name] = rng.normal(0, 0.15, n.shape)
        if n.role == "vector":
            W[n.name] = 1 + 0.1 * W[n.name]
        if n.role == "identity":
            W[n.name] = np.eye(n.shape[0]) + 0.1 * W[n.name]
    ids = rng.integers(0, doc["vocab"], 12).tolist()
    whole = plain.forward(doc, W, ids)
    assert np.allclose(plain.forward(doc, W, ids[:7]), whole[:7], rtol=1e-9, atol=1e-9)


def test_the_plain_router():
    """Scores over all outputs, the correction on the choice only, no renormalizing."""
    W = {"p.router": np.array([[1.0, 0], [0, 1.0], [0.5, 0.5], [-1.0, 0]]),
         "p.correction": np.array([0.0, 0.0, 0.0, 10.0])}
    mlp = {"router": {"experts": 3, "identity": 1, "top": 2, "scale": 2.0}}
    h = np.array([[2.0, 0.0]])
    ids, w, _ = plain.route(h, W, mlp, "p.")
    z = np.array([2.0, 0.0, 1.0, -2.0])
    s = np.exp(z) / np.exp(z).sum()
    assert ids[0].tolist() == [3, 0]                     # the corrected one first, then the largest
    assert np.allclose(w[0], 2.0 * s[[3, 0]])
