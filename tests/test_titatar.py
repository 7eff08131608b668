"""Titatar on the host: the reader and its refusals, the program of layer calls, tensor names and shapes, cache needs,
and the plain implementation against closed forms and against itself."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_titatar as pt
import titatar_helpers as th


def build(doc):
    from sglang_rs_b200 import models  # noqa: F401
    from sglang_rs_b200.config import RawConfig, resolve_architecture
    raw = RawConfig.from_dict(copy.deepcopy(doc))
    entry = resolve_architecture(raw)
    config = entry.parse_config(raw)
    return config, entry.build_model(config)


def random_weights(doc, seed):
    from sglang_rs_b200.weights.random_init import random_tensors
    _, model = build(doc)
    tensors = th.spread(random_tensors(model.tensor_specs(), seed), seed)
    return {k: v.to(torch.float64).numpy() for k, v in tensors.items()}


@pytest.mark.parametrize("doc", [th.SMALL_A, th.SMALL_B, th.SMALL_C, th.SMALL_D, th.SMALL_E], ids="abcde")
def test_the_reader_takes_every_size_from_the_document(doc):
    config, model = build(doc)
    assert config.width == doc["width"] and config.vocab == doc["vocab"] and len(config.layers) == len(doc["layers"])
    specs = model.tensor_specs()
    for index, entry in enumerate(doc["layers"]):
        m, p = entry["mixer"], f"l{index}.mix."
        if entry["type"] == "attention":
            assert specs[p + "q"].shape == (m["heads"] * m["dim"], doc["width"])
            assert specs[p + "v"].shape == (m["kv_heads"] * m["vdim"], doc["width"])
            assert specs[p + "q.norm"].shape == (m["heads"] * m["dim"],) and specs[p + "k.norm"].shape == (m["kv_heads"] * m["dim"],)
            assert specs[p + "g"].shape == (m["heads"], doc["width"]) and specs[p + "o"].shape == (doc["width"], m["heads"] * m["vdim"])
        else:
            assert specs[p + "uq"].shape == (m["heads"] * (m["dim"] + m["rot_dim"]), m["q_rank"])
            assert specs[p + "dkv"].shape == (m["kv_rank"] + m["rot_dim"], doc["width"])
            assert specs[p + "g"].shape == (m["heads"] * m["vdim"], doc["width"]) and specs[p + "sink"].shape == (m["heads"],)
        f = entry["mlp"]
        if f is None:
            assert f"l{index}.norm2" not in specs
        elif f["kind"] == "moe":
            routes = f["router"]["experts"] + f["router"].get("identity", 0)
            assert specs[f"l{index}.mlp.router"].shape == (routes, doc["width"]) and specs[f"l{index}.mlp.correction"].shape == (routes,)
            assert f"l{index}.mlp.e{f['router']['experts']}.up" not in specs
            assert (f"l{index}.mlp.shared.up" in specs) == bool(f.get("shared"))


def test_the_program_walks_the_stretch_and_opens_every_pass_but_the_first():
    _, model = build(th.SMALL_A)
    assert [(c.layer, c.entry, c.pass_index) for c in model.program] == [
        (0, None, 0), (1, None, 0), (2, None, 0), (1, 0, 1), (2, None, 1), (1, 0, 2), (2, None, 2), (3, None, 0)]
    assert [run for run in pt.layer_runs(th.SMALL_A)] == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True),
                                                          (2, False), (3, False)]
    needs = model.cache_needs()
    assert len(needs) == 8 and needs[1] == needs[3] and needs[1] is not needs[0]
    assert needs[0].window == 24 and needs[0].value_dim == 8 and needs[2].window == 40 and needs[1].window is None
    _, once = build(th.SMALL_E)
    assert once.pass_entries == [] and all(call.entry is None for call in once.program)
    _, none = build(th.SMALL_B)
    assert [c.layer for c in none.program] == [0, 1, 2]


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].__setitem__("type", "convolution"), "not a mixer"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda d: d["layers"][1]["mlp"]["router"].__setitem__("top", 9), "exceeds"),
    (lambda d: d["layers"][1]["mlp"].__setitem__("kind", "conv"), "not a feed-forward"),
    (lambda d: d["loop"].__setitem__("stop", 9), "stretch"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
])
def test_the_reader_refuses_what_it_cannot_build(change, message):
    from sglang_rs_b200.config import ConfigError
    doc = copy.deepcopy(th.SMALL_A)
    change(doc)
    with pytest.raises(ConfigError, match=message):
        build(doc)


def test_stretched_wavelengths_against_the_closed_form():
    from sglang_rs_b200.parts import RotaryEncoding, WavelengthScaling
    rot = {"base": 10000.0, "dims": 16, "scaling": th.STRETCH}
    plain, magnitude = pt.frequencies(rot)
    s = th.STRETCH
    package = RotaryEncoding(16, 10000.0, rotary_dim=16, interleaved=True,
                             scaling=WavelengthScaling(s["factor"], s["original"], s["fast"], s["slow"]))
    assert np.allclose(package.inverse_frequencies().double().numpy(), plain, rtol=1e-6)
    assert magnitude == pytest.approx(0.1 * math.log(8.0) + 1.0) and package.scaling.magnitude == pytest.approx(magnitude)
    base = np.array([10000.0 ** (-2 * i / 16) for i in range(8)])
    assert plain[0] == pytest.approx(base[0]) and plain[-1] == pytest.approx(base[-1] / 8.0)       # fast pairs kept, slow ones slowed
    assert np.all(plain <= base * (1 + 1e-12)) and np.all(plain >= base / 8.0 * (1 - 1e-12))


def test_the_plain_mechanisms_against_closed_forms():
    # a row of equal entries has root mean square |entry|; a zero weight multiplies by one
    assert np.allclose(pt.norm_one_plus(np.full((1, 8), 3.0), np.zeros(8), 0.0), 1.0)
    # one key, score 0: the unit sink halves the value; a sink of -inf leaves it whole
    q, k, v = np.zeros((1, 1, 4)), np.ones((1, 1, 4)), np.full((1, 1, 2), 6.0)
    assert np.allclose(pt.attend(q, k, v, 1.0, None, np.zeros(1)), 3.0)
    assert np.allclose(pt.attend(q, k, v, 1.0, None, np.full(1, -np.inf)), 6.0)
    # a window of two: the third row sees rows 1 and 2 only
    q, k = np.zeros((3, 1, 2)), np.zeros((3, 1, 2))
    v = np.array([10.0, 20.0, 60.0]).reshape(3, 1, 1)
    assert pt.attend(q, k, v, 1.0, 2, np.full(1, -np.inf))[2, 0, 0] == pytest.approx(40.0)
    # rotations keep lengths (magnitude 1) and are the identity at position 0
    x = np.random.default_rng(0).normal(size=(5, 2, 8))
    for interleaved in (False, True):
        y = pt.rotate(x, np.arange(5), {"base": 100.0, "dims": 6}, interleaved)
        assert np.allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1)) and np.allclose(y[0], x[0])
        assert np.allclose(y[..., 6:], x[..., 6:]) and not np.allclose(y[1:, :, :6], x[1:, :, :6])
    half = pt.rotate(x, np.arange(5), {"base": 100.0, "dims": 4}, False)
    pairs = pt.rotate(x, np.arange(5), {"base": 100.0, "dims": 4}, True)
    a = 3 * 100.0 ** (-2 / 4)
    assert pairs[3, 0, 2] == pytest.approx(x[3, 0, 2] * math.cos(a) - x[3, 0, 3] * math.sin(a))
    assert half[3, 0, 1] == pytest.approx(x[3, 0, 1] * math.cos(a) - x[3, 0, 3] * math.sin(a))


def test_experts_without_tensors_return_their_input():
    width = 6
    f = {"router": {"experts": 1, "identity": 2, "top": 1}}
    w = {"p.router": np.zeros((3, width)), "p.correction": np.array([0.0, 0.5, 0.1]),
         "p.e0.gate": np.ones((4, width)), "p.e0.up": np.ones((4, width)), "p.e0.down": np.ones((width, 4))}
    h = np.arange(12.0).reshape(2, width)
    # equal scores of a third each; the correction picks output 1, which has no tensors; the weight is the score
    assert np.allclose(pt.routed(h, w, "p.", f), h / 3.0)
    w["p.correction"] = np.array([0.9, 0.5, 0.1])
    assert np.allclose(pt.routed(h, w, "p.", f), pt.gated(h, w, "p.e0.") / 3.0)


def test_prefix_rows_do_not_depend_on_what_follows():
    """The plain implementation is causal: the logits of a prefix equal the first rows of the longer run."""
    for doc in (th.SMALL_A, th.SMALL_C):
        w = random_weights(doc, 3)
        tokens = th.random_requests(doc, (45,), seed=1)["r0"]
        collect = []
        whole = pt.forward(doc, w, tokens, collect)
        assert len(collect) == len(pt.layer_runs(doc))
        assert np.allclose(pt.forward(doc, w, tokens[:19]), whole[:19], atol=1e-9)


@pytest.mark.parametrize("mixer,window", [("attention", 12), ("latent_attention", None)])
def test_a_marked_key_decides_the_logits_of_the_made_models(tmp_path, mixer, window):
    """The models of ``titatar_helpers.marked_folder`` do what the GPU tests rely on: a row's logits hang on the marked key
    while it is visible, and (for the window) not at all once it is out."""
    folder = th.marked_folder(tmp_path, torch.float32, mixer, window)
    doc, w = th.load_folder(folder)
    mark = 5
    tokens = [th.PLAIN_TOKEN if t == th.MARK_TOKEN else t for t in th.random_requests(doc, (60,), seed=2)["r0"]]
    with_mark = tokens[:mark] + [th.MARK_TOKEN] + tokens[mark + 1:]
    a, b = pt.forward(doc, w, with_mark), pt.forward(doc, w, tokens)
    moved = np.abs(a - b).max(axis=1) / np.abs(a).max()
    if window:
        assert moved[mark + window - 1] > 0.3 and moved[mark + window] == 0.0 and moved[mark + 1] > 0.3
    else:
        assert moved[-1] > 0.3 and moved[mark + 1] > 0.3
    assert np.all(moved[:mark] == 0.0)
