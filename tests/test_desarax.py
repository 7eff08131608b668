"""Desarax on the host: the configuration reader, the order of layer calls, the checkpoint names, the needs for cache
and state, and the plain implementation against itself and against sums written out by hand."""
import copy
import math

import pytest
import torch

import desarax_helpers as dh
import plain_desarax as pd
from sglang_rs_b200.config import ConfigError, RawConfig, resolve_architecture
from sglang_rs_b200.parts import PagedKV, RequestState
from sglang_rs_b200.weights import build_model, random_tensors

F = torch.float64


def test_the_design_is_found_by_its_name():
    import sglang_rs_b200.models  # noqa: F401
    assert resolve_architecture(RawConfig.from_dict(copy.deepcopy(dh.SMALL_A))).name == "Desarax"


def test_a_layer_that_reads_another_layers_latents_is_a_call_on_that_layers_cache():
    model, config = build_model(dh.SMALL_A)
    assert [(c.layer, c.cache_from) for c in model.program] == [(0, None), (1, None), (2, None), (3, 1), (4, None)]
    needs = model.cache_needs()
    assert len(needs) == 5 and needs[3] is None
    # the convolution's last three inputs over 48 + 2 * 2 * 8 channels, then four states of 8 x 12
    assert needs[0] == RequestState((3 * 80 + 4 * 8 * 12,), torch.float32)
    assert needs[2] == RequestState((1 * 56 + 3 * 16 * 8,), torch.float32)
    # the cache of layer 1 keeps what the wider window of its reader sees
    assert needs[1] == PagedKV(1, 32, 37, values=False) and needs[4] == PagedKV(1, 16, None, values=False)
    assert config.cache_windows() == (None, 37, None, 37, None)
    model, config = build_model(dh.SMALL_B)                   # read without a window: every latent is kept
    assert config.cache_windows() == (None, None, None, None)
    assert model.cache_needs()[0] == PagedKV(1, 24, None, values=False)
    assert model.cache_needs()[1] == RequestState((24 * 8,), torch.float32)        # one tap: no inputs kept


def test_tensor_names_and_shapes():
    model, _ = build_model(dh.SMALL_A)
    specs = {name: spec.shape for name, spec in model.tensor_specs().items()}
    assert specs["embed"] == (90, 48) and specs["side.embed"] == (90, 50) and specs["final.norm"] == (48,) and "head" not in specs
    assert specs["l0.mix.in"] == (48 + 48 + 16 + 16 + 4, 48) and specs["l0.mix.conv"] == (80, 4) and specs["l0.mix.conv.b"] == (80,)
    assert specs["l0.mix.dt_bias"] == specs["l0.mix.A_log"] == specs["l0.mix.D"] == (4,)
    assert specs["l0.mix.norm"] == (48,) and specs["l0.mix.o"] == (48, 48)
    assert specs["l2.mix.in"] == (24 + 24 + 16 + 16 + 3, 48) and specs["l2.mix.conv"] == (56, 2)
    assert specs["l1.mix.q"] == (48, 48) and specs["l1.mix.dkv"] == (32, 48) and specs["l1.mix.dkv.norm"] == (32,)
    assert specs["l1.mix.uk"] == (48, 32) and specs["l1.mix.uv"] == (24, 32) and specs["l1.mix.o"] == (48, 24)
    assert "l3.mix.dkv" not in specs and "l3.mix.dkv.norm" not in specs and specs["l3.mix.uk"] == (16, 32) and specs["l3.mix.uv"] == (32, 32)
    assert specs["l0.mlp.router"] == (5, 48) and specs["l0.mlp.correction"] == (5,) and specs["l0.mlp.e4.gate"] == (24, 48)
    assert specs["l2.mlp.e3.down"] == (48, 20) and "l2.mlp.e4.up" not in specs and "l4.mlp.router" not in specs
    assert specs["l4.side.gate"] == (10, 48) and specs["l4.side.proj"] == (48, 10) and specs["l4.side.norm"] == (48,)
    assert "l0.norm2" not in specs and specs["l0.norm1"] == (48,)
    model, _ = build_model(dh.SMALL_B)
    assert not any("side" in name for name in model.tensor_specs())


@pytest.mark.parametrize("change,message", [
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["layers"][0].update(type="mamba3"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(groups=3), "groups"),
    (lambda d: d["layers"][0]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda d: d["layers"][0]["mixer"].pop("state"), "state"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(kv_rank=16), "kv_from"),
    (lambda d: d["layers"][4]["mixer"].update(kv_from=3), "kv_from"),
    (lambda d: d["layers"][1]["mixer"]["mask"].update(size=0), "size"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda d: d["norm"].update(groups=5), "groups"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["token_side"].pop("dim"), "dim"),
])
def test_documents_that_cannot_describe_a_model_are_refused(change, message):
    doc = copy.deepcopy(dh.SMALL_A)
    change(doc)
    with pytest.raises(ConfigError, match=message):
        build_model(doc)


def _tensors(doc, seed):
    model, _ = build_model(doc)
    return dh.spread(random_tensors(model.tensor_specs(), seed, "cpu", torch.float32), seed)


@pytest.mark.parametrize("doc", [dh.SMALL_A, dh.SMALL_B, dh.SMALL_C], ids=["a", "b", "c"])
def test_plain_implementation_is_causal(doc):
    tensors = _tensors(doc, 3)
    tokens = dh.random_requests(doc, (45,), seed=2)["r0"]
    whole = pd.forward(doc, tensors, tokens)
    for n in (1, 4, 26, 44):
        assert torch.allclose(pd.forward(doc, tensors, tokens[:n]), whole[:n], atol=1e-9)


def test_plain_recurrence_against_the_sum_over_earlier_tokens():
    """y_t = sum over s <= t of (prod of the decays after s up to t) dt_s (C_t . B_s) x_s + D x_t, written out."""
    torch.manual_seed(0)
    m = {"heads": 2, "vdim": 3, "state": 4, "groups": 1, "conv": 1, "norm_groups": 1}
    T, width, inner = 7, 5, 6
    w = {"in": torch.randn(2 * inner + 8 + 2, width, dtype=F), "conv": torch.ones(inner + 8, 1, dtype=F), "conv.b": torch.zeros(inner + 8, dtype=F),
         "dt_bias": torch.randn(2, dtype=F), "A_log": torch.randn(2, dtype=F), "D": torch.randn(2, dtype=F),
         "norm": torch.ones(inner, dtype=F), "o": torch.eye(inner, dtype=F)}
    h = torch.randn(T, width, dtype=F)
    got = pd.mamba2(h, w, m, 0.0)
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], pd.silu(proj[:, inner:2 * inner + 8]), pd.softplus(proj[:, 2 * inner + 8:] + w["dt_bias"])
    x, B, C = xbc[:, :inner].reshape(T, 2, 3), xbc[:, inner:inner + 4], xbc[:, inner + 4:]
    y = torch.zeros(T, 2, 3, dtype=F)
    for head in range(2):
        rate = torch.exp(w["A_log"][head])
        for t in range(T):
            for s in range(t + 1):
                keep = math.exp(-float(rate) * float(dt[s + 1:t + 1, head].sum()))
                y[t, head] += keep * dt[s, head] * (C[t] @ B[s]) * x[s, head]
            y[t, head] += w["D"][head] * x[t, head]
    y = y.reshape(T, inner) * pd.silu(z)
    want = y / torch.sqrt((y * y).mean(-1, keepdim=True))
    assert torch.allclose(got, want, atol=1e-10)


def test_plain_convolution_reads_zeros_before_the_start_and_its_last_column_now():
    u = torch.arange(1, 6, dtype=F)[:, None] * torch.tensor([1.0, 10.0], dtype=F)
    weight = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=F)
    out = pd.causal_conv(u, weight, torch.tensor([0.5, 0.0], dtype=F))
    assert out[:, 0].tolist() == [1.5, 2.5, 3.5, 4.5, 5.5]            # the current token's input plus the bias
    assert out[:, 1].tolist() == [0.0, 0.0, 10.0, 20.0, 30.0]         # the input two tokens back; nothing before the start


def test_plain_window_and_norm_in_parts():
    torch.manual_seed(1)
    m = {"heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "mask": {"size": 3}}
    w = {"q": torch.randn(4, 4, dtype=F), "uk": torch.eye(4, dtype=F), "uv": torch.eye(4, dtype=F), "o": torch.eye(4, dtype=F)}
    h, c = torch.randn(6, 4, dtype=F), torch.randn(6, 4, dtype=F)
    out = pd.latent_attention(h, c, w, m)
    q = h @ w["q"].T
    for i in range(6):
        keys = list(range(max(0, i - 2), i + 1))                       # itself and the two before it
        p = torch.softmax(torch.stack([q[i] @ c[j] for j in keys]) * 0.5, 0)
        assert torch.allclose(out[i], sum(p[k] * c[j] for k, j in enumerate(keys)))
    x = torch.randn(3, 12, dtype=F)
    weight = torch.rand(12, dtype=F)
    got = pd.group_norm(x, weight, 3, 1e-3)
    for part in range(3):
        piece = x[:, 4 * part:4 * part + 4]
        assert torch.allclose(got[:, 4 * part:4 * part + 4], piece / torch.sqrt((piece ** 2).mean(-1, keepdim=True) + 1e-3) * weight[4 * part:4 * part + 4])


def test_plain_router_chooses_with_the_correction_and_weighs_without_it():
    h = torch.eye(3, dtype=F)[:1] * 2.0
    router = torch.tensor([[1.0, 0, 0], [0.5, 0, 0], [-1.0, 0, 0]], dtype=F)       # logits 2, 1, -2
    s = torch.sigmoid(torch.tensor([2.0, 1.0, -2.0], dtype=F))
    chosen, weights = pd.route(h, router, torch.zeros(3, dtype=F), 2, 3.0)
    assert sorted(chosen[0].tolist()) == [0, 1] and torch.allclose(weights.sum(), torch.tensor(3.0, dtype=F))
    chosen, weights = pd.route(h, router, torch.tensor([0.0, -1.0, 1.0], dtype=F), 2, 3.0)
    order = chosen[0].tolist()
    assert sorted(order) == [0, 2]                                                 # the correction lifts the last expert
    want = {0: s[0] / (s[0] + s[2]) * 3.0, 2: s[2] / (s[0] + s[2]) * 3.0}           # weights from the scores without it
    for k, e in enumerate(order):
        assert torch.allclose(weights[0, k], want[e])


def test_plain_expert_clamps_the_gate_from_above_and_the_other_half_on_both_sides():
    gate, up, down = torch.tensor([[1.0]], dtype=F), torch.tensor([[1.0]], dtype=F), torch.tensor([[1.0]], dtype=F)
    def one(v):
        return float(pd.expert(torch.tensor([[v]], dtype=F), gate, up, down, 2.0))
    def by_hand(g, u):
        return g / (1.0 + math.exp(-1.702 * g)) * (u + 1.0)
    assert one(0.5) == pytest.approx(by_hand(0.5, 0.5))
    assert one(5.0) == pytest.approx(by_hand(2.0, 2.0))                # both at the limit
    assert one(-5.0) == pytest.approx(by_hand(-5.0, -2.0))             # the gate has no lower limit


def test_plain_token_input_takes_the_layers_slice_of_the_tokens_row():
    torch.manual_seed(2)
    x = torch.randn(2, 4, dtype=F)
    table = torch.randn(5, 6, dtype=F)
    w = {"gate": torch.randn(2, 4, dtype=F), "proj": torch.randn(4, 2, dtype=F), "norm": torch.rand(4, dtype=F)}
    got = pd.token_side(x, torch.tensor([3, 1]), table, 2, 2, w, 1e-6, 0.5)
    for r, token in enumerate((3, 1)):
        z = w["gate"] @ x[r]
        g = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))) * table[token, 4:6]
        y = w["proj"] @ g
        assert torch.allclose(got[r], x[r] + 0.5 * y / torch.sqrt((y * y).mean() + 1e-6) * w["norm"])
