"""Titatar on the GPU against the plain implementation: each mechanism alone, whole prompts, prompts with a tail decoded
token by token, portions down to two tokens, mixed batches over a small pool (pages are used again), keys just inside and
just outside a window and far away at page borders, the first tokens, long decoding, and greedy generation through the
entry point."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_titatar as pt
import replay_helpers as rh
import titatar_helpers as th

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [("float32", torch.float32, 2e-5), ("bfloat16", torch.bfloat16, 4e-2)]


def seen(tensor, dtype):
    """What the kernel sees of a tensor: rounded to the storage type, as a float64 array."""
    return tensor.to(dtype).to(torch.float64).numpy()


def close(got, want, dtype, what, fraction=None):
    tolerance = fraction if fraction is not None else (2e-5 if dtype == torch.float32 else 2e-2)
    want = np.asarray(want, dtype=np.float64)
    scale = float(np.abs(want).max()) or 1.0
    error = float(np.abs(got.detach().double().cpu().numpy() - want).max()) / scale
    assert error <= tolerance, (what, error)


# ------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_with_weights_around_zero_and_a_second_term_of_the_sum(dtype):
    from sglang_rs_b200.parts import GroupedRmsNorm, NormedDelta, PassSum
    g = torch.Generator().manual_seed(1)
    rows, width, eps = 9, 44, 1e-5
    stored = {"a": torch.randn(width, generator=g) * 0.3, "b": torch.randn(width, generator=g) * 0.3}
    ahead, behind = GroupedRmsNorm(width, eps, "a", weight_offset=1.0), GroupedRmsNorm(width, eps, "b", weight_offset=1.0)
    for norm in (ahead, behind):
        norm.load(stored, DEV, dtype)
    x, y, x0 = (torch.randn(rows, width, generator=g) * 2 for _ in range(3))
    residual = x.to(DEV)
    out = ahead.add_norm(residual, NormedDelta(y.to(dtype).to(DEV), behind), dtype)
    total = x.double().numpy() + pt.norm_one_plus(seen(y, dtype), stored["b"].double().numpy(), eps)
    close(residual, total, torch.float32, "the stream after the normed term", 1e-6)
    close(out, pt.norm_one_plus(total, stored["a"].double().numpy(), eps), dtype, "norm of the sum")
    # the head of a later pass: pending term, then the embedding output, in one kernel
    residual = x.to(DEV)
    after = PassSum().forward(None, residual, NormedDelta(y.to(dtype).to(DEV), behind), x0.to(DEV), 1)
    assert after is residual
    close(residual, total + x0.double().numpy(), torch.float32, "stream + normed term + embedding output", 1e-6)
    residual = x.to(DEV)
    PassSum().forward(None, residual, None, x0.to(DEV), 1)
    close(residual, (x + x0).double().numpy(), torch.float32, "stream + embedding output", 1e-7)
    # the pending term as partial sums of a product cut along K: added in order, then normed
    pieces = torch.randn(5, rows, width, generator=g)
    residual = x.to(DEV)
    out = ahead.add_norm(residual, NormedDelta(pieces.to(DEV), behind), dtype)
    total = x.double().numpy() + pt.norm_one_plus(pieces.double().sum(0).numpy(), stored["b"].double().numpy(), eps)
    close(residual, total, torch.float32, "the stream after the normed sum of the parts", 1e-6)
    close(out, pt.norm_one_plus(total, stored["a"].double().numpy(), eps), dtype, "norm of that sum")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d,vd,rot,interleaved,parts", [(4, 2, 16, 8, 8, False, 0), (3, 3, 10, 14, 6, False, 3),
                                                                  (2, 1, 64, 64, 64, True, 0), (5, 1, 12, 4, 0, False, 2)])
def test_norms_over_whole_projections_rotation_pages_and_gates(dtype, n_q, n_kv, d, vd, rot, interleaved, parts):
    from sglang_rs_b200 import ops
    g = torch.Generator().manual_seed(n_q * 100 + d)
    rows, page, pages, eps, magnitude = 11, 4, 9, 1e-5, 1.3
    width = (n_q + n_kv) * d + n_kv * vd + n_q
    proj = torch.randn(rows, width + 3, generator=g) * 2                  # three spare columns behind the row
    qw, kw = torch.rand(n_q * d, generator=g) + 0.5, torch.rand(n_kv * d, generator=g) + 0.5
    positions = torch.randint(0, 500, (rows,), generator=g).int()
    slots = torch.randperm(pages * page, generator=g)[:rows].int()
    inv_freq = torch.tensor([50.0 ** (-2 * i / rot) for i in range(rot // 2)], dtype=torch.float32) if rot else None
    if parts and dtype == torch.bfloat16:
        pieces = torch.randn(parts, rows, width + 3, generator=g)
        given, exact = pieces.to(DEV), pieces.double().sum(0).numpy()
    else:
        given, exact = proj.to(dtype).to(DEV), seen(proj, dtype)
    q_out = torch.zeros(rows, n_q, d, dtype=dtype, device=DEV)
    k_pool = torch.zeros(pages, n_kv, page, d, dtype=dtype, device=DEV)
    v_pool = torch.zeros(pages, n_kv, page, vd, dtype=dtype, device=DEV)
    gates = torch.zeros(rows, n_q, dtype=torch.float32, device=DEV)
    word = ops.new_error_word(DEV)
    ops.proj_norm_rope_kv(given, q_out, k_pool, v_pool, positions.to(DEV), slots.to(DEV), qw.to(DEV), kw.to(DEV), eps,
                          inv_freq.to(DEV) if rot else None, rot, interleaved, n_q, n_kv, d, vd, word, magnitude=magnitude,
                          gate_out=gates)
    ops.raise_on_error_word(word)
    q = pt.rms(exact[:, :n_q * d], eps) * qw.double().numpy()
    k = pt.rms(exact[:, n_q * d:(n_q + n_kv) * d], eps) * kw.double().numpy()
    q, k = q.reshape(rows, n_q, d), k.reshape(rows, n_kv, d)
    if rot:
        turn = {"base": 50.0, "dims": rot}
        q, k = (pt.rotate(t, positions.numpy(), turn, interleaved) for t in (q, k))
        # the factor on cosines and sines multiplies the rotated entries only
        q[..., :rot] *= magnitude
        k[..., :rot] *= magnitude
    v = exact[:, (n_q + n_kv) * d:(n_q + n_kv) * d + n_kv * vd].reshape(rows, n_kv, vd)
    close(q_out, q, dtype, "q")
    close(gates, pt.sigmoid(exact[:, width - n_q:width]), torch.float32, "gates", 1e-5)
    page_of, inside = (slots // page).long(), (slots % page).long()
    close(k_pool[page_of.to(DEV), :, inside.to(DEV)], k, dtype, "keys in their slots")
    close(v_pool[page_of.to(DEV), :, inside.to(DEV)], v, dtype, "values in their slots")
    used = torch.zeros(pages, page, dtype=torch.bool)
    used[page_of, inside] = True
    assert float(k_pool.float().abs().sum(dim=(1, 3)).cpu()[~used].sum()) == 0.0, "a slot of another row was written"


def paged(keys, values, page, dtype, seed):
    """Keys [T, G, d] and values [T, G, dv] of one request laid into shuffled pages; (k_pool, v_pool, block table)."""
    tokens = keys.shape[0]
    count = -(-tokens // page)
    order = torch.randperm(count + 3, generator=torch.Generator().manual_seed(seed))[:count]
    k_pool = torch.zeros(count + 3, keys.shape[1], page, keys.shape[2], dtype=dtype)
    v_pool = torch.zeros(count + 3, values.shape[1], page, values.shape[2], dtype=dtype)
    for t in range(tokens):
        k_pool[order[t // page], :, t % page] = keys[t].to(dtype)
        v_pool[order[t // page], :, t % page] = values[t].to(dtype)
    return k_pool.to(DEV), v_pool.to(DEV), order.int().view(1, -1).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,d,vd,window,split", [(4, 2, 16, 8, 24, 0), (3, 1, 10, 14, 0, 32), (34, 1, 8, 12, 70, 64),
                                                        (2, 2, 20, 20, 1, 0)])
def test_attention_with_a_unit_sink_gates_and_values_of_their_own_width(dtype, heads, kv, d, vd, window, split):
    """The generic kernel: a sink in the denominator (once, also when the keys are split), a gate per (row, head), values
    narrower and wider than the keys, a window; rows anywhere in a sequence of 150 keys."""
    from sglang_rs_b200 import ops
    g = torch.Generator().manual_seed(heads + d)
    tokens, page, scale = 150, 8, 0.4
    q, k, v = torch.randn(tokens, heads, d, generator=g), torch.randn(tokens, kv, d, generator=g), torch.randn(tokens, kv, vd, generator=g)
    sinks, gates = torch.randn(heads, generator=g), torch.rand(tokens, heads, generator=g)
    k_pool, v_pool, table = paged(k, v, page, dtype, 3)
    rows = torch.tensor([0, 1, 7, 8, 23, 24, 25, 63, 64, 100, 149])
    out = torch.zeros(len(rows), heads, vd, dtype=dtype, device=DEV)
    word = ops.new_error_word(DEV)
    splits = -(-tokens // split) + 1 if split else 1
    acc = torch.zeros(len(rows) * heads * splits * vd, device=DEV) if split else None
    ml = torch.zeros(len(rows) * heads * splits * 2, device=DEV) if split else None
    ops.paged_attention(q[rows].to(dtype).to(DEV), k_pool, v_pool, out, rows.int().to(DEV),
                        torch.zeros(len(rows), dtype=torch.int32, device=DEV), table, scale=scale, window=window,
                        split_size=split, max_splits=splits, scratch_acc=acc, scratch_ml=ml, error_word=word,
                        sinks=sinks.to(DEV), gates=gates[rows].contiguous().to(DEV))
    ops.raise_on_error_word(word)
    per = heads // kv
    want = pt.attend(seen(q, dtype), np.repeat(seen(k, dtype), per, 1), np.repeat(seen(v, dtype), per, 1), scale,
                     window or None, sinks.double().numpy()) * gates.double().numpy()[:, :, None]
    close(out, want[rows.numpy()], dtype, "attention")


@pytest.mark.parametrize("d,heads,kv,window", [(64, 4, 2, 48), (128, 2, 1, 0), (64, 3, 3, 200)])
def test_the_tensor_core_kernels_take_the_sink_and_the_gates(d, heads, kv, window):
    """The three bfloat16 kernels (tcgen05 tiles and mma.sync tiles for prompt portions, split keys for decoded rows)
    against the plain attention, with a sink per head that is counted once and a gate per (row, head)."""
    from sglang_rs_b200 import ops
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(d + heads)
    tokens, page, scale = 300, 16, d ** -0.5
    q, k, v = (torch.randn(tokens, n, d, generator=g) for n in (heads, kv, kv))
    sinks, gates = torch.randn(heads, generator=g) * 2, torch.rand(tokens, heads, generator=g)
    k_pool, v_pool, table = paged(k, v, page, dtype, 5)
    per = heads // kv
    want = pt.attend(seen(q, dtype), np.repeat(seen(k, dtype), per, 1), np.repeat(seen(v, dtype), per, 1), scale,
                     window or None, sinks.double().numpy()) * gates.double().numpy()[:, :, None]
    word = ops.new_error_word(DEV)
    qd, gd, sd = q.to(dtype).to(DEV), gates.to(DEV), sinks.to(DEV)
    for name, rows_per_tile, run in (("tcgen05 tiles", ops.TC_TILE_ROWS, ops.tiled_attention_tc), ("mma tiles", 64, ops.tiled_attention)):
        first = 37                                           # the portion starts in the middle of a page
        tiles = torch.tensor([[b - first, min(rows_per_tile, tokens - b), 0, b] for b in range(first, tokens, rows_per_tile)],
                             dtype=torch.int32, device=DEV)
        out = torch.zeros(tokens - first, heads, d, dtype=dtype, device=DEV)
        run(qd[first:].contiguous(), k_pool, v_pool, out, tiles, table, scale=scale, window=window, error_word=word,
            sinks=sd, gates=gd[first:].contiguous())
        close(out, want[first:], dtype, name)
    rows = torch.tensor([0, 1, 15, 16, 63, 64, 65, 200, 299])
    for batch in (rows, rows[-2:]):                           # many rows: splits through memory; two rows: a cluster merges
        out = torch.zeros(len(batch), heads, d, dtype=dtype, device=DEV)
        ops.decode_attention(qd[batch.to(DEV)].contiguous(), k_pool, v_pool, out, batch.int().to(DEV),
                             torch.zeros(len(batch), dtype=torch.int32, device=DEV), table, scale=scale, window=window,
                             scratch_acc=torch.zeros(1 << 20, device=DEV), scratch_ml=torch.zeros(1 << 16, device=DEV),
                             counters=torch.zeros(256, dtype=torch.int32, device=DEV), error_word=word, sinks=sd,
                             gates=gd[batch.to(DEV)].contiguous(), max_keys=300 if len(batch) == 2 else None)
        close(out, want[batch.numpy()], dtype, f"split keys, {len(batch)} rows")
    ops.raise_on_error_word(word)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latents_with_interleaved_stretched_rotation_and_a_gate_per_entry(dtype):
    from sglang_rs_b200 import ops
    g = torch.Generator().manual_seed(4)
    rows, q_rank, kv_rank, rot_dim, heads, eps = 7, 12, 20, 6, 3, 1e-5
    rot = {"base": 300.0, "dims": rot_dim, "scaling": th.STRETCH}
    freq, magnitude = pt.frequencies(rot)
    inv_freq = torch.tensor(freq, dtype=torch.float32, device=DEV)
    proj = torch.randn(rows, q_rank + kv_rank + rot_dim + 5, generator=g)
    qw, kw = torch.rand(q_rank, generator=g) + 0.5, torch.rand(kv_rank, generator=g) + 0.5
    positions = torch.tensor([0, 1, 2, 63, 64, 1000, 4097], dtype=torch.int32)
    pool = torch.zeros(3, 1, 4, kv_rank + rot_dim, dtype=dtype, device=DEV)
    slots = torch.tensor([3, 0, 11, 5, 6, 9, 2], dtype=torch.int32)
    q_latent = torch.zeros(rows, q_rank, dtype=dtype, device=DEV)
    word = ops.new_error_word(DEV)
    ops.latent_prepare(proj.to(dtype).to(DEV), q_rank, kv_rank, rot_dim, qw.to(DEV), kw.to(DEV), eps, positions.to(DEV), inv_freq,
                       rot_dim, q_latent, pool, slots.to(DEV), word, interleaved=True, magnitude=magnitude)
    ops.raise_on_error_word(word)
    x = seen(proj, dtype)
    close(q_latent, pt.rms(x[:, :q_rank], eps) * qw.double().numpy(), dtype, "query latent")
    stored = pool.view(-1, kv_rank + rot_dim)[slots.long().to(DEV)]
    close(stored[:, :kv_rank], pt.rms(x[:, q_rank:q_rank + kv_rank], eps) * kw.double().numpy(), dtype, "latent")
    turned = pt.rotate(x[:, None, q_rank + kv_rank:q_rank + kv_rank + rot_dim], positions.numpy(), rot, True)[:, 0]
    close(stored[:, kv_rank:], turned, dtype, "shared key part, interleaved pairs, stretched")
    # a slice of every head, the same rotation
    heads_in = torch.randn(rows, heads, 4 + rot_dim, generator=g)
    out = torch.zeros(rows, heads, 9 + rot_dim, dtype=dtype, device=DEV)
    ops.rope_slice(heads_in.to(dtype).to(DEV), 4, out, 9, rot_dim, rot_dim, positions.to(DEV), inv_freq, interleaved=True,
                   magnitude=magnitude)
    close(out[:, :, 9:], pt.rotate(seen(heads_in, dtype)[:, :, 4:], positions.numpy(), rot, True), dtype, "rotated slice of every head")
    # one matrix per head with a gate per entry of the result
    n_in, n_out = 10, 6
    a, w, gate = torch.randn(rows, heads, n_in, generator=g), torch.randn(heads, n_out, n_in, generator=g), torch.randn(rows, heads * n_out + 2, generator=g)
    result = torch.zeros(rows, heads, n_out, dtype=dtype, device=DEV)
    ops.head_linear(a.to(dtype).to(DEV), w.to(dtype).to(DEV), result, gate=gate.to(dtype).to(DEV), gate_per_entry=True)
    want = np.einsum("rhi,hoi->rho", seen(a, dtype), seen(w, dtype)) * pt.sigmoid(seen(gate, dtype)[:, :heads * n_out]).reshape(rows, heads, n_out)
    close(result, want, dtype, "per-head product with a gate per entry")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,identity,top,rows,shared", [(5, 3, 2, 9, True), (2, 6, 3, 200, False), (4, 0, 1, 33, True),
                                                              (1, 1, 2, 140, True)])
def test_experts_with_and_without_tensors(dtype, experts, identity, top, rows, shared):
    """Softmax over all router outputs, the choice by score + correction, the scores themselves as weights, outputs
    behind the experts' standing for experts that return their input, an expert that all rows share; few rows and many
    (the grouped products gather only the slots that the plan handed out)."""
    from sglang_rs_b200.parts import GatedMlp, GatedMlpNames, RoutedExperts
    g = torch.Generator().manual_seed(experts * 10 + identity)
    width, ff = 40, 24
    names = lambda e: GatedMlpNames(gate=f"p.e{e}.gate", up=f"p.e{e}.up", down=f"p.e{e}.down")
    part = RoutedExperts(width, ff, experts, top, "silu", "p.router", names, choice_bias_name="p.correction", identity=identity,
                         shared=GatedMlp(width, 16, "silu", names("s"), float_result=True) if shared else None)
    stored = {name: (torch.randn(spec.shape, generator=g) * (3.0 if name == "p.router" else 0.3)).to(dtype)
              for name, spec in part.tensor_specs().items()}
    stored["p.correction"] = (torch.randn(experts + identity, generator=g) * 0.3).to(dtype)
    part.load(stored, DEV, dtype)
    h = torch.randn(rows, width, generator=g)

    class Ctx:
        error_word = None
    from sglang_rs_b200 import ops
    Ctx.error_word = ops.new_error_word(DEV)
    out = part.forward(Ctx, h.to(dtype).to(DEV))
    ops.raise_on_error_word(Ctx.error_word)
    w = {k: v.double().numpy() for k, v in stored.items()}
    w.update({k.replace("p.es.", "p.shared."): v for k, v in w.items() if k.startswith("p.es.")})
    f = {"router": {"experts": experts, "identity": identity, "top": top}, "shared": shared}
    want = pt.routed(seen(h, dtype), w, "p.", f)
    assert out.dtype == torch.float32
    errors = np.abs(out.double().cpu().numpy() - want).max(axis=1) / np.abs(want).max()
    limit = 2e-5 if dtype == torch.float32 else 3e-2
    assert (errors > limit).sum() <= (0 if dtype == torch.float32 else 0.03 * rows), float(errors.max())


# ------------------------------------------------------------------------------ whole models, every way of cutting
@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
@pytest.mark.parametrize("doc", [th.SMALL_A, th.SMALL_B, th.SMALL_C, th.SMALL_D, th.SMALL_E], ids="abcde")
def test_prompts_tails_portions_and_mixed_batches(tmp_path, doc, dtype_name, stored, tolerance):
    folder = th.make_folder(tmp_path, "m", doc, seed=5, dtype=stored)
    requests = th.random_requests(doc, (1, 2, 23, 64, 65, 150, 131), seed=3)
    expected = th.oracle(folder, requests)
    worst = {}
    for name, trace, page in (("whole", rh.trace_whole(requests), 16), ("tail", rh.trace_tail_by_one(requests, tail=45), 16),
                              ("portions", rh.trace_portions(requests), 8), ("mixed", rh.trace_mixed(requests, seed=9), 16)):
        # the pool holds what is live at any time and no more, so pages go from one request to the next
        rows, session = rh.run_in_process(folder, dtype_name, trace, page_size=page)
        assert all(len(rows[rid]) == len(tokens) for rid, tokens in requests.items())
        worst[name] = rh.worst_error(rows, expected)
        th.assert_rows_close(rows, expected, tolerance, dtype_name, name)
        if name == "mixed":
            assert any(len(owners) > 1 for owners in session.page_owners.values()), "no page was used again"
    print(doc["width"], dtype_name, worst)


def test_layers_one_by_one_against_the_plain_stream(tmp_path):
    """The residual stream after every layer run (a layer of the stretch counts each time), 32-bit, a prompt in one step."""
    from sglang_rs_b200.engine.replay import ReplaySession
    folder = th.make_folder(tmp_path, "m", th.SMALL_A, seed=2, dtype=torch.float32)
    doc, w = th.load_folder(folder)
    tokens = th.random_requests(doc, (50,), seed=6)["r0"]
    after = []
    logits = pt.forward(doc, w, tokens, after)
    session = ReplaySession(folder, "float32", 64, 16, use_cuda_graphs=False)
    streams = []
    for block in session.model.layers:
        def forward(ctx, cache, residual, delta, inner=block.forward):
            residual, delta = inner(ctx, cache, residual, delta)
            _, weight, _, eps = delta.norm.spec()[:4]              # the normed term that the next kernel will add
            streams.append(residual.double().cpu().numpy() + pt.rms(delta.values.double().cpu().numpy(), eps) * weight.double().cpu().numpy())
            return residual, delta
        block.forward = forward
    out = session.run({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": list(range(len(tokens)))}], "end": ["a"]})
    assert len(streams) == len(after) == 8
    for index, (got, want) in enumerate(zip(streams, after)):
        assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max(), f"stream after layer run {index}"
    assert np.abs(out - logits).max() <= 2e-5 * np.abs(logits).max()


def test_the_cut_and_the_batch_change_nothing_beyond_rounding(tmp_path):
    """In 32-bit the logits of a position agree to rounding whatever the portions, the pages and the requests beside it."""
    folder = th.make_folder(tmp_path, "m", th.SMALL_A, seed=6, dtype=torch.float32)
    requests = th.random_requests(th.SMALL_A, (40, 97, 130), seed=4)
    whole, _ = rh.run_in_process(folder, "float32", rh.trace_whole(requests), page_size=16)
    for trace, page in ((rh.trace_portions(requests, sizes=(2, 2, 3, 33, 2, 15)), 4), (rh.trace_mixed(requests, seed=2, max_live=3), 32)):
        rows, _ = rh.run_in_process(folder, "float32", trace, page_size=page)
        for rid in requests:
            for pos, row in rows[rid].items():
                assert float(np.abs(row - whole[rid][pos]).max()) <= 2e-5 * float(np.abs(whole[rid][pos]).max()), (rid, pos)


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
@pytest.mark.parametrize("window", [16, 33, 96])
def test_a_marked_key_just_inside_and_just_outside_the_window(tmp_path, window, dtype_name, stored, tolerance):
    """A model made so that head 0 looks at the marked token only (``titatar_helpers.marked_folder``).  The row that is
    window - 1 positions behind it still sees it, the next one does not: in a whole prompt, decoded token by token (the
    window passes over decoded tokens and pages behind it go back to the pool), and in portions cut at the edge."""
    folder = th.marked_folder(tmp_path, stored, "attention", window)
    doc, w = th.load_folder(folder)
    for mark in (0, 7, 31):
        tokens = [th.PLAIN_TOKEN if t == th.MARK_TOKEN else t for t in th.random_requests(doc, (mark + window + 12,), seed=mark)["r0"]]
        tokens[mark] = th.MARK_TOKEN
        requests = {"r0": tokens}
        expected = th.oracle(folder, requests)
        plain = pt.forward(doc, w, tokens[:mark] + [th.PLAIN_TOKEN] + tokens[mark + 1:])
        inside, outside = mark + window - 1, mark + window
        assert np.abs(plain[inside] - expected["r0"][inside]).max() > 0.3 * np.abs(expected["r0"]).max(), "the marked key decides nothing"
        assert np.abs(plain[outside] - expected["r0"][outside]).max() == 0.0
        traces = (rh.trace_whole(requests), rh.trace_tail_by_one(requests, tail=window + 11),
                  rh.trace_portions(requests, sizes=(inside, 1, 1, 2)), rh.trace_portions(requests, sizes=(mark + 1, 2, window - 4, 2, 2, 3)))
        for trace in traces:
            rows, _ = rh.run_in_process(folder, dtype_name, trace, page_size=16)
            th.assert_rows_close(rows, expected, tolerance, dtype_name, (window, mark))


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
def test_a_far_key_at_a_page_border_decides_the_logits(tmp_path, dtype_name, stored, tolerance):
    """Attention over latents has no window: the logits of late positions hang on a key 280 tokens back, the last one of a
    page or the first one of the next, in whole prompts, in decoded tokens and in portions."""
    folder = th.marked_folder(tmp_path, stored, "latent_attention")
    doc, w = th.load_folder(folder)
    for mark in (15, 16):
        tokens = [th.PLAIN_TOKEN if t == th.MARK_TOKEN else t for t in th.random_requests(doc, (300,), seed=mark)["r0"]]
        tokens[mark] = th.MARK_TOKEN
        requests = {"r0": tokens}
        expected = th.oracle(folder, requests)
        plain = pt.forward(doc, w, tokens[:mark] + [th.PLAIN_TOKEN] + tokens[mark + 1:])
        assert np.abs(plain[-1] - expected["r0"][-1]).max() > 0.3 * np.abs(expected["r0"]).max(), "the far key decides nothing"
        for trace in (rh.trace_whole(requests), rh.trace_tail_by_one(requests, tail=40), rh.trace_portions(requests, sizes=(17, 2, 30))):
            rows, _ = rh.run_in_process(folder, dtype_name, trace, page_size=16)
            th.assert_rows_close(rows, expected, tolerance, dtype_name, mark)


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
def test_long_decoding_from_the_first_token(tmp_path, dtype_name, stored, tolerance):
    """Two tokens of prompt, then 300 decoded one by one (windows pass, pages go back, several key splits); beside it a
    request that is fed token by token from position 0.  The decode steps replay captured graphs."""
    # (routers and gates spread less than elsewhere: one sequence of 300 tokens has to stay within the rule on close calls)
    folder = th.make_folder(tmp_path, "m", th.SMALL_D, seed=8, dtype=stored, router=4.0, gate=4.0)
    requests = th.random_requests(th.SMALL_D, (302, 9), seed=5)
    expected = th.oracle(folder, requests)
    long, short = requests["r0"], requests["r1"]
    trace = [{"entries": [{"id": "r0", "tokens": long[:2], "want": [0, 1]}], "end": []}]
    for p in range(2, len(long)):
        entries = [{"id": "r0", "tokens": [long[p]], "want": [0]}]
        if p - 2 < len(short):
            entries.append({"id": "r1", "tokens": [short[p - 2]], "want": [0]})
        trace.append({"entries": entries, "end": ["r1"] if p - 2 == len(short) - 1 else []})
    trace[-1]["end"] = ["r0"]
    for i, step in enumerate(trace):
        step["step"] = i
    rows, session = rh.run_in_process(folder, dtype_name, trace)
    th.assert_rows_close(rows, expected, tolerance, dtype_name)
    assert len(rows["r0"]) == 302 and len(rows["r1"]) == 9
    assert session.runner.graphs is not None and session.runner.graphs.replays > 200


@pytest.mark.parametrize("dtype_name,stored", [("float32", torch.float32), ("bfloat16", torch.bfloat16)])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype_name, stored):
    from sglang_rs_b200 import Engine
    folder = th.make_folder(tmp_path, "m", th.SMALL_A, seed=11, dtype=stored)
    doc, w = th.load_folder(folder)
    prompts = list(th.random_requests(th.SMALL_A, (5, 17, 33, 70), seed=8).values())
    engine = Engine(model_path=folder, dtype=dtype_name, page_size=16, max_total_tokens=400, max_running_requests=3,
                    chunked_prefill_size=16)
    results = engine.generate(prompts, {"max_new_tokens": 12})
    for prompt, result in zip(prompts, results):
        assert result["finished"] and len(result["output_ids"]) == 12
        tokens = list(prompt)
        for token in result["output_ids"]:
            logits = pt.forward(doc, w, tokens)[-1]
            best = int(np.argmax(logits))
            limit = 0.0 if dtype_name == "float32" else 4e-2
            assert float(logits[best] - logits[token]) <= limit * float(np.abs(logits).max()), (prompt[:4], token, best)
            tokens.append(token)
    again = Engine(model_path=folder, dtype=dtype_name, page_size=8, max_total_tokens=400, max_running_requests=1,
                   chunked_prefill_size=7, disable_cuda_graph=True)
    if dtype_name == "float32":
        assert [again.generate(p, {"max_new_tokens": 12})["output_ids"] for p in prompts] == [r["output_ids"] for r in results]
    engine.cache.check_invariants()
    assert engine.flush_cache()
    assert all(a.free_count == a.num_pages for a in engine.cache.allocators.values())


def test_the_command_line_and_the_trace_program_take_the_design(tmp_path):
    """`sglang-rs random-model` writes a folder from a configuration, `sglang-rs generate` decodes from it, and `trace_run`
    replays steps on it: the same programs as for every model."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(th.SMALL_C))
    folder = str(tmp_path / "written")
    made = subprocess.run([sys.executable, os.path.join(root, "bin", "sglang-rs"), "random-model", "--config", str(config_path),
                           "--out", folder, "--seed", "4", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr[-2000:]
    doc, w = th.load_folder(folder)
    command = [sys.executable, os.path.join(root, "bin", "sglang-rs"), "generate", f"--model-path={folder}", "--device", "cuda",
               "--dtype", "float32", "--input-ids", "5,17,3", "--input-ids", "9 8 7 6", "--max-new-tokens", "5",
               "--max-total-tokens", "256"]
    process = subprocess.run(command, capture_output=True, text=True, timeout=600)
    assert process.returncode == 0, process.stderr[-2000:]
    lines = [json.loads(line) for line in process.stdout.strip().splitlines()]
    assert [l["output_ids"] for l in lines] == [th.plain_greedy(doc, w, p, 5) for p in ([5, 17, 3], [9, 8, 7, 6])]
    tokens = th.random_requests(doc, (37,), seed=1)["r0"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[30:], "want": [6]}], "end": ["a"]}]
    out = tmp_path / "out"
    replay = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                             "--out", str(out), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                            capture_output=True, text=True, timeout=600)
    assert replay.returncode == 0 and replay.stdout.split() == ["done", "0", "done", "1"], replay.stderr[-2000:]
    want = pt.forward(doc, w, tokens)
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    last = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    for got, pos in ((first[0], 0), (first[1], 29), (last[0], 36)):
        assert float(np.abs(got - want[pos]).max()) <= 2e-5 * float(np.abs(want).max())
