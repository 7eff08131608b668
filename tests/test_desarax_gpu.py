"""Desarax on the GPU against the plain implementation: each mechanism alone, whole prompts, prompts with a tail decoded
token by token, portions down to two tokens, mixed batches over a small pool (pages and state slots are used again), keys
just inside and just outside a window (a layer's own and that of the layer that reads its latents), a state that must
survive hundreds of tokens, long decoding from captured graphs, and greedy generation through the entry point, the command
line and the trace program."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import desarax_helpers as dh
import plain_desarax as pd
import replay_helpers as rh

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [("float32", torch.float32, 1e-4), ("bfloat16", torch.bfloat16, 4e-2)]
BOTH = [torch.float32, torch.bfloat16]


def seen(tensor, dtype):
    """What the kernel sees of a tensor: rounded to the storage type, as float64."""
    return tensor.to(dtype).to(torch.float64)


def close(got, want, dtype, what, fraction=None):
    tolerance = fraction if fraction is not None else (2e-5 if dtype == torch.float32 else 2e-2)
    scale = float(want.abs().max()) or 1.0
    error = float((got.detach().cpu().to(torch.float64) - want).abs().max()) / scale
    assert error <= tolerance, (what, error)


def dev(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("width,groups", [(48, 3), (70, 1), (36, 2), (256, 8), (30, 30)])
def test_norm_in_equal_parts_of_the_row(dtype, width, groups):
    """residual += delta; out = every part of the row over its own root mean square, times the weight over the whole row;
    as the norm of a delta (with a factor) that is added before the next norm; on picked rows."""
    from sglang_rs_b200 import ops
    torch.manual_seed(width)
    rows, eps = 11, 1e-3
    x, delta = torch.randn(rows, width) * 3, torch.randn(rows, width)
    x[:, :width // groups] *= 20                              # one part far larger than the others: a mean over the row shows
    w_in, w_out = torch.rand(width) + 0.5, torch.rand(width) + 0.5
    on = x.to(DEV)
    out = torch.empty((rows, width), dtype=dtype, device=DEV)
    ops.norm_add_norm(on, delta.to(DEV, dtype), ("rms", w_in.to(DEV), None, eps, 1, 0.7), ("rms", w_out.to(DEV), None, eps, groups, 1.0), out)
    total = x.double() + 0.7 * pd.group_norm(seen(delta, dtype), w_in.double(), 1, eps)
    close(on, total, torch.float32, "the sum", 1e-6)
    close(out, pd.group_norm(total, w_out.double(), groups, eps), dtype, "the norm in parts")
    index = dev([7, 0, 3])
    picked = torch.empty((3, width), dtype=dtype, device=DEV)
    ops.norm_add_norm(on, None, None, ("rms", w_out.to(DEV), None, eps, groups, 1.0), picked, row_index=index, write_residual=False)
    close(picked, pd.group_norm(total, w_out.double(), groups, eps)[[7, 0, 3]], dtype, "picked rows")


@pytest.mark.parametrize("dtype", BOTH)
def test_sum_of_two_sublayers_times_a_factor(dtype):
    from sglang_rs_b200 import ops
    torch.manual_seed(1)
    rows, width = 9, 70
    x, a, b = torch.randn(rows, width), torch.randn(rows, width), torch.randn(rows, width)
    parts = torch.randn(3, rows, width)
    on = x.to(DEV)
    rounded = torch.empty((rows, width), dtype=dtype, device=DEV)
    ops.scaled_sum(on, a.to(DEV, dtype), b.to(DEV), 0.6, rounded)
    want = x.double() + 0.6 * (seen(a, dtype) + b.double())
    close(on, want, torch.float32, "one rounded term and one 32-bit term", 1e-6)
    close(rounded, want, dtype, "the rounded copy")
    ops.scaled_sum(on, parts.to(DEV), None, -1.5)
    close(on, want - 1.5 * parts.double().sum(0), torch.float32, "partial sums alone", 1e-6)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("dim,offset,table_width", [(10, 20, 50), (6, 0, 6), (72, 72, 150)])
def test_gate_times_the_layers_slice_of_the_tokens_row(dtype, dim, offset, table_width):
    from sglang_rs_b200 import ops
    torch.manual_seed(dim)
    rows, vocab = 13, 40
    gate, table = torch.randn(rows, dim) * 2, torch.randn(vocab, table_width)
    ids = torch.randint(0, vocab, (rows,))
    out = torch.empty((rows, dim), dtype=dtype, device=DEV)
    word = ops.new_error_word(DEV)
    ops.token_gate(gate.to(DEV, dtype), ids.to(DEV, torch.int32), table.to(DEV, dtype), offset, out, word)
    close(out, pd.gelu_tanh(seen(gate, dtype)) * seen(table, dtype)[ids][:, offset:offset + dim], dtype, "gate times slice")
    assert int(word.item()) == 0


def mamba_inputs(heads, vdim, nstate, groups, taps, rows, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    inner, channels = heads * vdim, heads * vdim + 2 * groups * nstate
    w = {"conv": torch.randn(channels, taps, generator=g) * 0.5, "conv.b": torch.randn(channels, generator=g) * 0.3,
         "dt_bias": torch.rand(heads, generator=g) * 4 - 3, "A_log": torch.rand(heads, generator=g) * 6 - 5,
         "D": torch.randn(heads, generator=g)}
    proj = torch.randn(rows, 2 * inner + 2 * groups * nstate + heads + 3, generator=g)     # three spare entries behind a row
    return w, proj


def plain_mixer_core(proj, w, sizes, dtype, inputs_before, state_before):
    """The convolution, SiLU and the recurrence of one request's rows from what came before: ``inputs_before``
    [taps - 1, channels] (zeros before the start) and the states [heads, N, P].  Returns (convolved inputs, y, last
    inputs, last states)."""
    heads, P, N, G, taps = sizes["heads"], sizes["vdim"], sizes["nstate"], sizes["groups"], sizes["taps"]
    inner, channels = heads * P, heads * P + 2 * G * N
    x = seen(proj, dtype)
    T = x.shape[0]
    u = torch.cat([inputs_before, x[:, inner:inner + channels]])
    conv = pd.causal_conv(u, w["conv"].double(), w["conv.b"].double())[taps - 1:]
    xbc = pd.silu(conv)
    dt = pd.softplus(x[:, inner + channels:inner + channels + heads] + w["dt_bias"].double())
    y, last = pd.recurrence(xbc[:, :inner].reshape(T, heads, P), xbc[:, inner:inner + G * N].reshape(T, G, N),
                            xbc[:, inner + G * N:].reshape(T, G, N), dt, w["A_log"].double(), w["D"].double(), state_before)
    return xbc, y.reshape(T, inner), u[u.shape[0] - (taps - 1):], last


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,vdim,nstate,groups,taps", [(4, 12, 8, 2, 4), (2, 64, 128, 1, 4), (3, 10, 6, 3, 3), (1, 24, 8, 1, 1),
                                                           (6, 4, 20, 3, 5), (2, 7, 200, 1, 2), (8, 64, 64, 4, 4)])
def test_state_space_mixer_over_states_in_slots(dtype, heads, vdim, nstate, groups, taps):
    """Four requests in one step (a prompt from position 0 in a slot that holds rubbish, a one-token prompt, a later
    portion from a given state, one decoded token), then a second step that continues them from what the first left
    (a portion shorter than the filter among them); a read-only run changes nothing."""
    from sglang_rs_b200 import ops
    sizes = dict(heads=heads, vdim=vdim, nstate=nstate, groups=groups, taps=taps)
    inner, channels = heads * vdim, heads * vdim + 2 * groups * nstate
    counts, starts, slots = [45, 1, 33, 1], [0, 0, 70, 9], [2, 5, 0, 3]
    counts2, slots2 = [2, 38, 1, 130], [2, 0, 3, 5]             # requests 0, 2, 3, 1 go on
    order2 = [0, 2, 3, 1]
    total, total2 = sum(counts), sum(counts2)
    w, proj = mamba_inputs(heads, vdim, nstate, groups, taps, total + total2, nstate + taps, dtype)
    floats = ops.mamba_slot_floats(**sizes)
    state = torch.randn(6, floats, device=DEV)
    given = state.cpu().double()
    weights = {k: v.to(DEV) for k, v in w.items()}

    def unpack(slot_row):
        return (slot_row[:(taps - 1) * channels].reshape(taps - 1, channels),
                slot_row[(taps - 1) * channels:].reshape(heads, vdim, nstate).transpose(1, 2))

    def run(rows, counts, starts, slots, read_only=False):
        cu = np.cumsum([0] + counts).tolist()
        positions = [s + i for s, c in zip(starts, counts) for i in range(c)]
        row_request = [r for r, c in enumerate(counts) for _ in range(c)]
        on = proj[rows].to(DEV, dtype)
        xbc = torch.full((len(positions), channels), float("nan"), device=DEV)
        ops.mamba_conv(on, weights["conv"], weights["conv.b"], dev(positions), dev(row_request), dev(cu), dev(slots), state, xbc,
                       len(counts), read_only=read_only, **sizes)
        y = torch.full((len(positions), inner), float("nan"), device=DEV)
        ops.mamba_scan(on, xbc, weights["A_log"], weights["D"], weights["dt_bias"], dev(positions), dev(cu), dev(slots), state, y,
                       len(counts), read_only=read_only, **sizes)
        return cu, xbc, y

    cu, xbc, y = run(slice(0, total), counts, starts, slots)
    after = {}
    for r in range(4):
        rows = slice(cu[r], cu[r + 1])
        inputs, begin = unpack(given[slots[r]])
        if starts[r] == 0:
            inputs, begin = torch.zeros_like(inputs), torch.zeros_like(begin)
        want_xbc, want_y, last_inputs, last = plain_mixer_core(proj[rows], w, sizes, dtype, inputs, begin)
        after[r] = (last_inputs, last)
        close(xbc[rows], want_xbc, torch.float32, f"convolved inputs of request {r}", 3e-5)
        close(y[rows], want_y, torch.float32, f"request {r}", 3e-5)
        kept_inputs, kept = unpack(state[slots[r]].cpu().double())
        close(kept, last, torch.float32, f"state of request {r}", 3e-5)
        if taps > 1:
            close(kept_inputs, last_inputs, torch.float32, f"kept inputs of request {r}", 1e-6)
    close(state[1], given[1], torch.float32, "a slot that no request holds", 0.0)
    starts2 = [starts[r] + counts[r] for r in order2]
    before = state.clone()
    for read_only in (True, False):
        cu2, xbc2, y2 = run(slice(total, total + total2), counts2, starts2, slots2, read_only=read_only)
        if read_only:
            assert torch.equal(state, before)
        for i, r in enumerate(order2):
            rows = slice(total + cu2[i], total + cu2[i + 1])
            want_xbc, want_y, last_inputs, last = plain_mixer_core(proj[rows], w, sizes, dtype, *after[r])
            close(y2[cu2[i]:cu2[i + 1]], want_y, torch.float32, f"second step, request {r}", 3e-5)
            if not read_only:
                kept_inputs, kept = unpack(state[slots2[i]].cpu().double())
                close(kept, last, torch.float32, f"second step, state of request {r}", 3e-5)
                if taps > 1:
                    close(kept_inputs, last_inputs, torch.float32, f"second step, kept inputs of request {r}", 1e-6)


@pytest.mark.parametrize("heads,vdim,nstate,groups,taps", [(8, 64, 64, 4, 4), (2, 64, 128, 1, 4), (4, 128, 64, 2, 3), (2, 128, 128, 2, 2)])
def test_state_space_mixer_in_chunks_on_the_tensor_cores(heads, vdim, nstate, groups, taps):
    """Prompt portions in bfloat16 run as chunks of 128 tokens in parallel: four requests in one step (a prompt of more
    than two chunks from position 0 in a slot that holds rubbish, a one-token prompt, a later portion of one chunk and
    one token from a given state, a portion of exactly one chunk), then a second step that continues them.  The
    recurrence is checked against the plain one over the convolved inputs as the kernel rounded them, so what is left is
    the error of the chunked arithmetic; the states go on into the token-by-token kernel."""
    from sglang_rs_b200 import ops
    dtype = torch.bfloat16
    sizes = dict(heads=heads, vdim=vdim, nstate=nstate, groups=groups, taps=taps)
    inner, channels = heads * vdim, heads * vdim + 2 * groups * nstate
    counts, starts, slots = [300, 1, 129, 128], [0, 0, 70, 9], [2, 5, 0, 3]
    counts2, slots2 = [2, 257, 1, 130], [2, 0, 3, 5]            # requests 0, 2, 3, 1 go on
    order2 = [0, 2, 3, 1]
    total, total2 = sum(counts), sum(counts2)
    w, proj = mamba_inputs(heads, vdim, nstate, groups, taps, total + total2, nstate + taps, dtype)
    state = torch.randn(6, ops.mamba_slot_floats(**sizes), device=DEV)
    given = state.cpu().double()
    weights = {k: v.to(DEV) for k, v in w.items()}

    def unpack(slot_row):
        return (slot_row[:(taps - 1) * channels].reshape(taps - 1, channels),
                slot_row[(taps - 1) * channels:].reshape(heads, vdim, nstate).transpose(1, 2))

    def run(rows, counts, starts, slots, chunked=True, read_only=False):
        cu = np.cumsum([0] + counts).tolist()
        positions = [s + i for s, c in zip(starts, counts) for i in range(c)]
        row_request = [r for r, c in enumerate(counts) for _ in range(c)]
        on = proj[rows].to(DEV, dtype)
        xbc = torch.full((len(positions), channels), float("nan"), device=DEV, dtype=dtype if chunked else torch.float32)
        ops.mamba_conv(on, weights["conv"], weights["conv.b"], dev(positions), dev(row_request), dev(cu), dev(slots), state, xbc,
                       len(counts), read_only=read_only, **sizes)
        y = torch.full((len(positions), inner), float("nan"), device=DEV)
        if chunked:
            chunks = sum(-(-c // ops.MAMBA_CHUNK_TOKENS) for c in counts)
            ops.mamba_chunks(on, xbc, weights["A_log"], weights["D"], weights["dt_bias"], dev(positions), dev(cu), dev(slots), state,
                             y, len(counts), chunks, read_only=read_only, **sizes)
        else:
            ops.mamba_scan(on, xbc, weights["A_log"], weights["D"], weights["dt_bias"], dev(positions), dev(cu), dev(slots), state, y,
                           len(counts), read_only=read_only, **sizes)
        return cu, xbc, y

    def plain(rows, xbc, begin):
        steps = pd.softplus(seen(proj[rows], dtype)[:, inner + channels:inner + channels + heads] + w["dt_bias"].double())
        x = xbc.cpu().double()
        T = x.shape[0]
        y, last = pd.recurrence(x[:, :inner].reshape(T, heads, vdim), x[:, inner:inner + groups * nstate].reshape(T, groups, nstate),
                                x[:, inner + groups * nstate:].reshape(T, groups, nstate), steps, w["A_log"].double(), w["D"].double(), begin)
        return y.reshape(T, inner), last

    cu, xbc, y = run(slice(0, total), counts, starts, slots)
    after = {}
    for r in range(4):
        rows = slice(cu[r], cu[r + 1])
        inputs, begin = unpack(given[slots[r]])
        if starts[r] == 0:
            inputs, begin = torch.zeros_like(inputs), torch.zeros_like(begin)
        want_xbc, _, last_inputs, _ = plain_mixer_core(proj[rows], w, sizes, dtype, inputs, begin)
        close(xbc[rows], want_xbc, dtype, f"convolved inputs of request {r}", 6e-3)
        want_y, last = plain(rows, xbc[rows], begin)
        after[r] = (last_inputs, last)
        close(y[rows], want_y, torch.float32, f"request {r}", 1e-4)
        kept_inputs, kept = unpack(state[slots[r]].cpu().double())
        close(kept, last, torch.float32, f"state of request {r}", 1e-4)
        close(kept_inputs, last_inputs, torch.float32, f"kept inputs of request {r}", 1e-6)
    close(state[1], given[1], torch.float32, "a slot that no request holds", 0.0)
    starts2 = [starts[r] + counts[r] for r in order2]
    before = state.clone()
    for chunked, read_only in ((True, True), (False, True), (True, False)):
        cu2, xbc2, y2 = run(slice(total, total + total2), counts2, starts2, slots2, chunked=chunked, read_only=read_only)
        if read_only:
            assert torch.equal(state, before)
        for i, r in enumerate(order2):
            rows = slice(total + cu2[i], total + cu2[i + 1])
            want_y, last = plain(rows, xbc2[cu2[i]:cu2[i + 1]], after[r][1])
            close(y2[cu2[i]:cu2[i + 1]], want_y, torch.float32, f"second step, request {r}, chunked {chunked}", 1e-4)
            if not read_only:
                _, kept = unpack(state[slots2[i]].cpu().double())
                close(kept, last, torch.float32, f"second step, state of request {r}", 1e-4)


def test_state_space_mixer_keeps_a_token_through_a_slow_decay():
    """One head decays by 0.9995 a token: after 700 tokens, cut into three steps, the first token still makes up most of
    the result; the head beside it forgets within a few tokens."""
    from sglang_rs_b200 import ops
    sizes = dict(heads=2, vdim=4, nstate=8, groups=1, taps=1)
    inner, channels, T = 8, 24, 700
    proj = torch.zeros(T, 2 * inner + 16 + 2)
    proj[:, inner + inner:inner + inner + 8] = 0.001           # B small everywhere ...
    proj[0, inner + inner:inner + inner + 8] = 3.0             # ... but at the first token
    proj[:, inner:inner + inner] = 1.0                         # x
    proj[:, inner + inner + 8:inner + channels] = 1.0          # C
    w = {"conv": torch.ones(channels, 1), "conv.b": torch.zeros(channels), "dt_bias": torch.zeros(2),
         "A_log": torch.tensor([math.log(0.0005 / math.log(2.0)), 1.0]), "D": torch.zeros(2)}
    state = torch.randn(2, ops.mamba_slot_floats(**sizes), device=DEV)
    ys, at = [], 0
    for count in (300, 399, 1):
        positions = list(range(at, at + count))
        on = proj[at:at + count].to(DEV)
        xbc = torch.empty((count, channels), device=DEV)
        ops.mamba_conv(on, w["conv"].to(DEV), w["conv.b"].to(DEV), dev(positions), dev([0] * count), dev([0, count]), dev([1]), state,
                       xbc, 1, **sizes)
        y = torch.empty((count, inner), device=DEV)
        ops.mamba_scan(on, xbc, w["A_log"].to(DEV), w["D"].to(DEV), w["dt_bias"].to(DEV), dev(positions), dev([0, count]), dev([1]),
                       state, y, 1, **sizes)
        ys.append(y.cpu())
        at += count
    got = torch.cat(ys)
    _, want, _, _ = plain_mixer_core(proj, w, sizes, torch.float32, torch.zeros(0, channels, dtype=torch.float64),
                                     torch.zeros(2, 8, 4, dtype=torch.float64))
    close(got, want, torch.float32, "700 tokens in three steps", 3e-5)
    without = proj.clone()
    without[0, inner + inner:inner + inner + 8] = 0.001
    _, lost, _, _ = plain_mixer_core(without, w, sizes, torch.float32, torch.zeros(0, channels, dtype=torch.float64),
                                     torch.zeros(2, 8, 4, dtype=torch.float64))
    assert float(want[-1, 0]) > 2 * float(lost[-1, 0]) and abs(float(want[-1, 4]) - float(lost[-1, 4])) < 1e-9


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("inner,parts", [(48, 2), (24, 3), (128, 1), (30, 5), (4096, 8)])
def test_gate_before_the_norm_in_parts(dtype, inner, parts):
    from sglang_rs_b200 import ops
    torch.manual_seed(inner)
    rows = 7
    y, proj, weight = torch.randn(rows, inner) * 3, torch.randn(rows, inner + 9), torch.rand(inner) + 0.5
    y[:, :inner // parts] *= 30
    out = torch.empty((rows, inner), dtype=dtype, device=DEV)
    ops.mamba_gate_norm(y.to(DEV), proj.to(DEV, dtype), weight.to(DEV), 1e-4, parts, out)
    want = pd.group_norm(y.double() * pd.silu(seen(proj, dtype)[:, :inner]), weight.double(), parts, 1e-4)
    close(out, want, dtype, "norm of the gated result")
    other = pd.group_norm(y.double(), weight.double(), parts, 1e-4) * pd.silu(seen(proj, dtype)[:, :inner])
    assert float((want - other).abs().max()) > 0.1            # the gate after the norm would be another function


def window_case(dtype, heads, width, value_dim, page, window, seed, lengths=(150, 70, 9)):
    """Requests whose latents lie scattered over shuffled pages; the last 41, 70 and 9 positions are the step's rows.
    Head 0 of the last row of request 0 is made to look at the key just inside its window and, a second query, at the
    key just outside."""
    g = torch.Generator().manual_seed(seed)
    portions = [(0, lengths[0] - 41, 41), (1, 0, lengths[1]), (2, 0, lengths[2])]
    keys = [torch.randn(n, width, generator=g) for n in lengths]
    rows = sum(n for _, _, n in portions)
    q = torch.randn(rows, heads, width, generator=g)
    last = lengths[0] - 1
    inside, outside = last - window + 1, last - window
    if outside >= 0:
        keys[0][inside] = 6.0 * q[40, 0] / q[40, 0].norm()
        keys[0][outside] = 6.0 * q[40, 1 % heads] / q[40, 1 % heads].norm() if heads > 1 else keys[0][outside]
    total_pages = sum(-(-n // page) for n in lengths) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    pool = torch.zeros((total_pages, 1, page, width), dtype=dtype, device=DEV)
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths) + 1), -1, dtype=torch.int32)
    for r, k in enumerate(keys):
        for pos in range(len(k)):
            if pos % page == 0:
                table[r, pos // page] = order.pop()
            pool[table[r, pos // page], 0, pos % page] = k[pos].to(dtype)
    tiles, positions, row_request, first = [], [], [], 0
    for request, start, count in portions:
        for offset in range(0, count, 64):
            tiles.append([first + offset, min(64, count - offset), request, start + offset])
        positions += list(range(start, start + count))
        row_request += [request] * count
        first += count
    return dict(keys=keys, q=q, pool=pool, table=table.to(DEV), tiles=dev(tiles), positions=positions, row_request=row_request,
                rows=rows, inside=inside, outside=outside, dtype=dtype, value_dim=value_dim, window=window)


def plain_window_row(case, row, scale):
    dtype, window = case["dtype"], case["window"]
    pos = case["positions"][row]
    first = max(0, pos - window + 1) if window else 0
    k = seen(case["keys"][case["row_request"][row]], dtype)[first:pos + 1]
    w = torch.softmax(torch.einsum("hd,jd->hj", seen(case["q"], dtype)[row], k) * scale, -1)
    return w, w @ k[:, :case["value_dim"]], first


@pytest.mark.parametrize("heads,width,value_dim,page,window", [(3, 48, 32, 8, 40), (4, 64, 64, 16, 96), (2, 32, 32, 16, 5), (5, 80, 64, 4, 37),
                                                               (2, 64, 32, 16, 64), (3, 32, 32, 8, 500)])
def test_tensor_core_attention_over_latents_inside_a_window(heads, width, value_dim, page, window):
    """The bfloat16 kernel: prompt portions as tiles and decoded rows with split keys see themselves and window - 1 rows
    before; the key just inside the window takes most of head 0's weight, the key just outside none of head 1's."""
    from sglang_rs_b200 import ops
    case = window_case(torch.bfloat16, heads, width, value_dim, page, window, seed=window)
    word = ops.new_error_word(DEV)
    out = torch.full((case["rows"], heads, value_dim), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.latent_attention(case["q"].to(DEV, torch.bfloat16), case["pool"], out, dev(case["positions"]), dev(case["row_request"]),
                         case["table"], scale=0.25, sinks=None, error_word=word, tiles=case["tiles"], window=window)
    for row in range(case["rows"]):
        w, want, first = plain_window_row(case, row, 0.25)
        close(out[row], want, torch.bfloat16, f"portion row {row}")
        if row == 40 and case["outside"] >= 0:
            assert float(w[0, case["inside"] - first]) > 0.5
    picks = [40, 0, case["rows"] - 1, 41, 20]
    splits = (window - 1) // 64 + 2
    acc = torch.empty(len(picks) * heads * splits * value_dim, device=DEV)
    ml = torch.empty(len(picks) * heads * splits * 2, device=DEV)
    single = torch.empty((len(picks), heads, value_dim), dtype=torch.bfloat16, device=DEV)
    ops.latent_attention(case["q"][picks].to(DEV, torch.bfloat16), case["pool"], single, dev([case["positions"][r] for r in picks]),
                         dev([case["row_request"][r] for r in picks]), case["table"], scale=0.25, sinks=None, error_word=word,
                         split_size=64, max_splits=splits, scratch_acc=acc, scratch_ml=ml, window=window)
    for i, row in enumerate(picks):
        close(single[i], plain_window_row(case, row, 0.25)[1], torch.bfloat16, f"decoded row {row}")
    assert int(word.item()) == 0


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,width,value_dim,page,window,split", [(3, 24, 16, 8, 40, 0), (3, 24, 16, 8, 40, 16), (2, 12, 6, 4, 7, 0),
                                                                     (2, 12, 6, 4, 19, 32), (1, 24, 24, 16, 5, 16)])
def test_attention_over_latents_inside_a_window(dtype, heads, width, value_dim, page, window, split):
    """The kernel that takes every size and both dtypes, on the same cases."""
    from sglang_rs_b200 import ops
    case = window_case(dtype, heads, width, value_dim, page, window, seed=window + 1)
    rows = case["rows"]
    splits = ((window - 1) // split + 2) if split else 1
    acc = torch.empty(rows * heads * splits * value_dim, device=DEV)
    ml = torch.empty(rows * heads * splits * 2, device=DEV)
    out = torch.empty((rows, heads, value_dim), dtype=dtype, device=DEV)
    word = ops.new_error_word(DEV)
    ops.paged_attention(case["q"].to(DEV, dtype), case["pool"], None, out, dev(case["positions"]), dev(case["row_request"]), case["table"],
                        scale=0.25, window=window, split_size=split, max_splits=splits, scratch_acc=acc, scratch_ml=ml, error_word=word)
    for row in range(rows):
        w, want, first = plain_window_row(case, row, 0.25)
        close(out[row], want, dtype, f"row {row}")
        if row == 40:
            assert float(w[0, case["inside"] - first]) > 0.5
    assert int(word.item()) == 0


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("experts,top,rows,limit", [(5, 2, 150, 0.7), (3, 3, 9, 2.0), (4, 1, 1, 1.0), (70, 4, 40, 0.5), (3, 2, 500, 1.0),
                                                    (16, 6, 1300, 1.5)])
def test_clamped_experts_chosen_by_sigmoid_scores_with_a_correction(dtype, experts, top, rows, limit):
    from sglang_rs_b200 import ops
    torch.manual_seed(5)
    width, inner = 40, 24
    h = torch.randn(rows, width)
    w = {"router": torch.randn(experts, width) * 0.6, "correction": torch.randn(experts) * 0.5}
    for e in range(experts):
        w.update({f"e{e}.gate": torch.randn(inner, width) * 0.3, f"e{e}.up": torch.randn(inner, width) * 0.3,
                  f"e{e}.down": torch.randn(width, inner) * 0.2})
    gate_up = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)]).to(DEV, dtype)
    down = torch.stack([w[f"e{e}.down"] for e in range(experts)]).to(DEV, dtype)
    word = ops.new_error_word(DEV)
    out = ops.routed_experts(h.to(DEV, dtype), w["router"].to(DEV, dtype), gate_up, down, top, "swiglu_clamp", True, word, scoring="sigmoid",
                             choice_bias=w["correction"].to(DEV), weight_scale=2.5, norm_eps=1e-20, activation_param=limit)
    rounded = {k: (v.double() if k == "correction" else seen(v, dtype)) for k, v in w.items()}
    f = {"router": {"experts": experts, "top": top, "scale": 2.5}, "expert": {"ff": inner, "limit": limit}}
    want = pd.routed_experts(seen(h, dtype), rounded, f)
    assert out.dtype == torch.float32 and int(word.item()) == 0
    close(out, want, dtype, "weighted sum of the chosen experts")
    s = torch.sigmoid(seen(h, dtype) @ rounded["router"].T)
    if top < experts and rows >= 9:          # the correction decides, and the clamp acts
        assert not torch.equal(torch.topk(s, top).indices.sort().values, torch.topk(s + rounded["correction"], top).indices.sort().values)
        assert float((seen(h, dtype) @ rounded["e0.gate"].T).max()) > limit
    chosen, weights = ops.route(h.to(DEV, dtype), w["router"].to(DEV, dtype), top, True, scoring="sigmoid", choice_bias=w["correction"].to(DEV),
                                weight_scale=2.5, norm_eps=1e-20)
    want_chosen, want_weights = pd.route(seen(h, dtype), rounded["router"], rounded["correction"], top, 2.5)
    assert torch.equal(chosen.cpu().long().sort(-1).values, want_chosen.sort(-1).values)
    close(weights.sum(-1), want_weights.sum(-1), torch.float32, "the weights add up to the factor", 1e-5)


# ------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
@pytest.mark.parametrize("doc", [dh.SMALL_A, dh.SMALL_B, dh.SMALL_C, dh.SMALL_D], ids=["a", "b", "c", "d"])
def test_prompts_tails_portions_and_mixed_batches(tmp_path, doc, dtype_name, stored, tolerance):
    folder = dh.make_folder(tmp_path, "m", doc, seed=5, dtype=stored)
    requests = dh.random_requests(doc, (1, 2, 23, 64, 65, 150, 131), seed=3)
    expected = dh.oracle(folder, requests)
    worst = {}
    for name, trace, page in (("whole", rh.trace_whole(requests), 16), ("tail", rh.trace_tail_by_one(requests, tail=45), 16),
                              ("portions", rh.trace_portions(requests), 8), ("mixed", rh.trace_mixed(requests, seed=9), 16)):
        # the pool holds what is live at any time and no more, so pages and state slots go from one request to the next
        rows, session = rh.run_in_process(folder, dtype_name, trace, page_size=page)
        assert all(len(rows[rid]) == len(tokens) for rid, tokens in requests.items())
        worst[name] = rh.worst_error(rows, expected)
        dh.assert_rows_close(rows, expected, tolerance, dtype_name, name)
        if name == "mixed":
            assert any(len(owners) > 1 for owners in session.page_owners.values()), "no page was used again"
            assert len(requests) > session.cache.max_requests, "no state slot was used again"
    print(doc["width"], dtype_name, worst)


def test_layers_one_by_one_against_the_plain_stream(tmp_path):
    """The residual stream after every layer (the token's own input included), 32-bit, for a prompt in one step."""
    from sglang_rs_b200.engine.replay import ReplaySession
    folder = dh.make_folder(tmp_path, "m", dh.SMALL_A, seed=2, dtype=torch.float32)
    doc, tensors = dh.load_folder(folder)
    tokens = dh.random_requests(doc, (50,), seed=6)["r0"]
    logits, after = pd.forward(doc, tensors, tokens, return_layers=True)
    session = ReplaySession(folder, "float32", 64, 16, use_cuda_graphs=False)
    session.model.native = None
    streams = []
    for block in session.model.layers:
        def forward(ctx, cache, residual, delta, inner=block.forward):
            residual, delta = inner(ctx, cache, residual, delta)
            x = residual.double().cpu()
            if delta is not None:                     # what the next norm kernel will add: the normed input of the token
                _, weight, _, eps, groups, scale = delta.norm.spec()
                x = x + pd.group_norm(delta.values.double().cpu(), weight.double().cpu(), groups, eps) * scale
            streams.append(x)
            return residual, delta
        block.forward = forward
    out = session.run({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": list(range(len(tokens)))}], "end": ["a"]})
    assert len(streams) == len(doc["layers"])
    for index, (got, want) in enumerate(zip(streams, after)):
        close(got, want, torch.float32, f"stream after layer {index}")
    close(torch.from_numpy(out), logits, torch.float32, "logits")


def test_the_cut_and_the_batch_change_nothing_beyond_rounding(tmp_path):
    """In 32-bit the logits of a position agree to rounding whatever the portions, the pages, the slots and the requests
    beside it."""
    folder = dh.make_folder(tmp_path, "m", dh.SMALL_A, seed=6, dtype=torch.float32)
    requests = dh.random_requests(dh.SMALL_A, (40, 97, 130, 5, 61), seed=4)
    whole, _ = rh.run_in_process(folder, "float32", rh.trace_whole(requests), page_size=16)
    for trace, page in ((rh.trace_portions(requests, sizes=(2, 2, 3, 33, 2, 15)), 4), (rh.trace_mixed(requests, seed=2, max_live=3), 32)):
        rows, _ = rh.run_in_process(folder, "float32", trace, page_size=page)
        for rid in requests:
            for pos, row in rows[rid].items():
                assert float(np.abs(row - whole[rid][pos]).max()) <= 1e-4 * float(np.abs(whole[rid][pos]).max()), (rid, pos)


def _with_mark(doc, length, place, seed):
    tokens = [dh.FILL if t == dh.MARK else t for t in dh.random_requests(doc, (length,), seed=seed)["r0"]]
    tokens[place] = dh.MARK
    return tokens


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
@pytest.mark.parametrize("shared", [False, True])
def test_a_key_at_the_edge_of_a_window_decides_the_logits(tmp_path, dtype_name, stored, tolerance, shared):
    """A model whose heads look for one token (``desarax_helpers.marked_folder``).  A window of 40 positions over pages of
    16: seen from the last position the mark is the window's first key, or the one before it (not seen), or near; in whole
    prompts, in decoded tokens and in portions cut inside the window.  ``shared``: the layer's own window has 20 positions
    and the layer that reads its latents 40, so the cache must keep what the second one sees."""
    folder = dh.marked_folder(tmp_path, stored, "attention", window=20 if shared else 40, shared=shared)
    doc, tensors = dh.load_folder(folder)
    for place, seen_from_the_end in ((95, True), (94, False), (133, True)) + (((115, True), (114, True)) if shared else ()):
        tokens = _with_mark(doc, 135, place, seed=place)
        requests = {"r0": tokens}
        expected = dh.oracle(folder, requests)
        without = pd.forward(doc, tensors, tokens[:place] + [dh.FILL] + tokens[place + 1:]).numpy()
        decides = np.abs(without[-1] - expected["r0"][-1]).max() > 0.2 * np.abs(expected["r0"]).max()
        assert decides == seen_from_the_end, place
        for trace in (rh.trace_whole(requests), rh.trace_tail_by_one(requests, tail=45), rh.trace_portions(requests, sizes=(17, 2, 30))):
            rows, _ = rh.run_in_process(folder, dtype_name, trace, page_size=16)
            dh.assert_rows_close(rows, expected, tolerance, dtype_name, place)


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
@pytest.mark.parametrize("wide", [False, True])
def test_a_state_keeps_a_token_from_hundreds_of_positions_back(tmp_path, dtype_name, stored, tolerance, wide):
    """The mark at position 3 of 420 tokens, in a model whose state-space head decays by 0.999 a token: the last logits
    hang on it.  A state that is lost between steps, zeroed with a slot or mixed up in a batch shows.  ``wide``: at the
    sizes whose prompt portions in bfloat16 run as parallel chunks, so a chunk's state that does not reach the next shows."""
    folder = dh.marked_folder(tmp_path, stored, "mamba", wide=wide)
    doc, tensors = dh.load_folder(folder)
    tokens = _with_mark(doc, 420, 3, seed=1)
    other = _with_mark(doc, 90, 50, seed=2)
    requests = {"r0": tokens, "r1": other, "r2": tokens[:200]}
    expected = dh.oracle(folder, requests)
    without = pd.forward(doc, tensors, tokens[:3] + [dh.FILL] + tokens[4:]).numpy()
    assert np.abs(without[-1] - expected["r0"][-1]).max() > 0.1 * np.abs(expected["r0"]).max(), "the far token decides nothing"
    for trace in (rh.trace_whole(requests), rh.trace_tail_by_one(requests, tail=40), rh.trace_portions(requests, sizes=(17, 2, 30, 64, 3)),
                  rh.trace_mixed(requests, seed=4, max_live=2)):
        rows, _ = rh.run_in_process(folder, dtype_name, trace, page_size=16)
        dh.assert_rows_close(rows, expected, tolerance, dtype_name)


@pytest.mark.parametrize("dtype_name,stored,tolerance", DTYPES)
def test_long_decoding_from_the_first_token(tmp_path, dtype_name, stored, tolerance):
    """Two tokens of prompt, then 300 decoded one by one (windows pass over decoded tokens, pages behind them are given
    back); beside it a request that is fed token by token from position 0.  The decode steps replay captured graphs."""
    folder = dh.make_folder(tmp_path, "m", dh.SMALL_A, seed=8, dtype=stored)
    requests = dh.random_requests(dh.SMALL_A, (302, 9), seed=5)
    expected = dh.oracle(folder, requests)
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
    dh.assert_rows_close(rows, expected, tolerance, dtype_name)
    assert len(rows["r0"]) == 302 and len(rows["r1"]) == 9
    assert session.runner.graphs is not None and session.runner.graphs.replays > 200


@pytest.mark.parametrize("dtype_name,stored", [("float32", torch.float32), ("bfloat16", torch.bfloat16)])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype_name, stored):
    from sglang_rs_b200 import Engine
    folder = dh.make_folder(tmp_path, "m", dh.SMALL_A, seed=11, dtype=stored)
    doc, tensors = dh.load_folder(folder)
    prompts = list(dh.random_requests(dh.SMALL_A, (5, 17, 33, 70), seed=8).values())
    engine = Engine(model_path=folder, dtype=dtype_name, page_size=16, max_total_tokens=400, max_running_requests=3,
                    chunked_prefill_size=16)
    results = engine.generate(prompts, {"max_new_tokens": 12})
    for prompt, result in zip(prompts, results):
        assert result["finished"] and len(result["output_ids"]) == 12
        tokens = list(prompt)
        for token in result["output_ids"]:
            logits = pd.forward(doc, tensors, tokens)[-1]
            best = int(torch.argmax(logits))
            limit = 0.0 if dtype_name == "float32" else 4e-2
            assert float(logits[best] - logits[token]) <= limit * float(logits.abs().max()), (prompt[:4], token, best)
            tokens.append(token)
    again = Engine(model_path=folder, dtype=dtype_name, page_size=8, max_total_tokens=400, max_running_requests=1,
                   chunked_prefill_size=7, disable_cuda_graph=True)
    if dtype_name == "float32":
        assert [again.generate(p, {"max_new_tokens": 12})["output_ids"] for p in prompts] == [r["output_ids"] for r in results]
    engine.cache.check_invariants()
    assert engine.flush_cache()
    assert all(a.free_count == a.num_pages for a in engine.cache.allocators.values())
    assert engine.cache.state_pool.free_count == engine.cache.max_requests


def test_preemption_on_a_small_pool_gives_the_same_tokens(tmp_path):
    """Three requests on a pool that cannot hold them: a request is preempted, gives its pages and its state slot back
    and is computed again from its first token, in other portions and another slot; every token stays what the plain
    implementation gives (32-bit)."""
    from sglang_rs_b200 import Engine
    folder = dh.make_folder(tmp_path, "m", dh.SMALL_B, seed=4, dtype=torch.float32)
    doc, tensors = dh.load_folder(folder)
    prompts = list(dh.random_requests(dh.SMALL_B, (40, 35, 50), seed=2).values())
    engine = Engine(model_path=folder, dtype="float32", page_size=16, max_total_tokens=160, max_running_requests=3,
                    chunked_prefill_size=64)
    results = engine.generate(prompts, {"max_new_tokens": 40})
    assert engine.scheduler.stats["preemptions"] >= 1
    assert [r["output_ids"] for r in results] == [dh.plain_greedy(doc, tensors, p, 40) for p in prompts]
    assert engine.cache.state_pool.free_count == engine.cache.max_requests


def test_the_command_line_and_the_trace_program_take_the_design(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(dh.SMALL_C))
    folder = str(tmp_path / "written")
    made = subprocess.run([sys.executable, os.path.join(root, "bin", "sglang-rs"), "random-model", "--config", str(config_path),
                           "--out", folder, "--seed", "4", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert made.returncode == 0, made.stderr[-2000:]
    doc, tensors = dh.load_folder(folder)
    command = [sys.executable, os.path.join(root, "bin", "sglang-rs"), "generate", f"--model-path={folder}", "--device", "cuda",
               "--dtype", "float32", "--input-ids", "5,17,3", "--input-ids", "9 8 7 6", "--max-new-tokens", "5",
               "--max-total-tokens", "256"]
    process = subprocess.run(command, capture_output=True, text=True, timeout=600)
    assert process.returncode == 0, process.stderr[-2000:]
    lines = [json.loads(line) for line in process.stdout.strip().splitlines()]
    assert [l["output_ids"] for l in lines] == [dh.plain_greedy(doc, tensors, p, 5) for p in ([5, 17, 3], [9, 8, 7, 6])]
    tokens = dh.random_requests(doc, (37,), seed=1)["r0"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[30:], "want": [6]}], "end": ["a"]}]
    out = tmp_path / "out"
    replay = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                             "--out", str(out), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                            capture_output=True, text=True, timeout=600)
    assert replay.returncode == 0 and replay.stdout.split() == ["done", "0", "done", "1"], replay.stderr[-2000:]
    want = pd.forward(doc, tensors, tokens).numpy()
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    last = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    for got, pos in ((first[0], 0), (first[1], 29), (last[0], 36)):
        assert float(np.abs(got - want[pos]).max()) <= 2e-5 * float(np.abs(want).max())
