"""Pametar on the GPU against the plain implementation: every mechanism's kernel alone, then whole models cut into
steps in every way, then generation through the entry point.

Kernel tests build their own index arrays, slots and pages and compare with the functions of ``plain_pametar`` in
float64.  Where random numbers would hide a fault (a lost state, a sink left out, a far key, a wrong previous token)
the inputs are made so that it shows.  Model tests make small model folders of four configurations that differ in
every size and option (copies of the stream from one to four, loops, layers without feed-forward, every expert or one
chosen, with and without the pair table) and replay requests whole, with a decoded tail, in portions down to two
tokens, and mixed with few pages and slots.
"""

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_pametar as plain
import traces
from pametar_models import pametar_dir

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def step_arrays(portions):
    """portions: list of (slot, start position, count) -> req_of_token, q_start, slots, positions."""
    req, pos, qs, slots = [], [], [0], []
    for r, (slot, start, count) in enumerate(portions):
        req += [r] * count
        pos += list(range(start, start + count))
        qs.append(qs[-1] + count)
        slots.append(slot)
    return i32(req), i32(qs), i32(slots), i32(pos)


def cuts(total, sizes):
    out, at, i = [], 0, 0
    while at < total:
        c = min(sizes[i % len(sizes)], total - at)
        out.append((at, c))
        at += c
        i += 1
    return out


# ---- the copies of the stream: write, read, norm ----------------------------------------------------------------

@pytest.mark.parametrize("copies, width, y_kind", [(1, 36, "float32"), (2, 64, "bfloat16"), (3, 50, "parts"), (4, 128, "bfloat16"),
                                                   (8, 20, "float32")])
def test_stream_step_writes_all_copies_from_the_old_ones_and_reads_their_weighted_sum(copies, width, y_kind):
    from yalis_b200.ops.streams import stream_step
    g = torch.Generator().manual_seed(copies * 100 + width)
    n = 23
    x = torch.randn(n, copies, width, generator=g)
    mix = torch.eye(copies) * 0.7 + 0.3 * torch.randn(copies, copies, generator=g)       # not symmetric: [from, to] shows
    w_out, w_in = torch.randn(copies, generator=g), torch.randn(copies, generator=g)
    scale, bias = 1 + 0.3 * torch.randn(width, generator=g), torch.randn(width, generator=g)
    gate = torch.randn(n, width, generator=g) * 2
    alpha, nw, nb = torch.tensor([0.4]), 1 + 0.2 * torch.randn(width, generator=g), 0.3 * torch.randn(width, generator=g)
    if y_kind == "parts":
        y = torch.randn(3, n, width, generator=g)
        y_sum = y.double().sum(dim=0)
    else:
        y = torch.randn(n, width, generator=g).to(getattr(torch, y_kind))
        y_sum = y.double()
    t = {"n.alpha": alpha.double(), "n": nw.double(), "n.b": nb.double()}
    yy = y_sum * scale.double() * plain.sigmoid(gate.double() + bias.double())
    want_x = plain.write_copies(x.double().transpose(0, 1), mix.double(), w_out.double(), yy)        # [S, N, D]
    want_h = plain.dynamic_tanh(plain.read_copies(want_x, w_in.double()), t, "n")
    xd = x.clone().to(DEV)
    h = stream_step(xd, y=y.to(DEV), gate=gate.to(DEV), gate_bias=bias.to(DEV), layer_scale=scale.to(DEV), mix=mix.to(DEV),
                    out_weights=w_out.to(DEV), in_weights=w_in.to(DEV), norm=(alpha.to(DEV), nw.to(DEV), nb.to(DEV)),
                    out_dtype=torch.float32)
    torch.testing.assert_close(xd.double().cpu().transpose(0, 1), want_x, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(h.double().cpu(), want_h, rtol=1e-5, atol=1e-5)
    # chosen rows only (the last step before the logits): the stream stays, a row of no request is skipped
    xd2 = x.clone().to(DEV)
    rows = [n - 1, 0, 7]
    some = stream_step(xd2, y=y.to(DEV), gate=gate.to(DEV), gate_bias=bias.to(DEV), layer_scale=scale.to(DEV), mix=mix.to(DEV),
                       out_weights=w_out.to(DEV), norm=(alpha.to(DEV), nw.to(DEV), nb.to(DEV)), rows=i32(rows), out_dtype=torch.float32)
    assert torch.equal(xd2.cpu(), x)
    want_sum = plain.dynamic_tanh(want_x.sum(dim=0), t, "n")                                       # no read weights: the sum
    torch.testing.assert_close(some.double().cpu(), want_sum[rows], rtol=1e-5, atol=1e-5)
    # a read alone, unnormed, in bfloat16
    u = stream_step(xd, in_weights=w_in.to(DEV), out_dtype=torch.bfloat16)
    torch.testing.assert_close(u.double().cpu(), plain.read_copies(want_x, w_in.double()), rtol=1e-2, atol=1e-2)
    # the stream's first pass: all copies are the entering rows, which the pass reads once and stores as copies
    src = torch.randn(n, width, generator=g)
    full = src[:, None, :].repeat(1, copies, 1).to(DEV)
    args = dict(y=y.to(DEV), gate=gate.to(DEV), gate_bias=bias.to(DEV), layer_scale=scale.to(DEV), mix=mix.to(DEV), out_weights=w_out.to(DEV),
                in_weights=w_in.to(DEV), norm=(alpha.to(DEV), nw.to(DEV), nb.to(DEV)), out_dtype=torch.float32)
    h_full = stream_step(full, **args)
    late = torch.full((n, copies, width), float("nan"), device=DEV)
    h_late = stream_step(late, source=src.to(DEV), **args)
    assert torch.equal(h_full, h_late) and torch.equal(full, late)
    late.fill_(float("nan"))
    only_read = stream_step(late, source=src.to(DEV), in_weights=w_in.to(DEV), out_dtype=torch.float32)        # no write: still stored
    assert torch.equal(late.cpu(), src[:, None, :].repeat(1, copies, 1))
    torch.testing.assert_close(only_read.double().cpu(), src.double() * w_in.double().sum(), rtol=1e-5, atol=1e-5)
    late.fill_(float("nan"))
    stream_step(late, source=src.to(DEV), rows=i32(rows), out_dtype=torch.float32)                              # chosen rows: nothing stored
    assert bool(late.isnan().all())


def test_one_copy_without_mixing_is_the_plain_residual_sum():
    from yalis_b200.ops.streams import stream_step
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(9, 40, generator=g), torch.randn(9, 40, generator=g)
    xd = x.clone().to(DEV)
    h = stream_step(xd, y=y.to(DEV), out_dtype=torch.float32)
    assert torch.equal(xd.cpu(), x + y) and torch.equal(h.cpu(), x + y)


# ---- the table of token pairs ----------------------------------------------------------------------------------------

@pytest.mark.parametrize("buckets, mul_prev, mul_cur, vocab", [(7, 5, 11, 50), (509, 31, 3, 96), (64, 1, 1, 64), (1000003, 99991, 7919, 200000)])
def test_pair_rows_know_the_token_before_a_portion(buckets, mul_prev, mul_cur, vocab):
    """Two requests in portions; a slot that is used again starts with the table's last row, not with what the request
    before left there.  The largest case overflows 32 bits in the product unless it is taken in 64."""
    from yalis_b200.ops.streams import pair_rows_add, remember_last_tokens
    g = torch.Generator().manual_seed(buckets)
    width = 12
    seqs = {1: torch.randint(0, vocab, (17,), generator=g).tolist(), 3: torch.randint(0, vocab, (9,), generator=g).tolist()}
    table = torch.randn(buckets + 1, width, generator=g) if buckets <= 4096 else None

    def want_rows(tokens):
        return [buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets for i, t in enumerate(tokens)]

    if table is None:
        # only the row numbers are checked: a table of one column whose entry is its row number in two float32 halves
        idx = torch.arange(buckets + 1)
        table = torch.stack([(idx // 4096).float(), (idx % 4096).float()], dim=1)
        width = 2
    last = torch.full((5,), 12345 % vocab, dtype=torch.int32, device=DEV)                    # what earlier requests left
    got = {s: [] for s in seqs}
    plan = [[(1, 0, 5), (3, 0, 2)], [(3, 2, 1), (1, 5, 1)], [(1, 6, 11)], [(3, 3, 6)]]
    for step in plan:
        req, qs, slots, pos = step_arrays(step)
        ids = i32([t for s, a, c in step for t in seqs[s][a:a + c]])
        x = torch.zeros(int(ids.numel()), width, device=DEV)
        pair_rows_add(x, table.to(DEV), buckets, mul_prev, mul_cur, ids, pos, req, qs, slots, last, vocab)
        remember_last_tokens(ids, qs, slots, last)
        o = 0
        for s, a, c in step:
            got[s].append(x[o:o + c].cpu())
            o += c
    for s, tokens in seqs.items():
        rows = torch.cat(got[s])
        assert torch.equal(rows, table[want_rows(tokens)]), s
    assert last.cpu().tolist()[1] == seqs[1][-1] and last.cpu().tolist()[3] == seqs[3][-1]
    # slot 1 again, by another request: position 0 takes the last row whatever the slot remembers
    req, qs, slots, pos = step_arrays([(1, 0, 3)])
    x = torch.zeros(3, width, device=DEV)
    pair_rows_add(x, table.to(DEV), buckets, mul_prev, mul_cur, i32(seqs[3][:3]), pos, req, qs, slots, last, vocab)
    assert torch.equal(x.cpu(), table[want_rows(seqs[3][:3])])


# ---- the generalized delta rule ----------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype, heads, dim", [(torch.float32, 3, 10), (torch.bfloat16, 2, 64), (torch.float32, 1, 20), (torch.float32, 4, 128)])
def test_general_delta_inputs_decay_unit_key_and_removal(dtype, heads, dim):
    from yalis_b200.ops.recurrent import general_delta_prepare
    g = torch.Generator().manual_seed(dim)
    n, hd, rate = 13, heads * dim, 0.61
    wide = (torch.randn(n, 3 * hd + 5, generator=g) * 2).to(dtype)                  # r, k, v side by side in a wider matrix
    wide[4, hd:2 * hd] = 0                                                          # a key of zeros: the eps keeps it finite
    a_raw, w_raw = (torch.randn(n, hd, generator=g) * 3).to(dtype), (torch.randn(n, hd, generator=g) * 3).to(dtype)
    a_b, w_b = torch.randn(hd, generator=g), torch.randn(hd, generator=g)
    wd = wide.to(DEV)
    q, k, v, decay, unit, removal = general_delta_prepare(wd[:, :hd], wd[:, hd:2 * hd], wd[:, 2 * hd:3 * hd], a_raw.to(DEV), a_b.to(DEV),
                                                          w_raw.to(DEV), w_b.to(DEV), heads, dim, rate, 1e-6, i32([0] * n))
    x = wide.double()
    kk = x[:, hd:2 * hd].reshape(n, heads, dim)
    want_unit = (kk / torch.sqrt((kk * kk).sum(dim=-1, keepdim=True) + 1e-6)).reshape(n, hd)
    want_decay = torch.exp(-rate * plain.sigmoid(w_raw.double() + w_b.double()))
    want_removal = plain.sigmoid(a_raw.double() + a_b.double()) * want_unit
    for got, want in ((q, x[:, :hd]), (k, x[:, hd:2 * hd]), (v, x[:, 2 * hd:3 * hd]), (decay, want_decay), (unit, want_unit), (removal, want_removal)):
        assert got.dtype == torch.float32                                           # float32 from the projections' results on
        torch.testing.assert_close(got.double().cpu(), want, rtol=2e-6, atol=2e-6)
    assert float(decay.min()) >= math.exp(-rate) - 1e-6 and float(decay.max()) <= 1.0


def rule_inputs(T, heads, dim, g, slow=False):
    hd = heads * dim
    d = {"r": torch.randn(T, hd, generator=g) / dim ** 0.5, "k": torch.randn(T, hd, generator=g) * (1.5 / dim ** 0.5),
         "v": torch.randn(T, hd, generator=g)}
    d["w"] = (1 - 0.0004 * torch.rand(T, hd, generator=g)) if slow else torch.exp(-0.6065 * torch.rand(T, hd, generator=g))
    d["a"] = torch.rand(T, hd, generator=g) * (0.01 if slow else 1.0)
    return d


def plain_rule(d, heads, dim, state=None):
    T = d["r"].shape[0]
    sh = lambda t: t.double().reshape(T, heads, dim)
    out, last = plain.general_delta_rule(sh(d["r"]), sh(d["k"]), sh(d["v"]), sh(d["w"]), sh(d["a"]), state)
    return out.reshape(T, heads * dim), last


def scan(d, rows, lay, qs, slots, heads, dim):
    from yalis_b200.ops.recurrent import state_scan
    k = d["k"].double().reshape(-1, heads, dim)
    unit = (k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)).reshape(-1, heads * dim)
    removal = d["a"].double() * unit
    f = lambda t: t.float().contiguous().to(DEV)
    return state_scan(f(d["r"]), f(d["k"]), f(d["v"]), rows, lay, qs, slots, kv_heads=heads, decay=f(d["w"]), unit=f(unit),
                      removal=f(removal))


@pytest.mark.parametrize("heads, dim", [(2, 16), (3, 10), (1, 20), (4, 48), (2, 64), (1, 128), (2, 6)])
def test_the_generalized_rule_against_the_plain_recurrence_however_the_tokens_are_cut(heads, dim):
    from yalis_b200.ops.recurrent import StateLayout
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    lay = StateLayout(heads, dim, dim)
    lengths = [37, 5, 64]
    data = [rule_inputs(T, heads, dim, g) for T in lengths]
    want = [plain_rule(d, heads, dim)[0] for d in data]

    def run(plan, rows):
        got = [torch.zeros(T, heads * dim, dtype=torch.float64) for T in lengths]
        for step in plan:
            _, qs, slots, _ = step_arrays([(r + 1, a, c) for r, a, c in step])
            cat = {key: torch.cat([data[r][key][a:a + c] for r, a, c in step]) for key in data[0]}
            out = scan(cat, rows, lay, qs, slots, heads, dim)
            o = 0
            for r, a, c in step:
                got[r][a:a + c] = out[o:o + c].double().cpu()
                o += c
        return got

    def fresh():
        rows = torch.zeros(5, lay.total, device=DEV)
        rows[0].fill_(3.0)
        rows[4].fill_(-2.0)
        return rows

    whole = run([[(r, 0, T)] for r, T in enumerate(lengths)], fresh())
    for r in range(3):
        assert float((whole[r] - want[r]).abs().max() / want[r].abs().max()) < 3e-5, r
    together = run([[(r, 0, T) for r, T in enumerate(lengths)]], fresh())
    pieces = {r: cuts(T, s) for (r, T), s in zip(enumerate(lengths), ([2, 1, 17, 3], [1, 2], [16, 1, 2, 30]))}
    plan = []
    for i in range(max(len(p) for p in pieces.values())):
        step = [(r, *pieces[r][i]) for r in pieces if i < len(pieces[r])]
        plan.append(step[::-1] if i % 2 else step)
    rows = fresh()
    cut = run(plan, rows)
    for r in range(3):
        assert torch.equal(together[r], whole[r]) and torch.equal(cut[r], whole[r]), r          # the same bits
    assert float(rows[0, 0]) == 3.0 and float(rows[4, 5]) == -2.0                                # nobody else's slot
    # the state the slot keeps is the plain one
    last = plain_rule(data[0], heads, dim)[1]                                                     # [H, d(key), d(value)]
    kept = rows[1, :lay.state_floats].reshape(heads, dim, lay.dim_padded)[:, :, :dim].double().cpu()   # per head [value, key]
    torch.testing.assert_close(kept.transpose(1, 2), last, rtol=1e-4, atol=1e-5)


def test_removal_and_decay_both_read_the_old_state():
    """One head, two channels, numbers small enough to follow by hand: with S = [[1, 2], [3, 4]] (key by value),
    w = (0.5, 1), a = (1, 0), k = (2, 0) (so u = (1, 0) up to the eps) and v = (10, 20):
    diag(w) S = [[0.5, 1], [3, 4]]; (a * u)(u^T S) = [[1, 2], [0, 0]] from the OLD S; k v^T = [[20, 40], [0, 0]];
    the new S = [[19.5, 39], [3, 4]].  A rule that decays first and removes from the decayed state gives 19.75."""
    from yalis_b200.ops.recurrent import StateLayout
    lay = StateLayout(1, 2, 2)
    rows = torch.zeros(2, lay.total, device=DEV)
    S = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    rows[1, :lay.state_floats].reshape(1, 2, lay.dim_padded)[0, :, :2] = S.T.to(DEV)
    d = {"r": torch.tensor([[1.0, 1.0]]), "k": torch.tensor([[2.0, 0.0]]), "v": torch.tensor([[10.0, 20.0]]),
         "w": torch.tensor([[0.5, 1.0]]), "a": torch.tensor([[1.0, 0.0]])}
    _, qs, slots, _ = step_arrays([(1, 5, 1)])
    out = scan(d, rows, lay, qs, slots, 1, 2)
    want_S = torch.tensor([[19.5, 39.0], [3.0, 4.0]])
    want, _ = plain_rule(d, 1, 2, state=S.double()[None])
    torch.testing.assert_close(want, (want_S.T @ torch.ones(2)).double()[None], rtol=1e-6, atol=1e-6)     # the plain rule agrees with the hand
    torch.testing.assert_close(out.cpu(), torch.tensor([[22.5, 43.0]]), rtol=1e-5, atol=1e-5)


def test_a_far_token_stays_readable_in_a_slowly_decaying_state():
    """A pair (key, value) written at the first token is read 500 tokens later, the later tokens decoded one by one:
    a state that is lost, reset or written to another slot on the way loses it."""
    from yalis_b200.ops.recurrent import StateLayout
    g = torch.Generator().manual_seed(8)
    heads, dim, T = 2, 32, 501
    lay = StateLayout(heads, dim, dim)
    d = rule_inputs(T, heads, dim, g, slow=True)
    d["k"] = d["k"] * 0.02                                                 # the other keys write little
    e = torch.zeros(heads * dim)
    e[3], e[dim + 7] = 1.0, 1.0
    d["k"][0], d["v"][0] = 2.0 * e, torch.arange(heads * dim).float() / 10
    d["r"][T - 1] = e
    want = plain_rule(d, heads, dim)[0]
    rows = torch.zeros(3, lay.total, device=DEV)
    got = []
    for a, c in cuts(T, [200] + [1] * 400):
        _, qs, slots, _ = step_arrays([(2, a, c)])
        got.append(scan({k: v[a:a + c] for k, v in d.items()}, rows, lay, qs, slots, heads, dim).double().cpu())
    got = torch.cat(got)
    assert float((got - want).abs().max() / want.abs().max()) < 1e-4
    planted = 2.0 * d["v"][0].double()
    assert float((got[-1] - planted).abs().max()) < 0.35 * float(planted.abs().max())           # still there, a little decayed


# ---- attention over the latent's rows with a sink ------------------------------------------------------------------

def rows_in_pages(rows, page, seed, dtype):
    """One request's rows [T, w] laid into shuffled pages of a pool whose other places hold NaN."""
    T, w = rows.shape
    pages = -(-T // page)
    perm = torch.randperm(pages + 3, generator=torch.Generator().manual_seed(seed))[:pages]
    pool = torch.full((pages + 3, 1, page, w), float("nan"), dtype=dtype, device=DEV)
    for t in range(T):
        pool[int(perm[t // page]), 0, t % page] = rows[t].to(dtype).to(DEV)
    return pool, perm.to(torch.int32).reshape(1, -1).to(DEV)


def plain_sink_attention(qc, rows, r, scale, sink, at=None):
    """qc [T, H, w] (one query per position), rows [T, w]: every head's keys are the rows, its values their first r
    sizes.  ``at``: the positions to compute (all); the result has one row for each."""
    T, H, w = qc.shape
    at = range(T) if at is None else at
    out = torch.zeros((len(at), H, r), dtype=qc.dtype)
    for n, i in enumerate(at):
        for h in range(H):
            s = (rows[:i + 1] @ qc[i, h]) * scale
            top = max(float(s.max()), float(sink[h]))
            e = torch.exp(s - top)
            out[n, h] = (e @ rows[:i + 1, :r]) / (e.sum() + math.exp(float(sink[h]) - top))
    return out


def test_the_rows_form_of_the_sink_softmax_is_the_plain_attention():
    """The helper above against the plain model's attention with per-head keys and values."""
    g = torch.Generator().manual_seed(2)
    T, H, w, r = 9, 2, 7, 5
    qc, rows, sink = torch.randn(T, H, w, generator=g).double(), torch.randn(T, w, generator=g).double(), torch.tensor([0.5, -1.0]).double()
    keys = rows[:, None, :].expand(T, H, w)
    want = plain.causal_attention_with_sink(qc, keys, keys[:, :, :r], 0.4, sink)
    torch.testing.assert_close(plain_sink_attention(qc, rows, r, 0.4, sink), want)


@pytest.mark.parametrize("dtype, r, p, page", [(torch.float32, 24, 8, 16), (torch.float32, 14, 4, 8), (torch.bfloat16, 96, 48, 16),
                                               (torch.float32, 20, 2, 64), (torch.bfloat16, 64, 32, 32)])
def test_the_sink_joins_the_denominator_once_unscaled_and_a_far_row_is_found(dtype, r, p, page):
    """Head 0: a sink that hardly counts; head 1: a sink of the order of the scores; head 2: a sink that takes nearly all
    the weight; head 3 asks for a row planted at the last place of the first page, 300 rows back.  A scale far from one
    shows a sink that was scaled with the scores."""
    from yalis_b200.ops.latent import latent_attention_exact
    g = torch.Generator().manual_seed(r * 10 + p)
    T, heads, scale = 330, 4, 0.37
    star = page - 1
    u = torch.nn.functional.normalize(torch.randn(r + p, generator=g), dim=0)
    rows = torch.randn(T, r + p, generator=g) * 0.5
    rows[star] = 6.0 * u
    rows = rows.to(dtype).double()
    qc = torch.randn(T, heads, r + p, generator=g)
    qc[:, 3] = (4.0 / scale) * u
    sink = torch.tensor([-30.0, 1.0, 9.0, 2.0])
    ask = [0, 1, star - 1, star, star + 1, page, 2 * page - 1, 200, T - 2, T - 1]
    want = torch.zeros(T, heads, r, dtype=torch.float64)
    want[ask] = plain_sink_attention(qc.double(), rows, r, scale, sink.double(), ask)
    pool, table = rows_in_pages(rows, page, 3, dtype)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for name, groups in (("a portion", [ask]), ("one by one", [[a] for a in ask])):
        for grp in groups:
            out = latent_attention_exact(qc[grp].contiguous().to(DEV), pool, i32(grp), i32([0] * len(grp)), table, r, scale, None,
                                         sink=sink.to(DEV)).double().cpu()
            torch.testing.assert_close(out, want[grp], rtol=tol, atol=tol, msg=lambda m: f"{name} {grp}: {m}")
    no_sink = torch.zeros_like(want)
    no_sink[ask] = plain_sink_attention(qc.double(), rows, r, scale, torch.full((heads,), -1e9, dtype=torch.float64), ask)
    assert float((want[:, 0] - no_sink[:, 0]).abs().max()) < 1e-9                       # exp(-30) is nothing
    assert float(want[200, 2].norm() / no_sink[200, 2].norm()) < 0.2                    # exp(9) among 200 scores of order one
    hit = float(torch.dot(want[T - 1, 3], rows[star, :r]) / rows[star, :r].norm() ** 2)
    assert 0.85 < hit < 1.0 + 1e-6                                                         # exp(24) against exp(2)


@pytest.mark.parametrize("r, p, page, heads", [(64, 16, 8, 3), (96, 48, 16, 5), (128, 0, 64, 2), (256, 64, 16, 16), (512, 64, 32, 5)])
@pytest.mark.parametrize("splits", [1, 4])
def test_the_sink_on_the_tensor_cores(r, p, page, heads, splits):
    """Two requests in one step, a portion behind cached rows beside a single token; with ``splits`` > 1 (a step of
    single tokens) the rows are dealt to several blocks, and the sink must still count once."""
    from yalis_b200.ops.latent import latent_attention_mma
    g = torch.Generator().manual_seed(r + p + heads)
    scale = 0.21
    lens, new = ([295, 130], [45, 1]) if splits == 1 else ([295, 130], [1, 1])
    sink = torch.linspace(-3.0, 6.0, heads)
    width = max(-(-l // page) for l in lens)
    table = torch.full((2, width), -1, dtype=torch.int32)
    pool = torch.full((sum(-(-l // page) for l in lens) + 2, 1, page, r + p), float("nan"), dtype=torch.bfloat16, device=DEV)
    perm = iter(torch.randperm(pool.shape[0], generator=g).tolist())
    want, q_all, pos, req = [], [], [], []
    for i, (l, c) in enumerate(zip(lens, new)):
        rows = (torch.randn(l, r + p, generator=g) * 0.5).to(torch.bfloat16)
        for j in range(-(-l // page)):
            table[i, j] = next(perm)
        for t in range(l):
            pool[int(table[i, t // page]), 0, t % page] = rows[t].to(DEV)
        qc = torch.zeros(l, heads, r + p)
        qc[l - c:] = (torch.randn(c, heads, r + p, generator=g) * 1.5).to(torch.bfloat16).float()
        want.append(plain_sink_attention(qc.double(), rows.double(), r, scale, sink.double(), list(range(l - c, l))))
        q_all.append(qc[l - c:])
        pos += list(range(l - c, l))
        req += [i] * c
    q = torch.cat(q_all).to(DEV)
    out = torch.zeros(len(pos), heads, r, device=DEV)
    latent_attention_mma(q[:, :, :r].contiguous(), q[:, :, r:].contiguous() if p else torch.zeros(len(pos), heads, 0, device=DEV),
                         out, pool, i32(pos), i32([0, new[0], new[0] + new[1]]), i32(req), table.to(DEV), 2, max(new), scale, None,
                         n_splits=splits, sink=sink.to(DEV))
    torch.testing.assert_close(out.double().cpu(), torch.cat(want), rtol=2e-2, atol=2e-2)
    # a sink of weight: leaving it out would double the last head's result
    assert float(torch.cat(want)[:, -1].abs().max()) > 0


# ---- the feed-forward: gated silu experts weighted by their scores -------------------------------------------------

def expert_tensors(hidden, experts, inner, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    t = {"router": (torch.randn(experts, hidden, generator=g) * (3.0 / hidden ** 0.5)).to(dtype)}
    for e in range(experts):
        for name, shape in (("gate", (inner, hidden)), ("up", (inner, hidden)), ("down", (hidden, inner))):
            t[f"e{e}.{name}"] = (torch.randn(shape, generator=g) / shape[1] ** 0.5).to(dtype)
    return t


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n, hidden, experts, top, inner, scale", [(5, 64, 4, 2, 24, 1.5), (70, 36, 5, 5, 18, 0.7), (900, 128, 8, 1, 64, 2.0),
                                                                 (300, 128, 16, 4, 40, 1.0), (1, 40, 2, 2, 7, 3.0)])
def test_gated_experts_weighted_by_unrenormalised_scores(dtype, n, hidden, experts, top, inner, scale):
    """The scores of the chosen experts are not brought to sum one: with one expert chosen of eight the weight is well
    below one, with all chosen the weights sum to ``scale``."""
    from yalis_b200.config.spec import PartSpec
    from yalis_b200.parts.base import make_part
    t = expert_tensors(hidden, experts, inner, n, dtype)
    part = make_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": hidden, "experts": experts, "top": top, "expert_size": inner, "activation": "silu", "gated": True,
        "shared_size": None, "renorm": False, "route_scale": scale}))
    local = {"router": t["router"].float().to(DEV)}
    for e in range(experts):
        for name in ("gate", "up", "down"):
            local[f"expert_{e}_{name}"] = t[f"e{e}.{name}"].to(DEV)
    part.load(local)
    x = torch.randn(n, hidden, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    got = part.forward(x.to(dtype).to(DEV), None).double().cpu()
    mlp = {"router": {"experts": experts, "top": top, "scale": scale}}
    want = plain.mixture_of_experts(x.double(), {"p." + k: v.double() for k, v in t.items()}, "p.", mlp)
    if dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    else:
        err = (got - want).abs().max(dim=1).values / want.abs().max()
        assert float(err.median()) < 2e-2 and float((err > 4e-2).float().mean()) <= 0.03, float(err.max())
    _, weights = plain.routing(x.double(), t["router"].double(), top, scale)
    if top == experts:
        torch.testing.assert_close(weights.sum(dim=1), torch.full((n,), scale, dtype=torch.float64))
    if top == 1 and n > 100:
        assert float(weights.mean()) < 0.9 * scale


# ---- whole models -----------------------------------------------------------------------------------------------------

TOL = {"float32": 1e-4, "bfloat16": 5e-2}       # relative to the largest |logit| of the request
LENGTHS = {"A": [1, 5, 33, 70, 21, 48], "B": [2, 40, 9, 64, 17, 90], "C": [3, 37, 18, 130, 12, 66], "D": [7, 1, 50, 19, 33, 4]}
PAGE = {"A": 16, "B": 8, "C": 64, "D": 16}
_oracle = {}


def requests_for(which):
    cfg, _ = plain.read_folder(pametar_dir(which))
    g = torch.Generator().manual_seed(ord(which) + 100)
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[which])}


def oracle(which):
    if which not in _oracle:
        cfg, w = plain.read_folder(pametar_dir(which))
        _oracle[which] = {rid: plain.forward(cfg, w, t).numpy() for rid, t in requests_for(which).items()}
    return _oracle[which]


def replay(which, dtype, steps, max_tokens, graphs=False):
    from yalis_b200.engine.replay import Replayer
    rep = Replayer(pametar_dir(which), dtype, max_tokens, page_size=PAGE[which], graphs=graphs)
    out = {}
    for s in steps:
        r = rep.run_step(s)
        if r is not None:
            out[s["step"]] = r
    rep.engine.manager.check()
    for grp in rep.engine.groups:
        assert rep.engine.manager.free_pages(grp.name) == grp.num_pages          # every page came back
    return out, rep


def compare(got, want, tol, what, outliers=0.0):
    assert set(got) == set(want), what
    total = bad = 0
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        scale = np.abs(want[rid]).max()
        err = np.abs(got[rid] - want[rid]).max(axis=1) / scale
        total += len(err)
        bad += int((err > tol).sum())
        if err.max() > tol and not outliers:
            raise AssertionError(f"{what}: request {rid} differs by {err.max():.3e} (tolerance {tol}); first wrong "
                                 f"position {int(np.argmax(err > tol))} of {len(err)}")
    assert bad <= outliers * total, f"{what}: {bad} of {total} positions differ by more than {tol}"


@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_cut_four_ways_agree_with_the_plain_model(which, dtype):
    reqs, want = requests_for(which), oracle(which)
    vocab = plain.read_folder(pametar_dir(which))[0]["vocab"]
    results = {}
    # bfloat16: a token whose best router scores are nearly equal may run another expert than the float64 model
    outliers = 0.0 if dtype == "float32" else 0.06
    for name, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail_decoded(reqs, tail=12)),
                        ("portions", traces.portions(reqs, seed=3)), ("mixed", traces.mixed(reqs, seed=5, tail=6))):
        steps = traces.number(steps)
        out, rep = replay(which, dtype, steps, traces.peak_tokens(steps, max(64, PAGE[which])))
        got = traces.collect(steps, out, vocab)
        compare(got, want, TOL[dtype], f"{which} {dtype} {name}", outliers=outliers)
        results[name] = got
    # how a request was cut, what ran beside it and which pages and slots it had leave (nearly) no trace
    for name in ("tail", "portions", "mixed"):
        for rid in want:
            scale = np.abs(want[rid]).max()
            diff = np.abs(results[name][rid] - results["whole"][rid]).max(axis=1) / scale
            if dtype == "float32":
                assert diff.max() < 2e-5, (name, rid)
            else:
                assert np.mean(diff > 5e-2) <= outliers, (name, rid)


@pytest.mark.parametrize("which", ["A", "C"])
def test_steps_replayed_from_recordings_give_the_same(which):
    """Decoded tokens through recorded steps (CUDA graphs): routing and the previous token are read on the device."""
    reqs, want = requests_for(which), oracle(which)
    vocab = plain.read_folder(pametar_dir(which))[0]["vocab"]
    steps = traces.number(traces.tail_decoded(reqs, tail=12))
    launched, _ = replay(which, "float32", steps, traces.peak_tokens(steps, max(64, PAGE[which])))
    recorded, rep = replay(which, "float32", steps, traces.peak_tokens(steps, max(64, PAGE[which])), graphs=True)
    assert rep.steps_replayed > 40
    a, b = traces.collect(steps, launched, vocab), traces.collect(steps, recorded, vocab)
    compare(b, want, TOL["float32"], f"{which} recorded")
    for rid in a:
        assert np.abs(a[rid] - b[rid]).max() / np.abs(a[rid]).max() < 1e-6


@pytest.mark.parametrize("which, runs", [("A", 6), ("D", 6), ("B", 5)])
def test_the_sum_of_the_copies_after_every_layer_run(which, runs):
    """A looped layer counts every time it runs."""
    from yalis_b200.engine.engine import Engine, StepEntry
    d = pametar_dir(which)
    cfg, w = plain.read_folder(d)
    tokens = requests_for(which)["r2"]
    want = []
    plain.forward(cfg, w, tokens, taps=want)
    eng = Engine(d, dtype="float32", page_size=16, num_pages=8, max_slots=2, max_context=128)
    eng.add_request("x")
    seen = []
    inner = eng.model.forward
    eng.model.forward = lambda ctx, caches: inner(ctx, caches, tap=lambda i, x: seen.append(x.double().cpu()))
    eng.run([StepEntry("x", tokens, [len(tokens) - 1])])
    assert len(seen) == len(want) == runs
    for i, (a, b) in enumerate(zip(seen, want)):
        assert float((a - b).abs().max() / b.abs().max()) < 2e-5, f"layer run {i}"


@pytest.mark.parametrize("which, dtype", [("A", "float32"), ("B", "float32"), ("D", "bfloat16")])
def test_long_decoding_keeps_to_the_plain_model(which, dtype):
    """300 tokens one by one after a two-token prompt, through pages of eight: the state is carried 300 times, every
    pass of a looped layer in its own slot row and pages."""
    from yalis_b200.engine.engine import Engine, StepEntry
    d = pametar_dir(which)
    cfg, w = plain.read_folder(d)
    g = torch.Generator().manual_seed(9)
    tokens = torch.randint(0, cfg["vocab"], (302,), generator=g).tolist()
    want = plain.forward(cfg, w, tokens).numpy()
    eng = Engine(d, dtype=dtype, page_size=8, num_pages=40, max_slots=2, max_context=384)
    eng.add_request("x")
    rows = [eng.run([StepEntry("x", tokens[:2], [0, 1])]).logits.cpu().numpy()]
    for t in tokens[2:]:
        rows.append(eng.run([StepEntry("x", [t], [0])]).logits.cpu().numpy())
    got = np.concatenate(rows)
    eng.check_device_errors()
    err = np.abs(got - want).max(axis=1) / np.abs(want).max()
    if dtype == "float32":
        assert err.max() < 1e-4
    else:
        assert np.mean(err > 5e-2) < 0.06


@pytest.mark.parametrize("which", ["C", "D"])
def test_a_slot_and_its_pages_used_again_start_clean(which):
    """The state of the rule, the previous token and the pages of a finished request must not show in the next one."""
    from yalis_b200.engine.engine import Engine, StepEntry
    d = pametar_dir(which)
    reqs = requests_for(which)
    eng = Engine(d, dtype="float32", page_size=64, num_pages=3, max_slots=1, max_context=192)
    first = None
    for rid in ("r3", "r2", "r3"):
        assert eng.add_request(rid) == 0                       # the only slot, every time
        cut = len(reqs[rid]) // 2                              # in two portions: the second starts from slot and pages
        eng.run([StepEntry(rid, reqs[rid][:cut], [])])
        out = eng.run([StepEntry(rid, reqs[rid][cut:], [len(reqs[rid]) - cut - 1])]).logits.cpu().numpy()
        eng.finish_request(rid)
        if rid == "r3":
            if first is None:
                first = out
            else:
                assert np.array_equal(first, out)


@pytest.mark.parametrize("which", ["A", "B", "D"])
def test_greedy_generation_through_the_entry_point(which):
    from yalis_b200 import InferenceConfig, LLMEngine, ModelConfig
    d = pametar_dir(which)
    cfg, w = plain.read_folder(d)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (3, 19, 40, 7, 26)]
    engine = LLMEngine(ModelConfig(model_name=f"pametar-tiny-{which}", model_path=d, precision="fp32"),
                       InferenceConfig(max_batch_size=3, max_length_of_generated_sequences=64, temperature=0.0, top_p=0.0,
                                       page_size=PAGE[which]))
    tokens, metrics = engine.generate(prompts, tokens_to_generate=10)[:2]
    for p, row in zip(prompts, tokens.cpu().tolist()):
        assert row == plain.greedy(cfg, w, p, 10)


def test_the_replay_program_runs_a_pametar_folder(tmp_path):
    reqs = {k: v for k, v in requests_for("B").items() if k in ("r1", "r2")}
    steps = traces.number(traces.portions(reqs, seed=1))
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", pametar_dir("B"), "--dtype", "float32",
                           "--out", str(out_dir), "--max-tokens", str(traces.peak_tokens(steps))],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    vocab = plain.read_folder(pametar_dir("B"))[0]["vocab"]
    outputs = {s["step"]: np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4") for s in steps}
    compare(traces.collect(steps, outputs, vocab), {k: oracle("B")[k] for k in reqs}, TOL["float32"], "program")


# ---- random configurations ---------------------------------------------------------------------------------------------

def random_pametar(rng):
    from yalis_b200.config.presets import _pametar, _pm_delta, _pm_latent, _pm_moe
    width = rng.choice([64, 96, 136, 192, 320])

    def mlp():
        if rng.random() < 0.15:
            return None
        experts = rng.choice([2, 3, 4, 8, 16])
        return _pm_moe(experts, rng.randint(1, min(experts, 6)), rng.choice([24, 40, 64, 128]), rng.choice([0.5, 1.0, 1.5, 2.5]))

    def layer():
        if rng.random() < 0.5:
            return _pm_delta(rng.choice([1, 2, 3, 4, 6]), rng.choice([8, 16, 24, 32, 48, 64, 96, 128]), rng.choice([4, 16, 32]), mlp())
        p = rng.choice([4, 8, 16, 32, 64])
        d = rng.choice([8, 16, 32, 48, 64, 80])
        return _pm_latent(rng.choice([1, 2, 3, 4, 6, 8]), d, p, rng.choice([8, 16, 32, 48, 64]), rng.choice([16, 40, 64, 96, 128, 160]),
                          rng.choice([24, 64, 96, 128]), rng.choice([(d + p) ** -0.5, 0.2]), rng.choice([100.0, 10000.0, 500000.0]), mlp())

    n = rng.randint(2, 5)
    layers = [layer() for _ in range(n)]
    loop = None
    if rng.random() < 0.7:
        a = rng.randint(0, n - 1)
        loop = (a, rng.randint(a + 1, n), rng.randint(1, 3))
    bigram = None if rng.random() < 0.2 else (rng.choice([5, 251, 1019, 4099]), rng.randint(0, 200), rng.randint(1, 50))
    return _pametar(width, rng.choice([80, 300, 700]), rng.randint(1, 4), layers, loop=loop, embedding_scale=rng.choice([1.0, 4.0, 12.0]),
                    bigram=bigram, eps=rng.choice([1e-5, 1e-6]))


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_replay_of_random_configurations(seed, tmp_path):
    import random
    from pametar_models import write_model
    from yalis_b200.engine.replay import Replayer
    rng = random.Random(seed)
    for trial in range(3):
        config = random_pametar(rng)
        d = write_model(config, str(tmp_path / f"m{trial}"), seed * 10 + trial)
        cfg, w = plain.read_folder(d)
        page = rng.choice([8, 16, 32, 64])
        g = torch.Generator().manual_seed(seed)
        reqs = {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
                for i, n in enumerate([rng.randint(1, 30), rng.randint(31, 110), rng.randint(40, 140), rng.randint(2, 9), rng.randint(10, 70)])}
        want = {rid: plain.forward(cfg, w, t).numpy() for rid, t in reqs.items()}
        for dtype in ("float32", "bfloat16"):
            for name, steps in (("portions", traces.portions(reqs, seed=seed)), ("mixed", traces.mixed(reqs, seed=seed + trial, tail=5))):
                steps = traces.number(steps)
                rep = Replayer(d, dtype, traces.peak_tokens(steps, max(64, page)), page_size=page)
                out = {}
                for s in steps:
                    r = rep.run_step(s)
                    if r is not None:
                        out[s["step"]] = r
                rep.engine.manager.check()
                got = traces.collect(steps, out, cfg["vocab"])
                what = f"seed {seed} trial {trial} {dtype} {name}: {config}"
                if dtype == "float32":
                    compare(got, want, TOL[dtype], what)
                    continue
                # bfloat16: a close call decides much in this design (a router's two scores; the sign of r.k at a sequence's
                # first token, which the read-out's norm turns into a whole head's sign) and the state carries it on, so one
                # request of the five may leave the plain model; the others keep to it
                off = [rid for rid in want
                       if np.mean(np.abs(got[rid] - want[rid]).max(axis=1) / np.abs(want[rid]).max() > TOL[dtype]) > 0.08]
                assert len(off) <= 1, f"{what}: requests {off} differ"
