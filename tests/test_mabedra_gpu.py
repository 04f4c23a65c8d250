"""Mabedra through the framework against the plain implementation: every mechanism's kernels alone (with inputs made so
that a key at a window's edge, a far key or a page border shows), then whole models under every way of cutting the work
(whole prompts, decoding token by token, portions down to two tokens, mixed batches whose pages and slots are used
again), in 32-bit and in bfloat16, and greedy generation through the engine's own entry point."""

import math
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from tests import helpers
from tests.plain import mabedra_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# a row of logits against the plain model in 64-bit, as fractions of the row's root mean square: (rms, largest).
# float32 is the sharp comparison.  bfloat16: the plain model rounds its activations where the engine stores them; a
# rounding that falls the other way moves single rows by several per cent, so a request passes when at most a tenth of its
# rows (or one) is beyond BF16_USUAL and none beyond BF16_WORST.  A row at which some router's last chosen logit lies within
# CLOSE_CALL of the first one left out is not compared: there the two models may rightly send the token to different experts.
TOL = {"float32": (3e-5, 2e-4)}
BF16_USUAL, BF16_WORST, CLOSE_CALL = 6e-2, 5e-1, 0.15


def dev(t):
    return t.to(DEV)


def _pages(seed, page, lengths, spare=3):
    """Block tables that scatter each sequence over pages in a shuffled order; returns (table, pages in use)."""

    rng = random.Random(seed)
    need = [-(-n // page) for n in lengths]
    ids = list(range(sum(need) + spare))
    rng.shuffle(ids)
    table = torch.full((len(lengths), max(need)), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(need):
        table[r, :n] = torch.tensor(ids[at:at + n], dtype=torch.int32)
        at += n
    return table, len(ids)


def _ctx(lengths, q_lens):
    """What the kernels read of a step's context: every sequence of ``lengths`` brings its last ``q_lens`` tokens."""

    positions = torch.cat([torch.arange(m - k, m) for m, k in zip(lengths, q_lens)]).int()
    entry = torch.cat([torch.full((k,), i) for i, k in enumerate(q_lens)]).int()
    return SimpleNamespace(positions=dev(positions), token_entry=dev(entry), all_decode=max(q_lens) == 1, num_entries=len(lengths),
                           q_lens=list(q_lens), kv_lens=list(lengths), max_kv_len=max(lengths))


def _fill(pool, table, page, rows):
    """Write each sequence's rows ``[T, heads, columns]`` into ``pool`` ``[pages, heads, page, columns]`` through its table."""

    for e, seq in enumerate(rows):
        for t in range(seq.shape[0]):
            pool[table[e, t // page], :, t % page] = seq[t]


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [90, 96, 1028])
def test_layer_norm_with_the_pending_sum_and_a_gather(out_dtype, width):
    from llm_runtime_study_b200.ops import block_steps as B

    torch.manual_seed(1)
    n, eps = 37, 1e-5
    x, delta, w = 3.0 + 2.0 * torch.randn(n, width), torch.randn(n, width), 1.0 + 0.3 * torch.randn(width)
    resid = dev(x.clone())
    got = B.layer_norm(resid, dev(delta), dev(w), eps, out_dtype).cpu().double()
    want = plain.layer_norm((x + delta).double(), w.double(), eps)
    assert torch.equal(resid.cpu(), x + delta)                          # the sum is left in the stream, in float32
    tol = 2e-5 if out_dtype == torch.float32 else 2e-2
    assert (got - want).abs().max() <= tol * float(want.abs().max())
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32)
    before = resid.clone()
    got = B.layer_norm(resid, None, dev(w), eps, out_dtype, rows=dev(rows)).cpu().double()
    assert torch.equal(resid, before) and (got - want[rows.long()]).abs().max() <= tol * float(want.abs().max())
    # a row of equal entries has no variance: eps alone is under the root
    flat = torch.full((1, width), 7.0)
    assert B.layer_norm(dev(flat), None, dev(w), eps, torch.float32).abs().max() <= 1e-3


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,cuts,width", [(4, [1, 2, 1, 9, 3, 30], 24), (2, [5, 1, 1], 24), (3, [46], 24), (5, [1, 1, 1, 1, 1, 1, 2], 24),
                                             (4, [2, 1, 700, 1, 3], 8), (3, [1, 515, 2], 12), (4, [3, 1, 20], 23), (1, [4, 1], 8)])
def test_input_convolutions_across_cuts(out_dtype, taps, cuts, width):
    """Two requests in one batch, fed in portions shorter than the convolution's reach, their kept inputs in slots that do
    not follow the batch's order; both sublayers' inputs against the convolution over the whole sequences.  Long portions
    take the kernel that walks runs of rows, a width that is no multiple of four and more than four taps the plain one."""

    from llm_runtime_study_b200.ops import block_steps as B
    from llm_runtime_study_b200.ops import sequence_state as S

    torch.manual_seed(taps)
    total = sum(cuts)
    seqs = [torch.randn(total, width), torch.randn(total, width)]
    wa, wb = torch.randn(width, taps), torch.randn(width, taps)
    kept = torch.zeros(6, taps - 1, width, dtype=torch.float32, device=DEV) if taps > 1 else None
    slots = dev(torch.tensor([4, 1], dtype=torch.int32))
    got_a, got_b = [[], []], [[], []]
    at = 0
    for n in cuts:
        h = torch.cat([s[at:at + n] for s in seqs])
        q_start = dev(torch.tensor([0, n, 2 * n], dtype=torch.int32))
        entry = dev(torch.tensor([0] * n + [1] * n, dtype=torch.int32))
        a, b = B.taps_pair(dev(h), dev(wa), dev(wb), kept, q_start=q_start, slots=slots, token_entry=entry, out_dtype=out_dtype)
        if taps > 1:
            S.conv_state_update(dev(h), kept, q_start, slots)
        for e in range(2):
            got_a[e].append(a[e * n:(e + 1) * n].cpu().double())
            got_b[e].append(b[e * n:(e + 1) * n].cpu().double())
        at += n
    tol = 1e-5 if out_dtype == torch.float32 else 3e-2
    for e, s in enumerate(seqs):
        s = s.double()
        assert (torch.cat(got_a[e]) - (s + plain.causal_taps(s, wa.double()))).abs().max() <= tol * 4
        assert (torch.cat(got_b[e]) - (s + plain.causal_taps(s, wb.double()))).abs().max() <= tol * 4
    if taps == 1:
        return
    assert torch.equal(kept[4].cpu(), seqs[0][total - taps + 1:]) and torch.equal(kept[1].cpu(), seqs[1][total - taps + 1:])
    assert float(kept[0].abs().max()) == 0.0 and float(kept[5].abs().max()) == 0.0        # other slots are left alone


@pytest.mark.parametrize("width", [40, 41])
def test_scaled_sum_and_the_average_over_all_results(width):
    from llm_runtime_study_b200.ops import block_steps as B

    torch.manual_seed(3)
    n, depth = 19, 4
    x0 = torch.randn(n, width)
    results = torch.zeros(depth + 1, n, width, device=DEV)
    results[0] = dev(x0)
    x = dev(x0.clone())
    history = [x0.double()]
    stream = x0.double()
    for i in range(depth):
        a, b, sa, sb, mix = torch.randn(n, width), torch.randn(n, width), torch.randn(width), torch.randn(width), torch.randn(i + 2)
        with_ff = i != 2
        B.scale_sum_average(x, dev(a), dev(sa), dev(b) if with_ff else None, dev(sb) if with_ff else None, results, dev(mix), i)
        new = stream + sa.double() * a.double() + (sb.double() * b.double() if with_ff else 0.0)
        history.append(new)
        stream = sum(mix.double()[j] * history[j] for j in range(i + 2))
        assert (results[i + 1].cpu().double() - new).abs().max() <= 1e-5
        assert (x.cpu().double() - stream).abs().max() <= 2e-5
    # without an average and without scales the stream is the plain residual sum
    y = dev(x0.clone())
    B.scale_sum_average(y, dev(a), None, dev(b), None, None, None, 0)
    assert (y.cpu() - (x0 + a + b)).abs().max() <= 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,ff", [(33, 40), (2, 257), (5, 1024), (2, 4104), (2, 25600)])
def test_polynomial_activation_of_normalised_powers(dtype, n, ff):
    from llm_runtime_study_b200.ops import block_steps as B

    torch.manual_seed(ff)
    z = (1.5 * torch.randn(n, ff)).to(dtype)
    coef = torch.tensor([0.7, -1.3, 0.4, 0.25])
    got = B.poly_norm(dev(z), dev(coef), 1e-6).cpu().double()
    want = plain.poly_norm(z.double(), coef.double(), 1e-6)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert (got - want).abs().max() <= tol * float(want.abs().max())


# ------------------------------------------------------------------------------------------ differential attention
def _qkv_rows(lengths, nq, nkv, d, dv, dtype, extra=3):
    return [torch.randn(m, (nq + nkv) * 2 * d + nkv * dv + extra).to(dtype) for m in lengths]


def _plain_maps(x, nq, nkv, d, dv, qw, kw, eps, freqs, first=0):
    """The plain q ``[T, nq, 2, d]``, k ``[T, nkv, 2, d]`` and v ``[T, nkv, dv]`` of rows ``[q | k | v]`` at positions from ``first``."""

    T = x.shape[0]
    q = x[:, : nq * 2 * d].reshape(T, nq, 2, d)
    k = x[:, nq * 2 * d : (nq + nkv) * 2 * d].reshape(T, nkv, 2, d)
    v = x[:, (nq + nkv) * 2 * d : (nq + nkv) * 2 * d + nkv * dv].reshape(T, nkv, dv)
    q, k = plain.unit(q, eps) * qw, plain.unit(k, eps) * kw
    if freqs is not None:
        positions = torch.arange(first, first + T, dtype=x.dtype)
        q, k = plain.rotate(q, positions, freqs), plain.rotate(k, positions, freqs)
    return q, k, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("extra", [3, 0])
@pytest.mark.parametrize("nq,nkv,d,dv,rot,page", [(3, 1, 8, 12, 4, 4), (2, 2, 16, 8, 16, 16), (4, 2, 24, 40, 0, 8), (6, 3, 64, 32, 32, 16),
                                                  (2, 1, 128, 256, 64, 16), (2, 1, 48, 80, 24, 16)])
def test_map_norm_rotation_and_page_write(dtype, nq, nkv, d, dv, rot, page, extra):
    """Each map of q and k normed with the shared weight and rotated on its leading columns by the token's position; k and v
    land in the request's pages.  The second request starts behind 37 cached tokens, so its positions do not start at 0.
    Rows with columns behind them that are no multiple of four values are moved value by value, the others four at a time."""

    from llm_runtime_study_b200.ops import attention_diff as A

    torch.manual_seed(d + dv)
    lengths, q_lens, eps = [21, 50], [21, 13], 1e-5
    scaling = {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 32}
    freqs = plain.scaled_frequencies(rot, 300.0, scaling, torch.float64) if rot else None
    rows = _qkv_rows(q_lens, nq, nkv, d, dv, dtype, extra)
    qw, kw = 1 + 0.2 * torch.randn(d), 1 + 0.2 * torch.randn(d)
    table, pages = _pages(d, page, lengths)
    ctx = _ctx(lengths, q_lens)
    k_pool = torch.zeros(pages, nkv, page, 2 * d, dtype=dtype, device=DEV)
    v_pool = torch.zeros(pages, nkv, page, dv, dtype=dtype, device=DEV)
    q = A.map_norm_rope_write(dev(torch.cat(rows)), num_q_heads=nq, num_kv_heads=nkv, maps=2, head_dim=d, value_dim=dv,
                              q_weight=dev(qw), k_weight=dev(kw), eps=eps, inv_freq=dev(freqs.float()) if rot else None, rotary_dim=rot,
                              positions=ctx.positions, token_entry=ctx.token_entry, block_table=dev(table), page_size=page,
                              k_pool=k_pool, v_pool=v_pool).cpu().double()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    at = 0
    for e, (m, n) in enumerate(zip(lengths, q_lens)):
        pq, pk, pv = _plain_maps(rows[e].double(), nq, nkv, d, dv, qw.double(), kw.double(), eps, freqs, first=m - n)
        assert (q[at:at + n].view(n, nq, 2, d) - pq).abs().max() <= tol * float(pq.abs().max())
        for i, t in enumerate(range(m - n, m)):
            slot = (int(table[e, t // page]), slice(None), t % page)
            assert (k_pool[slot].cpu().double().view(nkv, 2, d) - pk[i]).abs().max() <= tol * float(pk.abs().max())
            assert torch.equal(v_pool[slot].cpu().double(), pv[i])
        at += n
    written = sum(q_lens) * nkv * 2 * d
    assert int((k_pool != 0).sum()) <= written          # no other row of the pool is touched


def _diff_case(dtype, lengths, nq, nkv, d, dv, page, seed, gain=1.0):
    """Random q for every position of each sequence and k, v in scattered pages; returns (q per sequence, k, v, pools, table)."""

    torch.manual_seed(seed)
    q = [(gain * torch.randn(m, nq, 2, d)).to(dtype) for m in lengths]
    k = [(gain * torch.randn(m, nkv, 2, d)).to(dtype) for m in lengths]
    v = [torch.randn(m, nkv, dv).to(dtype) for m in lengths]
    table, pages = _pages(seed, page, lengths)
    k_pool, v_pool = torch.zeros(pages, nkv, page, 2 * d, dtype=dtype), torch.zeros(pages, nkv, page, dv, dtype=dtype)
    _fill(k_pool, table, page, [x.reshape(x.shape[0], nkv, 2 * d) for x in k])
    _fill(v_pool, table, page, v)
    return q, k, v, dev(k_pool), dev(v_pool), table


def _run_diff(kind, q, k_pool, v_pool, ctx, table, **kw):
    from llm_runtime_study_b200.ops import attention_diff as A

    if kind == "mma":
        return A.diff_attention_mma(q, k_pool, v_pool, ctx, dev(table), **kw).cpu().double()
    return A.diff_attention_simt(q, k_pool, v_pool, positions=ctx.positions, token_entry=ctx.token_entry, block_table=dev(table),
                                 **kw).cpu().double()


DIFF_SIZES = [("simt", torch.float32, 3, 1, 8, 12, 4), ("simt", torch.float32, 4, 2, 24, 40, 8), ("simt", torch.bfloat16, 2, 2, 16, 8, 16),
              ("simt", torch.float32, 5, 5, 40, 24, 16), ("mma", torch.bfloat16, 4, 2, 32, 64, 16), ("mma", torch.bfloat16, 2, 1, 64, 32, 4),
              ("mma", torch.bfloat16, 3, 3, 16, 16, 8), ("mma", torch.bfloat16, 8, 1, 48, 80, 16), ("mma", torch.bfloat16, 70, 1, 16, 32, 16),
              ("mma", torch.bfloat16, 2, 2, 128, 128, 16)]


@pytest.mark.parametrize("kind,dtype,nq,nkv,d,dv,page", DIFF_SIZES)
@pytest.mark.parametrize("q_lens,window", [([150, 41], 9), ([150, 41], 0), ([1, 1], 40), ([2, 37], 33), ([1, 41], 0)])
def test_differential_attention_against_plain(kind, dtype, nq, nkv, d, dv, page, q_lens, window):
    """Both kernels, prompt portions behind cached tokens and single tokens, several tokens and head groups a tile: the
    second map subtracted, the head's unit norm and the scale."""

    lengths, lam, out_scale, eps = [150, 41], 0.37, 0.7, 1e-5
    q, k, v, k_pool, v_pool, table = _diff_case(dtype, lengths, nq, nkv, d, dv, page, seed=d + nq)
    ctx = _ctx(lengths, q_lens)
    new = torch.cat([x[m - n:] for x, m, n in zip(q, lengths, q_lens)]).reshape(sum(q_lens), nq, 2 * d)
    got = _run_diff(kind, dev(new), k_pool, v_pool, ctx, table, scale=0.3, window=window, lam=lam, out_scale=out_scale, eps=eps)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    at = 0
    for e, (m, n) in enumerate(zip(lengths, q_lens)):
        want = plain.differential_read_out(q[e].double(), k[e].double(), v[e].double(), scale=0.3, window=window or None, lam=lam,
                                           out_scale=out_scale, eps=eps)[m - n:]
        err = float((got[at:at + n] - want).abs().max())
        assert err <= tol * max(1.0, float(want.abs().max())), (e, err)
        at += n


@pytest.mark.parametrize("nq,nkv,d,dv", [(4, 2, 32, 48), (8, 2, 32, 64), (6, 1, 16, 32), (16, 1, 64, 64), (40, 2, 16, 16)])
def test_single_tokens_whose_keys_are_cut_into_parts(nq, nkv, d, dv):
    """Three requests of unequal length, one token each: the longest is cut into several parts that a second launch merges
    per map before the maps are subtracted; a part may hold no visible key at all (the short request).  Up to 16 heads a
    key/value head take the kernel's form in which a map's warps share out the value columns (in four parts, two or one by
    the value size); more heads take the form of the prompt portions."""

    from llm_runtime_study_b200.ops import attention_diff as A

    page = 16
    lengths = [1500, 3, 700]
    for window in (0, 600):
        keys = min(window, max(lengths)) if window else max(lengths)
        assert A.decode_splits(len(lengths) * nkv, keys) > 1
        q, k, v, k_pool, v_pool, table = _diff_case(torch.bfloat16, lengths, nq, nkv, d, dv, page, seed=window + 1)
        ctx = _ctx(lengths, [1, 1, 1])
        new = torch.cat([x[-1:] for x in q]).reshape(3, nq, 2 * d)
        kw = dict(scale=0.3, window=window, lam=0.6, out_scale=0.8, eps=1e-6)
        got = _run_diff("mma", dev(new), k_pool, v_pool, ctx, table, **kw)
        one = _run_diff("mma", dev(new), k_pool, v_pool, _ctx(lengths, [1, 1, 1]), table, splits=1, **kw)
        for e in range(3):
            want = plain.differential_read_out(q[e].double(), k[e].double(), v[e].double(), **{**kw, "window": window or None})[-1]
            assert (got[e] - want).abs().max() <= 3e-2 * max(1.0, float(want.abs().max())), (window, e)
            assert (one[e] - want).abs().max() <= 3e-2 * max(1.0, float(want.abs().max())), (window, e)


def _marked_case(dtype, which, page, length, marked, seed):
    """One sequence in which key ``marked`` stands out in map ``which`` alone (every query's map points at it; the other map
    points away from it) and carries a value of 4 in column 1: a query that sees it gets 4 (first map) or ``-lam * 4``
    (second map) there, one that does not gets little."""

    torch.manual_seed(seed)
    nq, nkv, d, dv = 2, 1, 16, 16
    q, k, v = 0.3 * torch.randn(length, nq, 2, d), 0.3 * torch.randn(length, nkv, 2, d), 0.3 * torch.randn(length, nkv, dv)
    k[marked] = 0.0
    k[marked, :, which, 1] = 4.0
    q[:, :, which, 1] = 4.0
    k[marked, :, 1 - which, 2] = -4.0        # the other map turns away from the marked key
    q[:, :, 1 - which, 2] = 4.0
    v[marked] = 0.0
    v[marked, :, 1] = 4.0
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    table, pages = _pages(seed + length, page, [length])
    k_pool, v_pool = torch.zeros(pages, nkv, page, 2 * d, dtype=dtype), torch.zeros(pages, nkv, page, dv, dtype=dtype)
    _fill(k_pool, table, page, [k.reshape(length, nkv, 2 * d)])
    _fill(v_pool, table, page, [v])
    return q, k, v, dev(k_pool), dev(v_pool), table


@pytest.mark.parametrize("kind,dtype", [("simt", torch.float32), ("simt", torch.bfloat16), ("mma", torch.bfloat16)])
@pytest.mark.parametrize("page,window,marked", [(16, 40, 15), (16, 40, 16), (8, 9, 63), (4, 5, 100), (16, 0, 3), (16, 64, 31), (16, 33, 32)])
@pytest.mark.parametrize("which", [0, 1])
@pytest.mark.parametrize("new", ["prompt", "single"])
def test_a_key_at_the_windows_edge_and_a_far_key(kind, dtype, page, window, marked, which, new):
    """In a whole prompt and for single tokens behind cached ones, in either map: the last position that sees the marked key
    shows its value, the next one does not; without a window a key hundreds of positions back is found.  The marked key sits
    at a page's border in several cases."""

    length, lam = 700, 0.5
    q, k, v, k_pool, v_pool, table = _marked_case(dtype, which, page, length, marked, seed=marked + which)
    kw = dict(scale=1.0, window=window, lam=lam, out_scale=1.0, eps=1e-6, normalise=False)
    want = plain.differential_read_out(q.double(), k.double(), v.double(), **{**kw, "window": window or None})
    last_seen = marked + window - 1 if window else length - 1
    places = sorted({marked, last_seen - 1, last_seen, min(last_seen + 1, length - 1), min(last_seen + 2, length - 1)})
    flat = q.reshape(length, 2, 32)
    if new == "prompt":
        out = _run_diff(kind, dev(flat), k_pool, v_pool, _ctx([length], [length]), table, **kw)
        assert (out - want).abs().max() <= (2e-5 if dtype == torch.float32 else 3e-2)
        probes = {p: out[p] for p in places}
    else:
        probes = {}
        for p in places:
            probes[p] = _run_diff(kind, dev(flat[p:p + 1].contiguous()), k_pool, v_pool, _ctx([p + 1], [1]), table, **kw)[0]
            assert (probes[p] - want[p]).abs().max() <= (2e-5 if dtype == torch.float32 else 3e-2)
    shown = 4.0 if which == 0 else -lam * 4.0
    for p, row in probes.items():
        if p <= last_seen:
            assert (row[:, 1] - shown).abs().max() < 0.5, (p, row[:, 1])
        else:
            assert row[:, 1].abs().max() < 1.0, (p, row[:, 1])


def test_the_chooser_takes_the_tensor_cores_where_the_sizes_allow():
    from llm_runtime_study_b200.ops import attention_diff as A

    assert A.supported(48, 80) and A.supported(16, 256) and not A.supported(24, 32) and not A.supported(32, 40) and not A.supported(272, 16)
    lengths, q_lens = [70, 9], [70, 9]
    for d, dv, dtype in ((16, 32, torch.bfloat16), (24, 32, torch.bfloat16), (16, 32, torch.float32)):
        q, k, v, k_pool, v_pool, table = _diff_case(dtype, lengths, 2, 1, d, dv, 16, seed=d)
        cache = SimpleNamespace(keys=k_pool, values=v_pool)
        new = torch.cat(q).reshape(sum(q_lens), 2, 2 * d)
        kw = dict(scale=0.2, window=20, lam=0.3, out_scale=0.9, eps=1e-5)
        got = A.diff_attention(dev(new), cache, _ctx(lengths, q_lens), dev(table), **kw).cpu().double()
        want = torch.cat([plain.differential_read_out(a.double(), b.double(), c.double(), **kw) for a, b, c in zip(q, k, v)])
        assert (got - want).abs().max() <= (2e-5 if dtype == torch.float32 else 3e-2) * max(1.0, float(want.abs().max()))


# ------------------------------------------------------------------------------------------ feed-forward parts
def _runtime(dtype):
    from llm_runtime_study_b200.parts import Runtime

    return Runtime(torch.device(DEV), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,ff,experts,top,shared", [(70, 48, 40, 5, 2, 16), (3, 64, 24, 3, 3, None), (200, 32, 16, 7, 1, 48),
                                                           (1, 40, 72, 12, 3, 8), (700, 64, 48, 5, 2, 32)])
def test_sigmoid_routed_experts_with_weights_on_their_inputs(dtype, n, width, ff, experts, top, shared):
    """The part as the model builds it: sigmoid scores that are not renormalised, the score times the expert's input, a
    shared expert for every token.  The last case brings enough rows for the wide tiles of the bfloat16 run type."""

    from llm_runtime_study_b200.parts import FEED_FORWARDS

    torch.manual_seed(n + top)
    part = FEED_FORWARDS.build({"kind": "routed_experts", "hidden_size": width, "intermediate_size": ff, "experts": experts, "top": top,
                                "act": "silu_glu", "score": "sigmoid", "weight_on": "input", "router_bias": False, "shared_size": shared})
    W = {"router": torch.randn(experts, width)}
    for e in range(experts):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = (0.3 * torch.randn(ff, width), 0.3 * torch.randn(ff, width), 0.3 * torch.randn(width, ff))
    if shared:
        W["shared.gate"], W["shared.up"], W["shared.down"] = (0.3 * torch.randn(shared, width), 0.3 * torch.randn(shared, width),
                                                              0.3 * torch.randn(width, shared))
    assert set(part.tensor_specs()) == set(W)
    W = {name: t.to(dtype) for name, t in W.items()}
    part.load(W, _runtime(dtype))
    h = torch.randn(n, width).to(dtype)
    got = part.forward(dev(h), None).cpu().double()
    store = plain.round_bfloat16 if dtype == torch.bfloat16 else plain.keep
    margins = []
    want = plain.routed_ff(h.double(), {k: v.double() for k, v in W.items()}, {"router": {"experts": experts, "top": top}, "shared": shared},
                           store, margins)
    clear = margins[0] > 1e-3
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    assert ((got - want).abs().amax(dim=1)[clear]).max() <= tol * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_feed_forward_with_the_polynomial_activation(dtype):
    from llm_runtime_study_b200.parts import FEED_FORWARDS

    torch.manual_seed(12)
    width, ff, n, eps = 40, 72, 29, 1e-5
    part = FEED_FORWARDS.build({"kind": "poly_norm_mlp", "hidden_size": width, "intermediate_size": ff, "eps": eps})
    W = {"up": 0.4 * torch.randn(ff, width), "down": 0.4 * torch.randn(width, ff), "act": torch.tensor([0.9, -0.4, 0.3, 0.1])}
    assert set(part.tensor_specs()) == set(W)
    W = {name: t.to(dtype) for name, t in W.items()}
    part.load(W, _runtime(dtype))
    h = torch.randn(n, width).to(dtype)
    got = part.forward(dev(h), None).cpu().double()
    store = plain.round_bfloat16 if dtype == torch.bfloat16 else plain.keep
    want = plain.dense_ff(h.double(), {k: v.double() for k, v in W.items()}, eps, store)
    assert (got - want).abs().max() <= (3e-5 if dtype == torch.float32 else 3e-2) * max(1.0, float(want.abs().max()))


# ------------------------------------------------------------------------------------------ whole models
LENGTHS = {"A": [1, 2, 5, 23, 64, 65, 131], "B": [3, 17, 48, 70, 1, 129], "C": [140, 2, 37, 66, 300]}


def _requests(name):
    config, seed, _ = helpers.MABEDRA[name]
    rng = random.Random(seed + 1)
    return {f"r{i}": helpers.random_tokens(rng, config["vocab"], n) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B", "C") for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    from llm_runtime_study_b200.engine.runtime import load

    name, dtype = request.param
    config, seed, page = helpers.MABEDRA[name]
    path, weights = helpers.make_mabedra_dir(tmp_path_factory.mktemp(f"mabedra{name}{dtype}"), config, seed, torch_dtype=dtype)
    requests = _requests(name)
    store = plain.round_bfloat16 if dtype == "bfloat16" else plain.keep
    expected, clear = {}, {}
    for rid, tokens in requests.items():
        margins = []
        expected[rid] = plain.forward(config, weights, tokens, store=store, margins=margins)
        clear[rid] = torch.stack(margins).min(dim=0).values > CLOSE_CALL if margins else torch.ones(len(tokens), dtype=torch.bool)
    loaded = load(path, device=DEV, dtype=dtype, strict_dtype=False)
    return dict(name=name, dtype=dtype, config=config, page=page, path=path, requests=requests, plain=expected, loaded=loaded,
                weights=weights, clear=clear)


def _replay(setup, steps, *, max_requests=4, max_tokens=None):
    from llm_runtime_study_b200.engine.replay import TraceReplayer

    replayer = TraceReplayer(setup["loaded"], max_tokens=max_tokens or helpers.pool_tokens(steps), page_size=setup["page"],
                             max_requests=max_requests)
    outputs = {}
    for record in steps:
        rows = replayer.run_step(record)
        if rows is not None:
            outputs[record["step"]] = torch.from_numpy(np.array(rows))
    manager = replayer.runner.manager
    manager.check()
    assert manager.active_sequences == 0 and manager.all_free and manager.free_slots == max_requests
    return helpers.collect_logits(steps, outputs)


def _compare(setup, got, requests=None):
    for rid, tokens in (requests or setup["requests"]).items():
        assert sorted(got[rid]) == list(range(len(tokens))), rid
        rows = torch.stack([got[rid][p] for p in range(len(tokens))]).double()
        if setup["dtype"] == "bfloat16":
            want = setup["plain"][rid]
            err = (rows - want).pow(2).mean(dim=1).sqrt() / want.pow(2).mean(dim=1).sqrt()
            assert torch.isfinite(err).all()
            clear = setup["clear"][rid]
            assert int(clear.sum()) >= len(tokens) // 2, "the weights make too many close calls for this test to compare anything"
            err = torch.where(clear, err, torch.zeros_like(err))
            assert float(err.max()) <= BF16_WORST, (rid, int(err.argmax()), float(err.max()))
            over = int((err > BF16_USUAL).sum())
            assert over <= max(1, len(tokens) // 10), f"request {rid}: {over} of {len(tokens)} rows beyond {BF16_USUAL}: {err}"
            continue
        bad, err, top = helpers.first_wrong_row(rows, setup["plain"][rid], TOL[setup["dtype"]])
        assert bad is None, f"request {rid}: first wrong position {bad} of {len(tokens)}, rms and largest |diff| / rms {err:.3e}, {top:.3e}"


def test_the_stream_after_every_layer(setup, monkeypatch):
    """Layer by layer: the averaged stream that each layer hands on, for one request in one step."""

    from llm_runtime_study_b200.engine.replay import TraceReplayer
    from llm_runtime_study_b200.parts.block import ParallelSublayersBlock

    if setup["dtype"] != "float32":
        pytest.skip("compared sharply in 32-bit")
    tokens = max(setup["requests"].values(), key=len)[:50]
    want, seen = [], []
    plain.forward(setup["config"], setup["weights"], tokens, layers_out=want)
    inner = ParallelSublayersBlock.forward

    def watched(self, stream, ctx, cache):
        inner(self, stream, ctx, cache)
        assert stream.delta is None
        seen.append(stream.resid.clone())

    monkeypatch.setattr(ParallelSublayersBlock, "forward", watched)
    replayer = TraceReplayer(setup["loaded"], max_tokens=64, page_size=setup["page"], max_requests=1)
    replayer.run_step({"step": 0, "entries": [{"id": "x", "tokens": tokens, "want": []}], "end": ["x"]})
    assert len(seen) == len(want)
    for i, (a, b) in enumerate(zip(seen, want)):
        assert (a.cpu().double() - b).abs().max() <= 1e-4 * max(1.0, float(b.abs().max())), i


def test_whole_prompts(setup):
    _compare(setup, _replay(setup, helpers.trace_whole(setup["requests"])))


def test_prefill_then_token_by_token(setup):
    """The tail is longer than every window but the widest, so windows pass over decoded tokens and pages behind them are
    given back."""

    _compare(setup, _replay(setup, helpers.trace_decode_tail(setup["requests"], tail=40)))


def test_portions_down_to_two_tokens(setup):
    rng = random.Random(5)
    _compare(setup, _replay(setup, helpers.trace_chunked(setup["requests"], rng, sizes=(2, 3, 2, 7, 13, 16, 17, 31))))


def test_mixed_batches_with_slots_and_pages_used_again(setup):
    """Three slots for all requests, portions beside single tokens, and a pool sized for what is live."""

    rng = random.Random(9)
    steps = helpers.trace_mixed(setup["requests"], rng, live_max=3, tail=6)
    _compare(setup, _replay(setup, steps, max_requests=3))


def test_every_token_decoded_alone(setup):
    """A sequence fed one token a step from its first token: the first tokens (shorter than the convolution's reach and than
    every window), long decoding."""

    requests = {rid: tokens for rid, tokens in setup["requests"].items() if len(tokens) in (23, 131, 70, 66)}
    _compare(setup, _replay(setup, helpers.trace_decode_tail(requests, tail=10_000)), requests)


def test_a_cut_changes_no_bit_in_float32(setup):
    if setup["dtype"] != "float32":
        pytest.skip("the 32-bit path is the one whose sums have an order fixed by the position")
    whole = _replay(setup, helpers.trace_whole(setup["requests"]))
    cut = _replay(setup, helpers.trace_chunked(setup["requests"], random.Random(1), sizes=(2, 5, 9)))
    for rid, rows in whole.items():
        for p, row in rows.items():
            assert torch.equal(row, cut[rid][p]), (rid, p)


def test_a_reused_slot_starts_from_zero(setup):
    """One slot: the second request takes the first one's kept convolution inputs and pages."""

    requests = {rid: tokens for rid, tokens in setup["requests"].items() if len(tokens) in (23, 17, 48, 65, 37, 66)}
    _compare(setup, _replay(setup, helpers.trace_chunked(requests, random.Random(3), sizes=(7, 16)), max_requests=1), requests)


def test_greedy_generation_through_the_engine(setup):
    """``Engine.generate`` with its scheduler (prompt portions, batching, graph decode where the model allows) gives the
    plain model's greedy tokens."""

    from llm_runtime_study_b200.engine.engine import Engine
    from llm_runtime_study_b200.sampling import SamplingConfig

    if setup["dtype"] != "float32":
        pytest.skip("greedy ties are decided by rounding in bfloat16")
    config, weights = setup["config"], setup["weights"]
    prompts = [setup["requests"]["r3"][:19], setup["requests"]["r2"], setup["requests"]["r1"] + [3, 1, 4]]
    new = 12
    want = []
    for prompt in prompts:
        tokens = list(prompt)
        for _ in range(new):
            tokens.append(int(plain.forward(config, weights, tokens)[-1].argmax()))
        want.append(tokens[len(prompt):])
    engine = Engine.from_model_dir(setup["path"], device=DEV, dtype="float32", max_seq_len=64, max_batch_size=2, page_size=setup["page"],
                                   max_tokens_per_step=16, strict_dtype=False)
    got = [[] for _ in prompts]
    for index, event in engine.generate(prompts, max_new_tokens=new, sampling=SamplingConfig(temperature=0.0)):
        if event.token_id is not None:
            got[index].append(event.token_id)
    assert got == want


def test_generation_in_bfloat16_follows_the_plain_model_until_a_close_call(setup):
    """The bfloat16 run type through the engine (tensor-core attention, graph decode): every generated token is the plain
    model's choice or one whose logit the plain model puts within rounding of the best."""

    from llm_runtime_study_b200.engine.engine import Engine
    from llm_runtime_study_b200.sampling import SamplingConfig

    if setup["dtype"] != "bfloat16":
        pytest.skip("the 32-bit run type is compared token by token above")
    config, weights = setup["config"], setup["weights"]
    prompts = [setup["requests"]["r3"][:30], setup["requests"]["r2"]]
    engine = Engine.from_model_dir(setup["path"], device=DEV, dtype="bfloat16", max_seq_len=96, max_batch_size=2, page_size=setup["page"],
                                   max_tokens_per_step=16, strict_dtype=False)
    got = [[] for _ in prompts]
    for index, event in engine.generate(prompts, max_new_tokens=10, sampling=SamplingConfig(temperature=0.0)):
        if event.token_id is not None:
            got[index].append(event.token_id)
    for prompt, new in zip(prompts, got):
        assert len(new) == 10
        tokens = list(prompt)
        for token in new:
            logits = plain.forward(config, weights, tokens, store=plain.round_bfloat16)[-1]
            spread = float(logits.std())
            assert float(logits.max() - logits[token]) <= 0.25 * spread, (len(tokens), token, int(logits.argmax()))
            tokens.append(token)


def test_command_line_and_trace_runner(tmp_path):
    """The command line writes a folder of random weights for the design and generates from it; the trace runner,
    started as a program with four request slots, replays a mixed trace on that folder."""

    import io
    import json
    import subprocess
    import sys
    from pathlib import Path

    from llm_runtime_study_b200.cli import main
    from llm_runtime_study_b200.weights import Checkpoint

    config = helpers.MABEDRA_B
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(config))
    out, err = io.StringIO(), io.StringIO()
    code = main(["--model", str(tmp_path / "m"), "--random-weights", str(config_path), "--weights-seed", "4",
                 "--prompt-ids", "5 17 3 90", "--max-new-tokens", "5", "--max-seq-len", "64", "--dtype", "float32", "--no-stream"],
                output=out, error=err)
    assert code == 0, err.getvalue()
    generated = [int(t) for t in out.getvalue().splitlines()[0].split()]
    weights = Checkpoint.from_model_dir(tmp_path / "m").get_tensors()
    tokens = [5, 17, 3, 90]
    for got in generated:
        logits = plain.forward(config, weights, tokens)[-1]
        top = torch.topk(logits, 2).values
        if float(top[0] - top[1]) < 1e-4:        # a tie: either token is right, and what follows differs
            break
        assert got == int(logits.argmax())
        tokens.append(got)
    rng = random.Random(2)
    requests = {f"q{i}": helpers.random_tokens(rng, config["vocab"], n) for i, n in enumerate([9, 30, 2, 17, 40])}
    steps = helpers.trace_mixed(requests, rng, live_max=4, tail=5)
    root = Path(__file__).resolve().parent.parent
    run = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32",
                          "--out", str(tmp_path / "out"), "--max-tokens", str(helpers.pool_tokens(steps))],
                         input=helpers.dump_trace(steps), capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [line for line in run.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outputs = {s["step"]: torch.from_numpy(np.fromfile(tmp_path / "out" / f"{s['step']}.f32", dtype="<f4").reshape(-1, config["vocab"]))
               for s in steps if any(e["want"] for e in s["entries"])}
    got = helpers.collect_logits(steps, outputs)
    for rid, toks in requests.items():
        want = plain.forward(config, weights, toks)
        rows = torch.stack([got[rid][p] for p in range(len(toks))]).double()
        bad, rms_err, top_err = helpers.first_wrong_row(rows, want, TOL["float32"])
        assert bad is None, (rid, bad, rms_err, top_err)
