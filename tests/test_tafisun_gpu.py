"""Tafisun through the framework against the plain implementation: every mechanism's kernels alone (with inputs made so
that a key at a block's edge, a far key or a page border shows), then whole models under every way of cutting the work
(whole prompts, decoding token by token, portions down to two tokens, mixed batches whose pages and slots are used
again), in 32-bit and in bfloat16, and greedy generation through the engine's own entry point."""

import math
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from tests import helpers
from tests.plain import tafisun_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# a row of logits against the plain model in 64-bit, as fractions of the row's root mean square: (rms, largest).
# float32 is the sharp comparison.  bfloat16: the plain model rounds its activations where the engine stores them; a
# rounding that falls the other way moves single rows by several per cent, so a request passes when at most a tenth of its
# rows (or one) is beyond BF16_USUAL and none beyond BF16_WORST.  A row at which some router's choice was closer than
# CLOSE_CALL is not compared: there the two models may rightly send the token to different experts.
TOL = {"float32": (3e-5, 2e-4)}
BF16_USUAL, BF16_WORST, CLOSE_CALL = 6e-2, 5e-1, 0.02


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


def _batch(lengths):
    positions = torch.cat([torch.arange(m) for m in lengths]).int()
    entry = torch.cat([torch.full((m,), i) for i, m in enumerate(lengths)]).int()
    return positions, entry


def _ctx(lengths, q_lens):
    """What the kernel chooser reads of a step's context: every sequence of ``lengths`` brings its last ``q_lens`` tokens."""

    positions = torch.cat([torch.arange(m - k, m) for m, k in zip(lengths, q_lens)]).int()
    entry = torch.cat([torch.full((k,), i) for i, k in enumerate(q_lens)]).int()
    return SimpleNamespace(positions=dev(positions), token_entry=dev(entry), all_decode=max(q_lens) == 1, num_entries=len(lengths),
                           q_lens=list(q_lens), kv_lens=list(lengths), max_kv_len=max(lengths), max_q_len=max(q_lens),
                           kv_len=dev(torch.tensor(lengths, dtype=torch.int32)))


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,buckets,mul_prev,mul_cur", [(10, 7, 3, 5), (64, 13, 40_000_003, 11), (7, 1, 1, 1), (48, 257, 1, 0)])
def test_summed_embedding_across_portions_and_slots(dtype, hidden, buckets, mul_prev, mul_cur):
    """Token row, hashed bigram row and sinusoid; the token before a portion comes from the request's slot, position 0 reads
    the table's last row, a slot taken by a new request forgets the old one's token, and positions far out stay exact."""

    from llm_runtime_study_b200.ops import functional as F

    torch.manual_seed(hidden)
    vocab = 50
    table, bigram = torch.randn(vocab, hidden).to(dtype), torch.randn(buckets + 1, hidden).to(dtype)
    freq = torch.tensor([10000.0 ** (-2.0 * i / hidden) for i in range((hidden + 1) // 2)], dtype=torch.float64)
    previous = torch.full((4, 1), 17, dtype=torch.int32, device=DEV)         # whatever an earlier request left there
    rng = random.Random(buckets)
    seqs = {2: [rng.randrange(vocab) for _ in range(23)], 0: [rng.randrange(vocab) for _ in range(9)]}

    def want(tokens, first, n, start=0):
        rows = plain.bigram_rows(tokens, buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur)[first:first + n]
        pos = torch.zeros(n, hidden, dtype=torch.float64)
        for j in range(n):
            for c in range(hidden):
                angle = (start + first + j) * float(freq[c // 2])
                pos[j, c] = math.sin(angle) if c % 2 == 0 else math.cos(angle)
        return (table.double()[tokens[first:first + n]] + bigram.double()[rows]) + pos

    done = {2: 0, 0: 0}
    for cuts in ([(2, 5), (0, 2)], [(0, 6), (2, 1)], [(2, 17)], [(0, 1)]):
        ids = torch.tensor([t for slot, n in cuts for t in seqs[slot][done[slot]:done[slot] + n]], dtype=torch.int32)
        positions = torch.cat([torch.arange(done[slot], done[slot] + n) for slot, n in cuts]).int()
        entry = torch.cat([torch.full((n,), i) for i, (_, n) in enumerate(cuts)]).int()
        q_start = torch.tensor([0] + list(np.cumsum([n for _, n in cuts])), dtype=torch.int32)
        slots = torch.tensor([slot for slot, _ in cuts], dtype=torch.int32)
        out = F.embedding_sum(dev(ids), dev(table), dev(bigram), positions=dev(positions), token_entry=dev(entry), q_start=dev(q_start),
                              slots=dev(slots), previous=previous, freq=dev(freq), buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur)
        at = 0
        for slot, n in cuts:
            assert (out[at:at + n].cpu().double() - want(seqs[slot], done[slot], n)).abs().max() < 2e-6, (slot, done[slot])
            done[slot] += n
            at += n
            assert int(previous[slot, 0]) == seqs[slot][done[slot] - 1]
    assert previous[1, 0] == 17 and previous[3, 0] == 17
    # far out: the angle is formed in 64-bit
    far = 3_000_001
    ids = torch.tensor([4, 9], dtype=torch.int32)
    out = F.embedding_sum(dev(ids), dev(table), None, positions=dev(torch.tensor([far, far + 1], dtype=torch.int32)),
                          token_entry=dev(torch.zeros(2, dtype=torch.int32)), q_start=dev(torch.tensor([0, 2], dtype=torch.int32)),
                          slots=dev(torch.tensor([1], dtype=torch.int32)), previous=None, freq=dev(freq)).cpu().double()
    for j in range(2):
        for c in range(hidden):
            angle = (far + j) * float(freq[c // 2])
            assert abs(float(out[j, c]) - float(table[ids[j], c]) - (math.sin(angle) if c % 2 == 0 else math.cos(angle))) < 2e-6


def _attention_case(dtype, nq, nkv, d, page, lengths, seed):
    """Rows [q | k | g-sized rest] of a stacked projection for whole sequences, the pools after the norm-and-write kernel,
    and the plain q, k (normed) and v (the keys as projected)."""

    from llm_runtime_study_b200.ops import mixer_steps as M

    torch.manual_seed(seed)
    n = sum(lengths)
    rows = torch.randn(n, (nq + nkv) * d + 8).to(dtype)
    qw, kw = (1 + 0.3 * torch.randn(d)), (1 + 0.3 * torch.randn(d))
    table, pages = _pages(seed, page, lengths)
    positions, entry = _batch(lengths)
    k_pool = torch.zeros(pages, nkv, page, d, dtype=dtype, device=DEV)
    v_pool = torch.zeros(pages, nkv, page, d, dtype=dtype, device=DEV)
    eps = 1e-5
    q = M.head_norm_write(dev(rows), num_q_heads=nq, num_kv_heads=nkv, head_dim=d, value_dim=d, eps=eps, q_weight=dev(qw), k_weight=dev(kw),
                          positions=dev(positions), token_entry=dev(entry), block_table=dev(table), page_size=page, k_pool=k_pool,
                          v_pool=v_pool, value_offset=nq * d)
    x = rows.double()
    pq = plain.rms_norm(x[:, : nq * d].view(n, nq, d), qw.double(), eps)
    pv = x[:, nq * d : (nq + nkv) * d].view(n, nkv, d)
    pk = plain.rms_norm(pv, kw.double(), eps)
    if dtype == torch.bfloat16:
        pq, pk = pq.bfloat16().double(), pk.bfloat16().double()
    return SimpleNamespace(q=q, pq=pq, pk=pk, pv=pv, table=table, positions=positions, entry=entry, k_pool=k_pool, v_pool=v_pool)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,page,chunk", [(4, 2, 16, 4, 6), (3, 3, 12, 16, 16), (2, 1, 40, 8, 5), (8, 2, 64, 16, 32), (1, 1, 8, 4, 1)])
def test_head_norm_with_weights_values_from_keys_and_chunked_attention(dtype, nq, nkv, d, page, chunk):
    """The per-head norm with one weight for all heads, the raw keys written as values, and attention under the mask in
    blocks with the bias by the logarithm of the distance, for two sequences in one batch."""

    from llm_runtime_study_b200.ops import functional as F

    lengths = [41, 7]
    case = _attention_case(dtype, nq, nkv, d, page, lengths, seed=d + chunk)
    r1, r2 = torch.rand(nq) * 2, torch.rand(nq)
    out = F.paged_attention_simt_rules(case.q, case.k_pool, case.v_pool, positions=dev(case.positions), token_entry=dev(case.entry),
                                       block_table=dev(case.table), scale=0.4, chunk=chunk, log_bias=(dev(r1), dev(r2))).cpu().double()
    at = 0
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for m in lengths:
        assert (case.q[at:at + m].cpu().double() - case.pq[at:at + m]).abs().max() <= (1e-5 if dtype == torch.float32 else 3e-2)
        want = plain.chunked_attention(case.pq[at:at + m], case.pk[at:at + m], case.pv[at:at + m], scale=0.4, size=chunk, r1=r1.double(), r2=r2.double())
        assert (out[at:at + m] - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
        at += m
    # the pages hold the normed keys and, as values, the keys before their norm
    t, e = 5, 0
    slot = (int(case.table[e, t // page]), t % page)
    assert (case.v_pool[slot[0], :, slot[1]].cpu().double() - case.pv[t]).abs().max() <= (0 if dtype == torch.float32 else 2e-2)
    assert (case.k_pool[slot[0], :, slot[1]].cpu().double() - case.pk[t]).abs().max() <= (1e-5 if dtype == torch.float32 else 3e-2)


def _marked_case(dtype, heads, d, page, length, marked, seed=0):
    """Keys and values of one sequence in scattered pages and a query for every position; key ``marked`` stands out: every
    query points at it, so whether it is seen decides the output."""

    torch.manual_seed(seed)
    k = 0.3 * torch.randn(length, 1, d)
    v = 0.3 * torch.randn(length, 1, d)
    q = 0.3 * torch.randn(length, heads, d)
    k[marked] = 0.0
    k[marked, 0, 1] = 4.0
    v[marked, 0, :] = 3.0
    q[:, :, 1] = 4.0
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    table, pages = _pages(seed + length, page, [length])
    k_pool, v_pool = torch.zeros(pages, 1, page, d, dtype=dtype), torch.zeros(pages, 1, page, d, dtype=dtype)
    for t in range(length):
        k_pool[table[0, t // page], 0, t % page] = k[t, 0]
        v_pool[table[0, t // page], 0, t % page] = v[t, 0]
    return q, k, v, dev(k_pool), dev(v_pool), table


@pytest.mark.parametrize("kernel", ["simt-float32", "simt-bfloat16", "mma"])
@pytest.mark.parametrize("page,chunk,marked", [(16, 40, 40), (16, 40, 79), (16, 64, 64), (16, 64, 127), (8, 9, 63), (4, 5, 100), (16, 1024, 3),
                                               (16, 48, 95), (16, 32, 511)])
@pytest.mark.parametrize("new", ["prompt", "single"])
def test_a_key_at_a_blocks_edge_and_a_far_key(kernel, page, chunk, marked, new):
    """One key stands out.  Queries in its block from its position on give nearly its value; the last position of the block
    still does, the first of the next block does not, nor does the position before the key; in a block longer than the
    sequence a key hundreds of positions back is found.  The marked key sits at a page's border in several cases.  Whole
    prompts and single tokens behind cached ones, on the CUDA cores and on the tensor cores."""

    from llm_runtime_study_b200.ops import attention_rules
    from llm_runtime_study_b200.ops import functional as F

    dtype = torch.float32 if kernel == "simt-float32" else torch.bfloat16
    heads, d, length = 2, 16, 700
    q, k, v, k_pool, v_pool, table = _marked_case(dtype, heads, d, page, length, marked, seed=marked)
    r1, r2 = torch.tensor([0.3, 0.0]), torch.tensor([0.5, 2.0])
    want = plain.chunked_attention(q.double(), k.double(), v.double(), scale=1.0, size=chunk, r1=r1.double(), r2=r2.double())
    block_end = min((marked // chunk + 1) * chunk, length) - 1
    probes = sorted({marked, min(marked + 1, block_end), block_end - 1 if block_end - 1 >= marked else marked, block_end,
                     min(block_end + 1, length - 1), min(block_end + 2, length - 1), max(marked - 1, 0)})
    cache = SimpleNamespace(keys=k_pool, values=v_pool, page_size=page)

    def run(ctx, queries):
        if kernel == "mma":
            return attention_rules.paged_attention_rules(dev(queries), cache, ctx, dev(table), scale=1.0, chunk=chunk,
                                                         log_bias=(dev(r1), dev(r2))).cpu().double()
        return F.paged_attention_simt_rules(dev(queries), k_pool, v_pool, positions=ctx.positions, token_entry=ctx.token_entry,
                                            block_table=dev(table), scale=1.0, chunk=chunk, log_bias=(dev(r1), dev(r2))).cpu().double()

    tol = 2e-5 if dtype == torch.float32 else 3e-2
    if new == "prompt":
        out = run(_ctx([length], [length]), q)
        assert (out - want).abs().max() <= tol
        rows = {p: out[p] for p in probes}
    else:
        rows = {}
        for p in probes:
            rows[p] = run(_ctx([p + 1], [1]), q[p:p + 1].contiguous())[0]
            assert (rows[p] - want[p]).abs().max() <= tol, p
    for p, row in rows.items():
        if marked <= p <= block_end:
            assert (row - 3.0).abs().max() < 0.1, (p, row[0, :3])
        else:
            assert (row - 3.0).abs().min() > 1.5, (p, row[0, :3])


@pytest.mark.parametrize("nq,nkv,d,page,chunk", [(4, 2, 32, 16, 16), (8, 4, 64, 16, 64), (3, 1, 64, 16, 48), (10, 1, 16, 16, 20), (20, 1, 32, 8, 200),
                                                 (2, 2, 128, 16, 33)])
@pytest.mark.parametrize("q_lens", [[150, 41], [1, 1], [2, 37], [70, 1]])
def test_tensor_core_chunked_attention(nq, nkv, d, page, chunk, q_lens):
    """The mma.sync kernels for prompt portions behind cached tokens and for single tokens, tiles that straddle a block's
    edge and several head groups, against the plain attention of each sequence."""

    from llm_runtime_study_b200.ops import attention_rules

    lengths = [150, 41]
    case = _attention_case(torch.bfloat16, nq, nkv, d, page, lengths, seed=nq * d)
    r1, r2 = torch.rand(nq) * 2, torch.rand(nq)
    ctx = _ctx(lengths, q_lens)
    starts = [0, lengths[0]]
    q = torch.cat([case.q[s + m - k:s + m] for s, m, k in zip(starts, lengths, q_lens)]).contiguous()
    cache = SimpleNamespace(keys=case.k_pool, values=case.v_pool, page_size=page)
    assert attention_rules.tensor_core_supported(q, cache)
    got = attention_rules.paged_attention_rules(q, cache, ctx, dev(case.table), scale=0.3, chunk=chunk, log_bias=(dev(r1), dev(r2))).cpu().double()
    at = 0
    for s, m, k in zip(starts, lengths, q_lens):
        want = plain.chunked_attention(case.pq[s:s + m], case.pk[s:s + m], case.pv[s:s + m].bfloat16().double(), scale=0.3, size=chunk,
                                       r1=r1.double(), r2=r2.double())[m - k:]
        assert (got[at:at + k] - want).abs().max() <= 3e-2 * max(1.0, float(want.abs().max())), float((got[at:at + k] - want).abs().max())
        at += k


def test_single_tokens_in_a_long_block_are_cut_into_parts():
    """Three requests of unequal length, one token each, in a block longer than all of them: the longest is cut into
    several parts and merged; a part may hold no visible key at all (the short request)."""

    from llm_runtime_study_b200.ops import attention_bf16, attention_rules

    nq, nkv, d, page, chunk = 4, 2, 64, 16, 4096
    lengths = [1500, 3, 700]
    assert attention_bf16.decode_splits(3, nkv, 1, max(lengths), head_dim=d) > 1
    case = _attention_case(torch.bfloat16, nq, nkv, d, page, lengths, seed=5)
    r1, r2 = torch.rand(nq), torch.rand(nq)
    ctx = _ctx(lengths, [1, 1, 1])
    ends = np.cumsum(lengths)
    q = torch.stack([case.q[e - 1] for e in ends]).contiguous()
    cache = SimpleNamespace(keys=case.k_pool, values=case.v_pool, page_size=page)
    got = attention_rules.paged_attention_rules(q, cache, ctx, dev(case.table), scale=0.3, chunk=chunk, log_bias=(dev(r1), dev(r2))).cpu().double()
    for i, (e, m) in enumerate(zip(ends, lengths)):
        s = e - m
        want = plain.chunked_attention(case.pq[s:e], case.pk[s:e], case.pv[s:e].bfloat16().double(), scale=0.3, size=chunk, r1=r1.double(),
                                       r2=r2.double())[-1]
        assert (got[i] - want).abs().max() <= 3e-2 * max(1.0, float(want.abs().max())), i


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,cuts", [(40, [1, 2, 1, 9, 3, 30]), (7, [5, 1, 1]), (130, [46]), (96, [3, 2, 8, 8, 17])])
def test_mingru_across_cuts(dtype, width, cuts):
    """A sequence fed in portions in a slot between two others: every portion's rows equal the plain whole-sequence values,
    the state carries over, and the neighbours' slots stay untouched."""

    from llm_runtime_study_b200.ops import mixer_steps as M

    torch.manual_seed(width)
    total = sum(cuts)
    other = 4
    proj = (2 * torch.randn(total, 3 * width + 5)).to(dtype)
    proj_other = (2 * torch.randn(other, 3 * width + 5)).to(dtype)
    x = proj.double()
    z = plain.sigmoid(x[:, 2:2 + width])
    S = plain.mingru_scan(z, plain.mingru_candidate(x[:, 2 + width:2 + 2 * width]))
    want = S * plain.silu(x[:, 5 + 2 * width:5 + 3 * width])
    state = torch.zeros(4, width, device=DEV)
    state[0], state[2] = 7.0, -3.0
    at = 0
    for i, n in enumerate(cuts):
        # the sequence's portion beside a one-token entry of another request in slot 3 (its state moves, ours must not notice)
        rows = torch.cat([proj_other[i % other:i % other + 1], proj[at:at + n]])
        q_start = torch.tensor([0, 1, 1 + n], dtype=torch.int32)
        slots = torch.tensor([3, 1], dtype=torch.int32)
        out = M.mingru_scan(dev(rows), width=width, z_offset=2, u_offset=2 + width, g_offset=5 + 2 * width, state=state,
                            q_start=dev(q_start), slots=dev(slots)).cpu().double()
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert (out[1:] - want[at:at + n]).abs().max() <= tol * max(1.0, float(want.abs().max())), (i, at)
        at += n
    # the bfloat16 run type forms its sigmoids with the fast exponential: a few units in the last place of a float32 a step
    assert (state[1].cpu().double() - S[-1]).abs().max() < (2e-5 if dtype == torch.float32 else 2e-4) * max(1.0, float(S[-1].abs().max()))
    assert (state[0] == 7.0).all() and (state[2] == -3.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,q_lens", [(40, [300, 1, 33]), (130, [32, 64, 31]), (7, [1, 1]), (96, [1000])])
def test_mingru_in_segments(dtype, width, q_lens):
    """The form in three launches for long portions: several requests of unequal length in one batch, each continued from
    a state of its own, segments that end with the portion, with a full segment and with one token."""

    from llm_runtime_study_b200.ops import mixer_steps as M

    torch.manual_seed(width + len(q_lens))
    n = sum(q_lens)
    proj = (2 * torch.randn(n, 3 * width)).to(dtype)
    slot_of = [3, 0, 2][: len(q_lens)]
    start = torch.randn(5, width)
    state = dev(start.clone())
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    segments = M.mingru_segment_map(q_lens, slot_of, DEV)
    out = M.mingru_scan(dev(proj), width=width, z_offset=0, u_offset=width, g_offset=2 * width, state=state, q_start=dev(q_start),
                        slots=dev(torch.tensor(slot_of, dtype=torch.int32)), segments=segments).cpu().double()
    at = 0
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for m, slot in zip(q_lens, slot_of):
        x = proj[at:at + m].double()
        z, c = plain.sigmoid(x[:, :width]), plain.mingru_candidate(x[:, width:2 * width])
        S, rows = start[slot].double(), []
        for t in range(m):
            S = (1.0 - z[t]) * S + z[t] * c[t]
            rows.append(S * plain.silu(x[t, 2 * width:]))
        want = torch.stack(rows)
        assert (out[at:at + m] - want).abs().max() <= tol * max(1.0, float(want.abs().max())), (slot, m)
        assert (state[slot].cpu().double() - S).abs().max() < (2e-5 if dtype == torch.float32 else 2e-4) * max(1.0, float(S.abs().max()))
        at += m
    untouched = [s for s in range(5) if s not in slot_of]
    assert torch.equal(state[untouched].cpu(), start[untouched])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,identity,top,groups,keep,width", [(5, 1, 2, 3, 2, 64), (3, 0, 3, 1, 1, 40), (5, 3, 1, 4, 1, 48), (10, 2, 4, 3, 2, 128),
                                                                  (34, 6, 5, 8, 3, 36), (6, 2, 2, 4, 2, 128)])
def test_the_router_with_groups_a_correction_identity_outputs_and_a_gate(dtype, experts, identity, top, groups, keep, width):
    """Choice and weights against the plain router for every token whose choice is clear; an identity output gets no row;
    the gate's sigmoid rides along; the plan sorts the other pairs by expert."""

    from llm_runtime_study_b200.ops import grouped as G

    torch.manual_seed(experts + width)
    n, outputs = 97, experts + identity
    h = torch.randn(n, width).to(dtype)
    router = torch.randn(outputs + 1, width) * 0.4
    correction = torch.randn(outputs) * 0.2 - 0.5
    r = {"experts": experts, "identity": identity, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}
    margins = []
    ids, w = plain.route(h.double(), router[:outputs].double(), correction.double(), r, torch.float64, margins)
    gate = plain.sigmoid(h.double() @ router[outputs].double())
    routing = G.route(dev(h), dev(router), None, top=top, score="softmax_all", correction=dev(correction), groups=groups, keep=keep, scale=1.7,
                      identity=identity, extra=1)
    assert (routing.extra[:, 0].cpu().double() - gate).abs().max() < 1e-5
    got_ids, got_w, pair_row = routing.ids.cpu(), routing.weights.cpu().double(), routing.pair_row.cpu().view(n, top)
    clear = margins[0] > 1e-4
    assert int(clear.sum()) > n // 2
    for t in range(n):
        if not clear[t]:
            continue
        order = {int(e): j for j, e in enumerate(ids[t])}
        assert sorted(order) == sorted(got_ids[t].tolist()), t
        for j, e in enumerate(got_ids[t].tolist()):
            assert abs(float(got_w[t, j]) - float(w[t, order[e]])) < 1e-5
            assert (int(pair_row[t, j]) < 0) == (e >= experts)
    sorted_token, tile_group = routing.sorted_token.cpu(), routing.tile_group.cpu()
    for t in range(n):
        for j, e in enumerate(got_ids[t].tolist()):
            if e < experts:
                row = int(pair_row[t, j])
                assert int(sorted_token[row]) == t and int(tile_group[row // routing.tile_rows]) == e
    # the weighted sum: rows of experts, the token's own row for an identity output, and the gated extra row
    rows = torch.randn(routing.rows, width)
    extra = torch.randn(n, width)
    out = G.combine_mixed(dev(rows), routing, dev(h), extra=dev(extra), extra_scale=routing.extra).cpu().double()
    want = routing.extra.cpu().double() * extra.double()
    for t in range(n):
        for j, e in enumerate(got_ids[t].tolist()):
            want[t] += got_w[t, j] * (h[t].double() if e >= experts else rows[int(pair_row[t, j])].double())
    assert (out - want).abs().max() < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_squared_relu(dtype):
    from llm_runtime_study_b200.ops import functional as F

    for shape in ((5, 24), (3, 7)):
        x = torch.randn(*shape).to(dtype)
        want = torch.relu(x.double()) ** 2
        assert (F.relu2(dev(x)).cpu().double() - want).abs().max() <= (1e-6 if dtype == torch.float32 else 3e-2)


# ------------------------------------------------------------------------------------------- whole models
LENGTHS = {"A": [1, 2, 5, 23, 64, 65, 131], "B": [3, 17, 48, 70, 1, 129], "C": [140, 2, 37, 66, 300], "D": [200, 33, 40, 1, 90]}


def _requests(name):
    config, seed, _ = helpers.TAFISUN[name]
    rng = random.Random(seed + 1)
    return {f"r{i}": helpers.random_tokens(rng, config["vocab"], n) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B") for d in ("float32", "bfloat16")] + [("C", "bfloat16"), ("C", "float32"), ("D", "bfloat16"), ("D", "float32")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    from llm_runtime_study_b200.engine.runtime import load

    name, dtype = request.param
    config, seed, page = helpers.TAFISUN[name]
    path, weights = helpers.make_tafisun_dir(tmp_path_factory.mktemp(f"tafisun{name}{dtype}"), config, seed, torch_dtype=dtype)
    requests = _requests(name)
    store = plain.round_bfloat16 if dtype == "bfloat16" else plain.keep
    expected, clear = {}, {}
    for rid, tokens in requests.items():
        margins = []
        expected[rid] = plain.forward(weights, config, tokens, store=store, margins=margins)
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
            err = torch.where(clear, err, torch.zeros_like(err))
            assert float(err.max()) <= BF16_WORST, (rid, int(err.argmax()), float(err.max()))
            over = int((err > BF16_USUAL).sum())
            assert over <= max(1, len(tokens) // 10), f"request {rid}: {over} of {len(tokens)} rows beyond {BF16_USUAL}: {err}"
            continue
        bad, err, top = helpers.first_wrong_row(rows, setup["plain"][rid], TOL[setup["dtype"]])
        assert bad is None, f"request {rid}: first wrong position {bad} of {len(tokens)}, rms and largest |diff| / rms {err:.3e}, {top:.3e}"


def test_whole_prompts(setup):
    _compare(setup, _replay(setup, helpers.trace_whole(setup["requests"])))


def test_prefill_then_token_by_token(setup):
    """The tail is longer than most blocks of the masks, so blocks end and begin among decoded tokens and pages behind them
    are given back."""

    _compare(setup, _replay(setup, helpers.trace_decode_tail(setup["requests"], tail=40)))


def test_portions_down_to_two_tokens(setup):
    rng = random.Random(5)
    _compare(setup, _replay(setup, helpers.trace_chunked(setup["requests"], rng, sizes=(2, 3, 2, 7, 13, 16, 17, 31))))


def test_mixed_batches_with_slots_and_pages_used_again(setup):
    """Three slots for the requests, portions beside single tokens, and a pool sized for what is live."""

    rng = random.Random(9)
    steps = helpers.trace_mixed(setup["requests"], rng, live_max=3, tail=6)
    _compare(setup, _replay(setup, steps, max_requests=3))


def test_every_token_decoded_alone(setup):
    """A sequence fed one token a step from its first token: the first tokens, long decoding."""

    requests = {rid: tokens for rid, tokens in setup["requests"].items() if len(tokens) in (23, 131, 70, 66, 90)}
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
    """One slot: the second request takes the first one's state row, previous token and pages."""

    requests = {rid: tokens for rid, tokens in setup["requests"].items() if len(tokens) in (23, 17, 48, 65, 37, 66, 33, 90)}
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
            tokens.append(int(plain.forward(weights, config, tokens)[-1].argmax()))
        want.append(tokens[len(prompt):])
    engine = Engine.from_model_dir(setup["path"], device=DEV, dtype="float32", max_seq_len=64, max_batch_size=2, page_size=setup["page"],
                                   max_tokens_per_step=16, strict_dtype=False)
    assert engine.model.graph_safe()
    got = [[] for _ in prompts]
    for index, event in engine.generate(prompts, max_new_tokens=new, sampling=SamplingConfig(temperature=0.0)):
        if event.token_id is not None:
            got[index].append(event.token_id)
    assert got == want


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

    config = helpers.TAFISUN_B
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
        logits = plain.forward(weights, config, tokens)[-1]
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
        want = plain.forward(weights, config, toks)
        rows = torch.stack([got[rid][p] for p in range(len(toks))]).double()
        bad, rms_err, top_err = helpers.first_wrong_row(rows, want, TOL["float32"])
        assert bad is None, (rid, bad, rms_err, top_err)
