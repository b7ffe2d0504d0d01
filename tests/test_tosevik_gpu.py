"""-m gpu: the Tosevik decoder in the engine against the plain implementation (tests/plain/tosevik.py), in float32 and
bfloat16.  Single kernels on inputs built so that a fault shows: a retention state carried across cuts and slots with
decays between 0.5 and 1, the rotation of part of a head, one loud key far back among hundreds of sigmoid weights, at a
page's border, at the query's own position and one position after it, the distance bias per head, the softmax choice
among groups.  Then whole prompts, prefill against token-by-token decoding, portions down to two tokens, batches of
unequal requests against each alone, pages and state slots used again, long decoding, and greedy generation through the
engine's own entry point and scheduler."""
import math

import numpy as np
import pytest
import torch

from tests import tosevik_helpers as S
from tests.gpu_harness import DEV, i32
from tests.plain import tosevik as plain

pytestmark = pytest.mark.gpu
DTYPES = ("float32", "bfloat16")
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KERNEL_BAR = {"float32": 2e-5, "bfloat16": 2e-2}          # of the largest value
F64 = torch.float64


def kernel_close(got, want, dtype, what, bar=None):
    got, want = np.asarray(got.detach().float().cpu(), np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert np.isfinite(got).all() and err <= (bar or KERNEL_BAR[dtype]), \
        f"{what}: {dtype} worst error {err:.3e} of the largest value"


def rnd(g, *shape, dtype="float32", scale=1.0):
    """random values that the storage dtype holds exactly, as float64"""
    return (torch.randn(*shape, generator=g) * scale).to(TD[dtype]).double()


# ------------------------------------------------------------------------------------------------ retention
def plain_recurrence(q, k, v, decay):
    """q, k (T, H, dim), v (T, H, vdim) float64 -> o (T, H, vdim), the final state (H, dim, vdim)"""
    T, H, dim = q.shape
    S_ = torch.zeros(H, dim, v.shape[-1], dtype=F64)
    o = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        for a in range(H):
            S_[a] = decay[a] * S_[a] + torch.outer(k[t, a], v[t, a])
            o[t, a] = S_[a].T @ q[t, a]
    return o, S_


@pytest.mark.parametrize("H,dim,vdim,decay", [(3, 16, 24, (0.5, 0.9, 1.0)), (2, 40, 20, (0.97, 0.999)), (1, 8, 72, (0.75,)),
                                              (2, 64, 32, (1.0, 0.99)), (1, 128, 40, (0.995,)), (2, 10, 6, (0.8, 0.95)),
                                              (1, 200, 12, (0.9,))])
def test_retention_carries_its_state_across_any_cut(H, dim, vdim, decay):
    """Three sequences advance side by side in portions of their own sizes (1 and 2 tokens among them, and stretches
    long enough for the split form, whose segments the cuts do not respect), in state slots that are not in order; the
    state lies inside a wider tensor, for an even number of heads off the 16-byte boundaries.  The scan and the split form
    with segments of several sizes (most portions one segment, most portions many), against the plain loop."""
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(dim)
    T = 150
    seqs = []
    for _ in range(3):
        q, k, v = rnd(g, T, H, dim), rnd(g, T, H, dim) * dim ** -0.5, rnd(g, T, H, vdim)
        seqs.append((q, k, v) + plain_recurrence(q, k, v, decay))
    dec = torch.tensor(decay, dtype=torch.float32, device=DEV)
    cuts = [[1, 1, 2, 33, 9, 70, 3, 31], [2, 97, 1, 7, 43], [65, 17, 1, 2, 64, 1]]
    for chunked, segment in ((False, None), (True, None), (True, 16), (True, 7), (True, 1)):
        pad, n = 40 + (H % 2 == 0), H * dim * vdim
        state = torch.zeros(5, pad + n + 8, device=DEV)
        slots = [3, 0, 4]
        at, got = [0, 0, 0], [[], [], []]
        for step in range(max(len(c) for c in cuts)):
            live = [s for s in range(3) if step < len(cuts[s])]
            lens = [cuts[s][step] for s in live]
            cat = lambda j, w: torch.cat([seqs[s][j][at[s]:at[s] + n_] for s, n_ in zip(live, lens)]) \
                .reshape(sum(lens), w).float().to(DEV).contiguous()
            q, k, v = cat(0, H * dim), cat(1, H * dim), cat(2, H * vdim)
            o = torch.full((sum(lens), H * vdim), float("nan"), device=DEV)
            q_start = np.concatenate([[0], np.cumsum(lens)[:-1]])
            ops.retention(q, k, v, dec, o, state[:, pad:pad + n], (i32(q_start), i32(lens), i32([slots[s] for s in live])),
                          H, dim, vdim, chunked=chunked, segment=segment)
            at_o = 0
            for s, n_ in zip(live, lens):
                got[s].append(o[at_o:at_o + n_].cpu())
                at_o += n_
                at[s] += n_
        assert at == [T, T, T]
        for s in range(3):
            kernel_close(torch.cat(got[s]).reshape(T, H, vdim), seqs[s][3], "float32",
                         f"retention ({f'segments of {segment}' if chunked else 'scan'}), sequence {s}", 1e-5)
            kept = state[slots[s], pad:pad + n].view(H, vdim, dim).transpose(1, 2)      # a head's state is stored (vdim, dim)
            kernel_close(kept, seqs[s][4], "float32", f"the state sequence {s} leaves", 1e-5)
        assert float(state[:, :pad].abs().max()) == 0.0 and float(state[:, pad + n:].abs().max()) == 0.0
        assert float(state[1].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0       # slots nobody has


def test_retention_keeps_a_far_token_only_as_its_decay_allows():
    """one loud key 600 tokens back: with decay 1 it counts in full, with decay 0.99 as 0.99^600, with 0.5 not at all"""
    from mashbox_b200 import ops
    H, dim, vdim, T = 3, 16, 8, 640
    decay = (1.0, 0.99, 0.5)
    q, k, v = torch.zeros(T, H, dim, dtype=F64), torch.zeros(T, H, dim, dtype=F64), torch.zeros(T, H, vdim, dtype=F64)
    k[20, :, 3], v[20, :, 5] = 2.0, 3.0
    q[620, :, 3] = 1.0
    for chunked, segment in ((False, None), (True, None), (True, 100), (True, 256)):
        state = torch.zeros(1, H * dim * vdim, device=DEV)
        o = torch.empty(T, H * vdim, device=DEV)
        dev = lambda x: x.reshape(T, -1).float().to(DEV).contiguous()
        ops.retention(dev(q), dev(k), dev(v), torch.tensor(decay, device=DEV), o, state, (i32([0]), i32([T]), i32([0])), H, dim,
                      vdim, chunked=chunked, segment=segment)
        o = o.view(T, H, vdim).cpu().double()
        want = torch.tensor([6.0 * d ** 600 for d in decay], dtype=F64)
        assert torch.allclose(o[620, :, 5], want, rtol=1e-4, atol=1e-30), (chunked, o[620, :, 5])
        assert float(o[619].abs().max()) == 0.0 and float(o[620, :, :5].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dim,vdim,R,base", [(3, 16, 24, 8, 100.0), (2, 24, 16, 24, 5000.0), (2, 8, 40, 0, 1.0),
                                               (1, 10, 6, 6, 300.0)])
def test_retention_rotation_and_key_scale(dtype, H, dim, vdim, R, base):
    """q, k, v from one product's rows (with other columns between and after them), positions far apart: the first R dims
    of every head turn in halves, the rest pass, k is scaled after the rotation, v passes"""
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(R + dim)
    N = 9
    pos = torch.tensor([0, 1, 2, 7, 63, 64, 999, 5000, 20000])
    extra = 5
    C = 2 * H * dim + extra + H * vdim + 3
    rows = rnd(g, N, C, dtype=dtype)
    q_off, k_off, v_off = 0, H * dim, 2 * H * dim + extra
    freqs = None
    if R:
        freqs = (base ** (-2.0 * torch.arange(R // 2, dtype=F64) / R)).float().to(DEV)
    q, k = torch.empty(N, H * dim, device=DEV), torch.empty(N, H * dim, device=DEV)
    v = torch.empty(N, H * vdim, device=DEV)
    ops.retention_prep(rows.to(DEV, TD[dtype]).contiguous(), q_off, k_off, v_off, i32(pos), freqs, q, k, v, H, dim, vdim, R,
                       dim ** -0.5)
    rot = dict(dims=R, base=base) if R else None
    wq = plain.rotate(rows[:, q_off:q_off + H * dim].view(N, H, dim), pos, rot)
    wk = plain.rotate(rows[:, k_off:k_off + H * dim].view(N, H, dim), pos, rot) * dim ** -0.5
    # float32 angles: position 20000 times a frequency is exact to about 1e-3 radians
    kernel_close(q.view(N, H, dim), wq, "float32", "rotated q", 2e-3)
    kernel_close(k.view(N, H, dim), wk, "float32", "rotated, scaled k", 2e-3)
    kernel_close(q.view(N, H, dim)[:5], wq[:5], "float32", "rotated q at near positions", 1e-5)
    kernel_close(v, rows[:, v_off:v_off + H * vdim], "float32", "v", 1e-7)


@pytest.mark.parametrize("dtype", DTYPES)
def test_unit_rms_heads_times_silu_gate(dtype):
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(1)
    N, H, vdim, eps = 7, 3, 20, 1e-3
    o = rnd(g, N, H, vdim, scale=0.05)                      # small values: eps matters, and it lies inside the root
    wide = rnd(g, N, 11 + H * vdim, dtype=dtype)
    gate = wide[:, 11:]
    out = torch.empty(N, H * vdim, device=DEV, dtype=TD[dtype])
    ops.gated_rms(o.reshape(N, -1).float().to(DEV), wide.to(DEV, TD[dtype])[:, 11:], None, out, H, vdim, eps, silu=True)
    want = plain.rms(o, eps).reshape(N, -1) * plain.silu(gate)
    kernel_close(out, want, dtype, "o / rms(o) * silu(gate)")
    off = o.reshape(N, -1) / torch.sqrt((o * o).mean(-1, keepdim=True)).expand(N, H, vdim).reshape(N, -1) * plain.silu(gate)
    assert float((want - off).abs().max() / want.abs().max()) > 0.05           # eps inside the root is seen


# ------------------------------------------------------------------------------------------------ the stream
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [64, 100, 257, 2052])
def test_dynamic_tanh_and_depth_average(dtype, D):
    """widths that take the four-wide kernels (one piece of a row, and two with a ragged end) and one that does not"""
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(D)
    N, L = 6, 4
    w, b, alpha = rnd(g, D), rnd(g, D, scale=0.3), 0.7
    wd, bd = w.float().to(DEV), b.float().to(DEV)
    x0 = rnd(g, N, D, scale=2.0)
    x = x0.float().to(DEV).clone()
    out = torch.empty(N, D, device=DEV, dtype=TD[dtype])
    ops.dyt(x, None, alpha, wd, bd, out)
    kernel_close(out, torch.tanh(alpha * x0) * w + b, dtype, "dynamic tanh")
    assert torch.equal(x.cpu().double(), x0)
    d1, d2 = rnd(g, N, D, dtype=dtype), rnd(g, N, D, dtype=dtype)
    ops.dyt(x, d1.to(DEV, TD[dtype]), alpha, wd, bd, out, delta2=d2.to(DEV, TD[dtype]))
    kernel_close(x, x0 + d1 + d2, "float32", "the stream after two deltas", 1e-6)
    kernel_close(out, torch.tanh(alpha * (x0 + d1 + d2)) * w + b, dtype, "dynamic tanh of the sum")
    # the depth average: the history of L + 1 streams, every layer's own coefficients
    hist = torch.zeros(L + 1, N + 3, D, device=DEV)
    X = [rnd(g, N, D)]
    hist[0, :N] = X[0].float().to(DEV)
    x = X[0].float().to(DEV).clone()
    for i in range(L):
        coef = rnd(g, i + 2, scale=0.7)
        delta = rnd(g, N, D, dtype=dtype)
        handed = x.cpu().double()
        X.append(handed + delta)
        normed = torch.empty(N, D, device=DEV, dtype=TD[dtype])
        ops.depth_average(x, delta.to(DEV, TD[dtype]), hist, coef.float().to(DEV), i, normed=normed, next_norm=(alpha, wd, bd))
        want = sum(coef[j] * X[j] for j in range(i + 2))
        kernel_close(x, want, "float32", f"depth average after layer {i}", 1e-5)
        kernel_close(hist[i + 1, :N], X[i + 1], "float32", f"history slot {i + 1}", 1e-6)
        kernel_close(normed, torch.tanh(alpha * want) * w + b, dtype, "the next norm")
    assert float(hist[:, N:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [64, 100, 2056, 8192, 8200])
def test_two_normed_outputs_halved(dtype, D):
    """widths of one 16-byte piece a thread, of none for most threads, of four (the widest row the bf16 kernel keeps in
    registers), and beyond it"""
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(D)
    N, eps = 5, 1e-2
    a, b = rnd(g, N, D, dtype=dtype, scale=0.1), rnd(g, N, D, dtype=dtype, scale=3.0)
    wa, wb = rnd(g, D), rnd(g, D)
    out = torch.empty(N, D, device=DEV, dtype=TD[dtype])
    ops.rms_pair_mean(a.to(DEV, TD[dtype]), b.to(DEV, TD[dtype]), wa.float().to(DEV), wb.float().to(DEV), out, eps)
    kernel_close(out, 0.5 * (plain.rms(a, eps, wa) + plain.rms(b, eps, wb)), dtype, "half the sum of two normed outputs")


# ------------------------------------------------------------------------------------------------ the routed feed-forward
@pytest.mark.parametrize("E,top,groups,keep,scale", [(12, 3, 3, 2, 1.7), (8, 2, 1, 1, 1.0), (6, 1, 6, 2, 1.0), (16, 2, 2, 1, 2.5),
                                                     (64, 6, 8, 3, 0.5), (5, 3, 1, 1, 2.0), (4, 4, 2, 2, 1.0)])
def test_softmax_choice_among_groups(E, top, groups, keep, scale):
    """scores are a softmax over ALL experts (also those of groups that are not kept), a group is worth its best expert,
    the weights are the chosen scores times a constant and are not renormalised; a column beside the experts' (the
    shared expert's gate rides in the same product) is no expert"""
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(E)
    N = 60
    z = rnd(g, N, E + 1, scale=1.5)
    s = torch.softmax(z[:, :E], -1)
    chosen = plain.choose(s, top, groups, keep)
    ids = torch.empty(N, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(N, top, device=DEV)
    ops.moe_select(z.float().to(DEV), None, ids, wts, groups, keep, experts=E, softmax=True, worth="max", scale=scale)
    ids, wts = ids.cpu().long(), wts.cpu().double()
    assert torch.equal(ids.sort(-1).values, chosen.sort(-1).values)
    assert torch.allclose(wts, scale * s.gather(1, ids), rtol=1e-5, atol=1e-7)
    if top < E and groups == 1:
        assert float(wts.sum(-1).max()) < scale                # not renormalised: the chosen scores do not add up to 1


@pytest.mark.parametrize("dtype", DTYPES)
def test_experts_sum_with_a_gated_shared_expert(dtype):
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(2)
    N, top, D = 9, 3, 40
    y, wts = rnd(g, N, top, D), rnd(g, N, top).abs()
    shared = rnd(g, N, D, dtype=dtype)
    z = rnd(g, N, 7)                                         # the gate's logit is the last column of a wider product
    out = torch.empty(N, D, device=DEV, dtype=TD[dtype])
    ops.moe_combine(y.float().to(DEV), wts.float().to(DEV), out, shared.to(DEV, TD[dtype]), z.float().to(DEV)[:, 6:])
    want = (wts[:, :, None] * y).sum(1) + torch.sigmoid(z[:, 6:]) * shared
    kernel_close(out, want, dtype, "experts' sum + sigmoid(gate) * shared")


# ------------------------------------------------------------------------------------------------ attention with sigmoid weights
def sigmoid_case(dtype, H, G, dim, vdim, lengths, q_lens, page, loud, kernel, temp=None, seed=0, pb=-4.0, scale=None):
    """Sequences whose keys and values the prep kernel writes into shuffled pages (a step of whole prompts), then a step
    whose queries are each sequence's last q_lens tokens, attended by `kernel` ("plain", "mma", or "tc5": the prompt
    form on tcgen05).  loud: (sequence, key
    position, query position): the query's row points along that key's row (all heads), so that the one score stands
    out wherever the query may see the key.  -> the kernel's output rows and the plain answer"""
    from mashbox_b200 import ops
    from mashbox_b200.parts.diff_attention import plan_diff_attention
    from mashbox_b200.parts.sigmoid_attention import geometric_slopes
    g = torch.Generator().manual_seed(seed)
    eps = 1e-5
    scale = scale if scale is not None else 4.0 / dim
    C = H * dim + G * dim + G * vdim
    nq, nk = 1.5 + torch.rand(H * dim, generator=g, dtype=F64), 0.75 + 0.5 * torch.rand(G * dim, generator=g, dtype=F64)
    bias = pb + rnd(g, H)
    eye = torch.eye(C, dtype=F64)
    W = {"a.q": eye[:H * dim], "a.k": eye[H * dim:H * dim + G * dim], "a.v": eye[H * dim + G * dim:],
         "a.o": torch.eye(H * vdim, dtype=F64), "a.q.norm": nq, "a.k.norm": nk, "a.pb": bias}
    m = dict(heads=H, kv_heads=G, dim=dim, vdim=vdim, scale=scale, q_temp=dict(coef=temp[0], every=temp[1]) if temp else None)
    rows = [rnd(g, n, C, dtype=dtype) for n in lengths]
    for s, kp, qp in loud:
        k = rows[s][kp, H * dim:H * dim + G * dim].view(G, dim)
        rows[s][qp, :H * dim] = (k.repeat_interleave(H // G, 0) / nk.view(G, dim).repeat_interleave(H // G, 0)).reshape(-1) \
            .to(TD[dtype]).double()
    want = torch.cat([plain.sigmoid_attention(W, "a.", m, rows[s], eps)[n - ql:] for s, (n, ql) in enumerate(zip(lengths, q_lens))])
    # pages in a shuffled order, a table row per sequence (not in order either)
    S_ = len(lengths)
    blocks = [-(-n // page) for n in lengths]
    num_pages = sum(blocks) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    seq_rows = list(range(S_))[::-1]
    table = np.full((S_, max(blocks) + 1), -1, np.int32)
    at = 0
    for s in range(S_):
        table[seq_rows[s], :blocks[s]] = perm[at:at + blocks[s]]
        at += blocks[s]
    table = i32(table)
    kpool = torch.full((num_pages, G, page, dim), float("nan") if dtype == "float32" else 0.0, device=DEV, dtype=TD[dtype])
    vpool = torch.full((num_pages, G, page, vdim), float("nan") if dtype == "float32" else 0.0, device=DEV, dtype=TD[dtype])
    err = ops.new_error_word(DEV)
    all_rows = torch.cat(rows).to(DEV, TD[dtype]).contiguous()
    positions = i32(np.concatenate([np.arange(n) for n in lengths]))
    tok_row = i32(np.repeat(seq_rows, lengths))
    q_all = torch.empty(sum(lengths), H * dim, device=DEV, dtype=TD[dtype])
    tc, te = (temp[0], temp[1]) if temp else (0.0, 0)
    ops.sigmoid_attention_prep(all_rows, nq.float().to(DEV), nk.float().to(DEV), positions, tok_row, table, q_all, kpool, vpool,
                               H, G, dim, vdim, page, num_pages, eps, tc, te, err)
    starts = np.concatenate([[0], np.cumsum(lengths)[:-1]])
    pick = np.concatenate([np.arange(st + n - ql, st + n) for st, n, ql in zip(starts, lengths, q_lens)])
    q = q_all[torch.as_tensor(pick, device=DEV)].contiguous()
    N = len(pick)
    o = torch.full((N, H * vdim), float("nan"), device=DEV, dtype=TD[dtype])
    slopes = torch.tensor(geometric_slopes(H, 8.0), dtype=torch.float32, device=DEV)
    pbd = bias.float().to(DEV)
    pos_q, row_q = positions[torch.as_tensor(pick, device=DEV)].contiguous(), tok_row[torch.as_tensor(pick, device=DEV)].contiguous()
    if kernel == "plain":
        ops.sigmoid_attention_simple(q, o, pos_q, row_q, table, kpool, vpool, slopes, pbd, H, G, dim, vdim, page, num_pages,
                                     scale, err)
    else:
        pos0 = [n - ql for n, ql in zip(lengths, q_lens)]
        tc5 = kernel == "tc5"
        plan = plan_diff_attention(q_lens, pos0, H // G, G, None, ops.sigmoid_attention_tc5_rows() if tc5 else ops.SIGMOID_MMA_ROWS,
                                   ops.SIGMOID_DECODE_ROWS, ops.SIGMOID_MAX_SPLITS, 296,
                                   kernel[1] if isinstance(kernel, tuple) else None, quads=tc5)
        q_start = i32(np.concatenate([[0], np.cumsum(q_lens)[:-1]]))
        seqs = (q_start, i32(q_lens), i32(pos0), i32(seq_rows))
        tail = (table, kpool, vpool, slopes, pbd, H, G, dim, vdim, page, num_pages, scale, err)
        if plan["pre"] and tc5:
            ops.sigmoid_attention_tc5(q, o, i32(plan["pre"]), len(plan["pre"]) // 4, *seqs, *tail)
        elif plan["pre"]:
            ops.sigmoid_attention_mma(q, o, i32(plan["pre"]), len(plan["pre"]) // 2, *seqs, *tail)
        if plan["dec"]:
            n_slots = len(plan["slots"]) // 2
            part_o = torch.empty(max(1, n_slots) * G * ops.SIGMOID_MAX_SPLITS * ops.SIGMOID_DECODE_ROWS, vdim, device=DEV)
            ops.sigmoid_attention_mma_decode(q, o, i32(plan["dec"]), len(plan["dec"]) // 4, i32(plan["slots"] or [0, 0]),
                                             n_slots, part_o, *seqs, *tail)
    assert int(err.item()) == 0
    return o, want


SIG_SHAPES = [("plain", 4, 2, 16, 24, 8), ("plain", 3, 1, 12, 20, 5), ("plain", 2, 2, 40, 8, 16),
              ("mma", 4, 2, 16, 32, 8), ("mma", 8, 2, 64, 64, 16), ("mma", 2, 1, 128, 32, 64), ("mma", 3, 3, 32, 128, 5),
              ("mma", 32, 1, 16, 16, 16), ("tc5", 8, 2, 64, 64, 16), ("tc5", 4, 1, 128, 128, 32), ("tc5", 3, 3, 64, 64, 8),
              ("tc5", 12, 2, 128, 128, 128)]


@pytest.mark.parametrize("kernel,H,G,dim,vdim,page", SIG_SHAPES)
def test_sigmoid_weights_far_away_at_page_borders_and_after_the_query(kernel, H, G, dim, vdim, page):
    """one loud key far back among hundreds (every key counts by itself: nothing normalises); at the last slot of a
    page and the first of the next; at the query's own position; and one position AFTER the query, which the query
    must not see; in a prompt's portion and decoded alone; the distance bias of every head"""
    n = 700
    dtypes = DTYPES if kernel == "plain" else ("bfloat16",)
    for dtype in dtypes:
        bar = 4e-2 if dtype == "bfloat16" else 2e-5
        for q_lens, loud in (([1, 1, 1], [(0, 3, n - 1), (1, page * 5 - 1, n - 1), (2, page * 5, n - 1)]),
                             ([300, 40, 2], [(0, 2, n - 7), (0, n - 100, n - 100), (0, n - 49, n - 50), (1, n - 17, n - 17),
                                             (1, page * 3, n - 3), (2, n - 1, n - 2), (2, 0, n - 1)])):
            got, want = sigmoid_case(dtype, H, G, dim, vdim, [n, n, n], q_lens, page, loud, kernel, temp=(0.4, 7), seed=dim)
            kernel_close(got, want, dtype, f"sigmoid attention ({kernel}), query stretches {q_lens}", bar)
        # unequal sequences, one of a single token (its own key is all it sees), one that ends at a page's last slot
        got, want = sigmoid_case(dtype, H, G, dim, vdim, [1, page * 4, 333, 64, 65], [1, 3, 70, 1, 65], page,
                                 [(2, 0, 332), (4, 63, 64)], kernel, seed=dim + 1)
        kernel_close(got, want, dtype, f"sigmoid attention ({kernel}), unequal sequences", bar)
    # the cases test something: a loud key one position after the query must not move the answer, one at it must
    dtype = dtypes[0]
    got, want = sigmoid_case(dtype, H, G, dim, vdim, [60], [2], page, [(0, 59, 58)], kernel, seed=1)
    kernel_close(got, want, dtype, "a key one position after the query", 4e-2 if dtype == "bfloat16" else 2e-5)
    quiet = sigmoid_case(dtype, H, G, dim, vdim, [60], [2], page, [], kernel, seed=1)[1]
    seen = sigmoid_case(dtype, H, G, dim, vdim, [60], [2], page, [(0, 58, 58)], kernel, seed=1)[1]
    assert float((seen[0] - quiet[0]).abs().max()) > 0.1 * float(quiet[0].abs().max())


def test_sigmoid_weights_are_not_normalised_and_fall_with_distance():
    """scale 0: the weight of key j is sigmoid(pb_h - slope_h (i - j)) whatever q and k hold, so the output is that sum
    of unit-rms values head by head, computed here by hand; nothing divides by the sum of the weights"""
    from mashbox_b200.parts.sigmoid_attention import geometric_slopes
    H, G, dim, vdim, page, n = 4, 1, 16, 16, 8, 128
    slopes = geometric_slopes(H, 8.0)
    assert abs(slopes[-1] - 2.0 ** -8) < 1e-12 and abs(slopes[0] - 2.0 ** -2) < 1e-12
    for kernel, dtype in (("plain", "float32"), ("mma", "bfloat16")):
        got, want = sigmoid_case(dtype, H, G, dim, vdim, [n], [1], page, [], kernel, seed=3, pb=1.0, scale=0.0)
        kernel_close(got, want, dtype, f"scale 0 ({kernel})", 2e-2 if dtype == "bfloat16" else 2e-5)
        # the same random stream as sigmoid_case: norm weights, biases, then the rows
        g = torch.Generator().manual_seed(3)
        torch.rand(H * dim, generator=g, dtype=F64), torch.rand(G * dim, generator=g, dtype=F64)
        bias = 1.0 + rnd(g, H)
        rows = rnd(g, n, H * dim + G * dim + G * vdim, dtype=dtype)
        v = plain.rms(rows[:, H * dim + G * dim:], 1e-5)
        dist = torch.arange(n - 1, -1, -1, dtype=F64)
        by_hand = torch.stack([(torch.sigmoid(bias[a] - slopes[a] * dist)[:, None] * v).sum(0) for a in range(H)])
        kernel_close(got.view(H, vdim), by_hand, dtype, f"the sum of the weights by hand ({kernel})", 2e-2 if dtype == "bfloat16" else 2e-5)
        total = torch.stack([torch.sigmoid(bias[a] - slopes[a] * dist).sum() for a in range(H)])
        assert float(total[-1]) > 30.0 and float(total[0]) < 8.0          # far keys count on the flat head, not on the steep one


@pytest.mark.parametrize("splits", [1, 2, 4, 16])
def test_sigmoid_decode_form_cut_along_the_keys(splits):
    """the decode form with its keys cut into splits that run side by side: the same answer for every number of splits"""
    H, G, dim, vdim, page = 8, 2, 64, 64, 16
    lengths, q_lens = [1500, 129, 64, 3], [1, 2, 4, 1]
    got, want = sigmoid_case("bfloat16", H, G, dim, vdim, lengths, q_lens, page, [(0, 5, 1499), (1, 63, 128)], ("mma", splits),
                             temp=(0.3, 50), seed=splits)
    kernel_close(got, want, "bfloat16", f"decode form, {splits} splits", 4e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_query_temperature_and_whole_row_norms(dtype):
    """the prep kernel alone: q and k normed over ALL heads at once (a loud head quiets the others), every head of v by
    itself, and the temperature's first move at position every - 1"""
    from mashbox_b200 import ops
    g = torch.Generator().manual_seed(4)
    H, G, dim, vdim, page, eps = 3, 1, 8, 12, 4, 1e-5
    C = H * dim + G * dim + G * vdim
    N = 12
    rows = rnd(g, N, C, dtype=dtype)
    rows[:, :dim] *= 8.0                                        # head 0 of q is loud
    nq, nk = rnd(g, H * dim), rnd(g, G * dim)
    table = i32(np.array([[2, 0, 1, -1]], np.int32))
    kpool = torch.zeros(3, G, page, dim, device=DEV, dtype=TD[dtype])
    vpool = torch.zeros(3, G, page, vdim, device=DEV, dtype=TD[dtype])
    q = torch.empty(N, H * dim, device=DEV, dtype=TD[dtype])
    err = ops.new_error_word(DEV)
    every, coef = 5, 0.6
    ops.sigmoid_attention_prep(rows.to(DEV, TD[dtype]).contiguous(), nq.float().to(DEV), nk.float().to(DEV), i32(np.arange(N)),
                               i32(np.zeros(N)), table, q, kpool, vpool, H, G, dim, vdim, page, 3, eps, coef, every, err)
    assert int(err.item()) == 0
    pos = torch.arange(N, dtype=F64)
    temp = 1.0 + coef * torch.log(torch.floor((pos + 1) / every) + 1.0)
    assert float(temp[every - 2]) == 1.0 and float(temp[every - 1]) > 1.4
    kernel_close(q, plain.rms(rows[:, :H * dim], eps, nq) * temp[:, None], dtype, "q: whole-row norm, weight, temperature")
    kp = torch.cat([kpool[p] for p in (2, 0, 1)], 1).transpose(0, 1).reshape(N, G * dim)
    vp = torch.cat([vpool[p] for p in (2, 0, 1)], 1).transpose(0, 1).reshape(N, G, vdim)
    kernel_close(kp, plain.rms(rows[:, H * dim:H * dim + G * dim], eps, nk), dtype, "cached k: whole-row norm")
    kernel_close(vp, plain.rms(rows[:, H * dim + G * dim:].view(N, G, vdim), eps), dtype, "cached v: unit rms per head")


# ------------------------------------------------------------------------------------------------ the model in the engine
def runner_for(tmp, name, dtype, max_tokens, options=None, max_requests=4):
    from mashbox_b200.engine.replay import make_runner
    folder = S.make_folder(tmp, name, "float32" if dtype == "float32" else "bfloat16")
    return folder, make_runner(folder, dtype, max_tokens, page_size=S.CONFIGS[name][2], options=options,
                               max_requests=max_requests)


def replay(runner, steps):
    from mashbox_b200.engine.replay import run_step
    out = {}
    for i, s in enumerate(steps):
        r = run_step(runner, dict(s, step=i))
        if r is not None:
            out[i] = r.numpy()
    return out


def cut_steps(rid, tokens, cuts, end=True):
    """the steps that feed `tokens` in portions of the given sizes, asking for every position's logits"""
    steps, at = [], 0
    for n in cuts:
        steps.append(dict(entries=[dict(id=rid, tokens=tokens[at:at + n], want=list(range(n)))], end=[]))
        at += n
    assert at == len(tokens)
    if end:
        steps[-1]["end"] = [rid]
    return steps


CASES = [(n, d) for n in S.CONFIGS for d in DTYPES]


def test_every_layers_result_in_the_history(tmp_path_factory):
    """float32: the embedding's output and every layer's own result, which the runner keeps for the depth averages,
    against the plain implementation's"""
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), "T", "float32", 128)
    (p,) = S.prompts_for("T", (45,))
    cfg, W = S._model(folder)
    _, results = plain.forward(cfg, W, p, keep_results=True)
    replay(runner, cut_steps("a", p, [len(p)]))
    (key,) = [k for k in runner.ws.buffers if k[0] == "depth_history"]
    hist = runner.ws.buffers[key]
    assert hist.shape[0] >= len(cfg["layers"]) + 1
    for j in range(len(cfg["layers"]) + 1):
        kernel_close(hist[j, :len(p)], results[j], "float32", f"result {j} of the history", 2e-5)


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_and_first_tokens(tmp_path_factory, name, dtype):
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 320)
    for p in S.prompts_for(name, (1, 2, 3, 5, 21, 64, 65, 150, 300)):
        got = replay(runner, cut_steps("a", p, [len(p)]))[0]
        S.assert_close(got, S.plain_logits(folder, p), dtype, f"{name}: whole prompt of {len(p)}")
    runner.cache.check()
    assert runner.cache.free_pages() == [runner.cache.num_pages] * len(runner.cache.groups)


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_against_token_by_token(tmp_path_factory, name, dtype):
    """every token alone from the first one, over many pages, against the whole prompt in one step and against the
    plain implementation; a second request in the same state slot and pages right after starts from nothing"""
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 192, max_requests=1)
    p, p2 = S.prompts_for(name, (170, 30), seed=1)
    whole = replay(runner, cut_steps("a", p, [len(p)]))[0]
    out = replay(runner, cut_steps("b", p, [1] * len(p)))
    single = np.concatenate([out[i] for i in range(len(p))])
    S.assert_close(single, S.plain_logits(folder, p), dtype, f"{name}: 170 tokens one by one")
    S.assert_close(single, whole, dtype, f"{name}: one by one against one step", S.BAR_SAME)
    again = replay(runner, cut_steps("c", p2, [len(p2)]))[0]
    S.assert_close(again, S.plain_logits(folder, p2), dtype, f"{name}: a request in a slot that was used before")
    runner.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_every_size(tmp_path_factory, name, dtype):
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 256)
    (p,) = S.prompts_for(name, (230,), seed=2)
    want = S.plain_logits(folder, p)
    whole = replay(runner, cut_steps("w", p, [len(p)]))[0]
    for cuts in ([2] * 115, [3, 37, 1, 2, 64, 17, 2, 2, 1, 50, 33, 5, 7, 6], [7, 8, 9, 1, 15, 16, 17, 157],
                 [63, 1, 1, 63, 2, 62, 38], [128, 2, 100]):
        out = replay(runner, cut_steps("a", p, cuts))
        got = np.concatenate([out[i] for i in range(len(cuts))])
        S.assert_close(got, want, dtype, f"{name}: portions {cuts[:6]}...")
        S.assert_close(got, whole, dtype, f"{name}: portions {cuts[:6]}... against one step", S.BAR_SAME)
    runner.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_requests_side_by_side_with_pages_and_slots_used_again(tmp_path_factory, name, dtype):
    """Two requests at most are live, portions of some beside single tokens of others; the pool holds less than all
    requests together, and two state slots only, so pages and slots come back and are taken again.  Every request's
    logits must be those it has alone."""
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 224, max_requests=2)
    prompts = dict(zip("abcdef", S.prompts_for(name, (90, 47, 3, 110, 66, 21), seed=3)))
    plans = dict(a=[30, 1, 1, 2, 50, 1, 1, 1, 1, 1, 1], b=[1, 1, 20, 2, 23], c=[1, 2], d=[64, 1, 40, 2, 1, 1, 1],
                 e=[2, 62, 1, 1], f=[21])
    order = ["a", "b", "c", "d", "e", "f"]
    at = {r: 0 for r in order}
    turn = {r: 0 for r in order}
    got = {r: [] for r in order}
    waiting, live, step = list(order), [], 0
    from mashbox_b200.engine.replay import run_step
    while waiting or live:
        while waiting and len(live) < 2:
            live.append(waiting.pop(0))
        entries, end = [], []
        for r in live:
            n = plans[r][turn[r]]
            entries.append(dict(id=r, tokens=prompts[r][at[r]:at[r] + n], want=list(range(n))))
            at[r] += n
            turn[r] += 1
            if turn[r] == len(plans[r]):
                assert at[r] == len(prompts[r])
                end.append(r)
        out = run_step(runner, dict(step=step, entries=entries, end=end)).numpy()
        o = 0
        for e in entries:
            got[e["id"]].append(out[o:o + len(e["tokens"])])
            o += len(e["tokens"])
        live = [r for r in live if r not in end]
        runner.cache.check()
        step += 1
    for r in order:
        S.assert_close(np.concatenate(got[r]), S.plain_logits(folder, prompts[r]), dtype, f"{name}: request {r} in a batch")
    assert runner.cache.free_pages() == [runner.cache.num_pages] * len(runner.cache.groups)


@pytest.mark.parametrize("name,dtype,options", [("V", "bfloat16", dict(plain_attention=True)),
                                                ("V", "bfloat16", dict(retention_scan_only=True)),
                                                ("V", "bfloat16", dict(attention_splits=4)),
                                                ("V", "bfloat16", dict(attention_prefill_kernel="mma")),
                                                ("V", "bfloat16", dict(plain_experts=True)),
                                                ("T", "float32", dict(retention_scan_only=True))])
def test_every_kernel_form_gives_the_same_model(tmp_path_factory, name, dtype, options):
    """the forms the engine chooses between by the step's size, forced: the plain attention kernel beside the
    tensor-core one, the token-by-token recurrence beside the split form, decode keys cut four ways, prompt tiles on
    mma.sync where heads of 64 x 64 would take tcgen05, experts pair by pair"""
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 512, options=options)
    (p,) = S.prompts_for(name, (300,), seed=7)
    want = S.plain_logits(folder, p)
    out = replay(runner, cut_steps("a", p, [200, 70] + [1] * 30))
    got = np.concatenate([out[i] for i in range(32)])
    S.assert_close(got, want, dtype, f"{name} with {options}")


@pytest.mark.parametrize("name,dtype", [("T", "float32"), ("T", "bfloat16"), ("V", "bfloat16"), ("W", "float32"),
                                        ("Z", "bfloat16")])
def test_long_decoding(tmp_path_factory, name, dtype):
    """a short prompt and 368 tokens one by one (graphs replayed), two requests side by side"""
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 896)
    a, b = S.prompts_for(name, (412, 380), seed=4)
    steps = [dict(entries=[dict(id="a", tokens=a[:12], want=[11])], end=[]),
             dict(entries=[dict(id="a", tokens=a[12:44], want=[31]), dict(id="b", tokens=b[:3], want=[2])], end=[])]
    for i in range(400 - 32):
        e = [dict(id="a", tokens=[a[44 + i]], want=[0])]
        if 3 + i < len(b):
            e.append(dict(id="b", tokens=[b[3 + i]], want=[0]))
        steps.append(dict(entries=e, end=[]))
    out = replay(runner, steps)
    wa, wb = S.plain_logits(folder, a), S.plain_logits(folder, b)
    ga = np.stack([out[0][0], out[1][0]] + [out[2 + i][0] for i in range(368)])
    gb = np.stack([out[1][1]] + [out[2 + i][1] for i in range(368)])
    S.assert_close(ga, wa[[11, 43] + list(range(44, 412))], dtype, f"{name}: 368 tokens decoded, request a")
    S.assert_close(gb, wb[[2] + list(range(3, 371))], dtype, f"{name}: 368 tokens decoded, request b")
    assert runner.stats["graph_replays"] > 300
    runner.cache.check()


@pytest.mark.parametrize("name,dtype", [("T", "float32"), ("U", "float32"), ("V", "bfloat16"), ("W", "float32")])
def test_greedy_generation_through_the_engine(tmp_path_factory, name, dtype):
    """Engine.generate with its scheduler, graphs and sampler: three prompts of unequal length in portions of at most
    32 tokens; in float32 the ids are the plain implementation's greedy ids."""
    from mashbox_b200.engine.engine import Engine
    folder = S.make_folder(tmp_path_factory.mktemp("m"), name, "float32" if dtype == "float32" else "bfloat16")
    eng = Engine.from_folder(folder, dtype=dtype, page_size=S.CONFIGS[name][2], max_tokens=512, max_requests=3, chunk=32,
                             max_tokens_per_step=40)
    prompts = S.prompts_for(name, (70, 5, 33), seed=5)
    new = 40
    r = eng.generate(prompts, max_new=new)
    assert r["finish"] == ["length"] * 3 and all(len(ids) == new for ids in r["ids"])
    again = eng.generate(prompts, max_new=new)                            # captured graphs now
    assert again["ids"] == r["ids"]
    assert eng.runner.stats["graph_replays"] > 0
    for p, ids in zip(prompts, r["ids"]):
        lg = S.plain_logits(folder, p + ids)
        for t, tok in enumerate(ids):
            row = lg[len(p) + t - 1]
            best = int(row.argmax())
            if dtype == "float32":
                assert tok == best or row[best] - row[tok] < 1e-4, f"{name}: token {t} is {tok}, plain says {best}"
            else:                                                          # bf16 may pick another of two near-equal ids
                assert row[best] - row[tok] < 0.05 * (row.max() - row.min()), f"{name}: token {t} = {tok} is far from the best"
    eng.cache.check()
