"""-m gpu: the Fipitar decoder in the engine against the plain implementation (tests/plain/fipitar.py), in float32 and
bfloat16.  Single kernels on inputs built so that a fault shows: gated recurrences carried across cuts and slots with a
decay per key channel and with one per head, the gates that feed them, layer norm on outputs, the clamped gated unit, head
norms and rotations in both pairings, the rotated strips of latent attention, and the general attention kernels (plain
and tensor-core) with one loud key far back among hundreds, at a page's border, at the query's own position and one
position after it, with sinks, caps, gates and rows wider than what is read.  Then the model layer by layer, whole
prompts, prefill against token-by-token decoding, portions down to two tokens, batches of unequal requests against each
alone, pages and state slots used again, long decoding, and greedy generation through the engine's own entry point."""
import math

import numpy as np
import pytest
import torch

from tests import fipitar_helpers as S
from tests.gpu_harness import DEV, i32, mma_items
from tests.plain import fipitar as plain

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


def dev(t, dtype="float32"):
    return t.to(DEV, TD[dtype]).contiguous()


# ------------------------------------------------------------------------------------------------ the recurrences
def plain_scan(q, k, v, g):
    """q, k (T, H, dim), v (T, H, vdim), g (T, H, dim) float64 -> o (T, H, vdim), the final state (H, dim, vdim)"""
    T, H, dim = q.shape
    S_ = torch.zeros(H, dim, v.shape[-1], dtype=F64)
    o = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        S_ = g[t][:, :, None] * S_ + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S_, q[t])
    return o, S_


@pytest.mark.parametrize("H,G,dim,vdim,per_head", [(3, 3, 16, 24, False), (2, 2, 40, 20, False), (1, 1, 8, 72, False),
                                                    (4, 2, 10, 12, True), (2, 1, 64, 32, True), (3, 3, 6, 10, True),
                                                    (1, 1, 128, 40, False), (2, 2, 200, 12, True), (6, 2, 48, 48, True)])
def test_gated_scan_carries_its_state_across_any_cut(H, G, dim, vdim, per_head):
    """Three sequences advance side by side in portions of their own sizes (1 and 2 tokens among them), in state slots
    that are not in order; the state lies inside a wider tensor.  Decays per key channel, or one per head with queries and
    keys shared by the heads of a group; against the plain loop."""
    from mashbox_b200 import ops
    gen = torch.Generator().manual_seed(dim + vdim)
    lens = [37, 5, 64]
    cuts = [[1, 2, 30, 4], [2, 1, 1, 1], [33, 1, 2, 28]]
    slots = [2, 0, 3]
    pad = 7
    state = torch.zeros(5, pad + H * dim * vdim + 3, device=DEV)
    view = state[:, pad:pad + H * dim * vdim]
    qs = [rnd(gen, n, G, dim, scale=dim ** -0.5) for n in lens]
    ks = [rnd(gen, n, G, dim) for n in lens]
    vs = [rnd(gen, n, H, vdim) for n in lens]
    gs = [torch.rand(n, H, 1 if per_head else dim, generator=gen).float().double() * 0.6 + 0.4 for n in lens]
    want = []
    for s in range(3):
        rep = H // G
        o, fin = plain_scan(qs[s].repeat_interleave(rep, 1), ks[s].repeat_interleave(rep, 1), vs[s],
                            gs[s].expand(lens[s], H, dim))
        want.append((o, fin))
    at = [0, 0, 0]
    got = [[] for _ in range(3)]
    for step in range(4):
        q_len = [cuts[s][step] for s in range(3)]
        q_start = np.concatenate([[0], np.cumsum(q_len)[:-1]])
        cat = lambda xs: torch.cat([xs[s][at[s]:at[s] + q_len[s]].reshape(q_len[s], -1) for s in range(3)])
        N = sum(q_len)
        o = torch.full((N, H * vdim), float("nan"), device=DEV)
        ops.gated_scan(dev(cat(qs)), dev(cat(ks)), dev(cat(vs)), dev(cat(gs)), o, view, (i32(q_start), i32(q_len), i32(slots)),
                       H, G, dim, vdim, per_head)
        for s in range(3):
            got[s].append(o[q_start[s]:q_start[s] + q_len[s]].cpu())
            at[s] += q_len[s]
    for s in range(3):
        kernel_close(torch.cat(got[s]).view(lens[s], H, vdim), want[s][0], "float32", f"sequence {s}")
        kernel_close(view[slots[s]].view(H, dim, vdim), want[s][1], "float32", f"state {s}")
    assert float(state[:, :pad].abs().max()) == 0.0 and float(state[:, pad + H * dim * vdim:].abs().max()) == 0.0
    assert float(state[1].abs().max()) == 0.0 and float(state[4].abs().max()) == 0.0


def test_a_token_600_positions_back_is_kept_as_its_decays_allow():
    """one write, then 600 tokens that write nothing: what a query reads back is the product of the decays, per channel"""
    from mashbox_b200 import ops
    H, dim, vdim, T = 1, 8, 4, 601
    g = torch.full((T, H, dim), 1.0, dtype=F64)
    g[:, 0, 1] = 0.99
    g[:, 0, 2] = 0.5
    k = torch.zeros(T, H, dim, dtype=F64)
    k[0] = 1.0
    v = torch.zeros(T, H, vdim, dtype=F64)
    v[0, 0, 0] = 1.0
    q = torch.zeros(T, H, dim, dtype=F64)
    q[600, 0, 0], q[599, 0, 1], q[598, 0, 2] = 1.0, 1.0, 1.0
    state = torch.zeros(1, H * dim * vdim, device=DEV)
    o = torch.empty(T, H * vdim, device=DEV)
    ops.gated_scan(dev(q.view(T, -1)), dev(k.view(T, -1)), dev(v.view(T, -1)), dev(g.view(T, -1)), o, state,
                   (i32([0]), i32([T]), i32([0])), H, H, dim, vdim, False)
    assert abs(float(o[600, 0]) - 1.0) < 1e-6 and abs(float(o[599, 0]) - 0.99 ** 599) / 0.99 ** 599 < 1e-3
    assert float(o[598, 0]) == 0.0 or float(o[598, 0]) < 1e-30


@pytest.mark.parametrize("dtype", DTYPES)
def test_gates_of_both_recurrences(dtype):
    from mashbox_b200 import ops
    gen = torch.Generator().manual_seed(3)
    N, H, dim, vdim, tau = 9, 3, 10, 6, 4.0
    rows = rnd(gen, N, 2 * H * dim + 2 * H * vdim + 5, dtype=dtype)
    z, zb = rnd(gen, N, H * dim, scale=3.0), rnd(gen, H * dim)
    q, k, g = (torch.empty(N, H * dim, device=DEV) for _ in range(3))
    v = torch.empty(N, H * vdim, device=DEV)
    ops.gla_gates(dev(rows, dtype), dev(z), dev(zb), tau, q, k, v, g, H, dim, vdim)
    kernel_close(q, rows[:, :H * dim] * dim ** -0.5, "float32", "q")
    kernel_close(k, rows[:, H * dim:2 * H * dim], "float32", "k")
    kernel_close(v, rows[:, 2 * H * dim:2 * H * dim + H * vdim], "float32", "v")
    kernel_close(g, torch.sigmoid(z + zb) ** (1 / tau), "float32", "decay = sigmoid^(1/tau)")
    # state-space duality: x, B, C after bias and silu; dt after softplus; dt x as the value; the decay per head
    H, G, P, NS = 4, 2, 6, 5
    xbc = rnd(gen, N, H * P + 2 * G * NS, dtype=dtype)
    cb, dt, dtb, A = rnd(gen, H * P + 2 * G * NS, scale=0.3), rnd(gen, N, H, scale=2.0), rnd(gen, H), rnd(gen, H, scale=0.5)
    dt[0, 0] = 30.0                                                                # softplus without a clamp: the step stays 30
    q, k = (torch.empty(N, G * NS, device=DEV) for _ in range(2))
    v, g = torch.empty(N, H * P, device=DEV), torch.empty(N, H, device=DEV)
    ops.ssd_gates(dev(xbc, dtype), dev(cb), dev(dt), dev(dtb), dev(A), q, k, v, g, H, G, P, NS)
    act = plain.silu(xbc + cb)
    step = plain.softplus(dt + dtb)
    kernel_close(v, (act[:, :H * P].view(N, H, P) * step[:, :, None]).reshape(N, -1), "float32", "dt x")
    kernel_close(k, act[:, H * P:H * P + G * NS], "float32", "B")
    kernel_close(q, act[:, H * P + G * NS:], "float32", "C")
    kernel_close(g, torch.exp(-torch.exp(A) * step), "float32", "decay per head")
    # skip, gate, grouped norm
    o, D, w = rnd(gen, N, H * P), rnd(gen, H), rnd(gen, H * P)
    zrows = rnd(gen, N, H * P + 3, dtype=dtype)
    for parts in (1, 2, 3, 4):
        out = torch.empty(N, H * P, device=DEV, dtype=TD[dtype])
        ops.ssd_out(dev(o), dev(xbc, dtype), dev(cb), dev(D), dev(zrows, dtype)[:, 3:], dev(w), out, H, P, parts, 1e-5)
        y = (o + (D[:, None] * act[:, :H * P].view(N, H, P)).reshape(N, -1)) * plain.silu(zrows[:, 3:])
        y = plain.rms(y.view(N, parts, -1), 1e-5).reshape(N, -1) * w
        kernel_close(out, y, dtype, f"skip, gate, {parts} norm groups")


# ------------------------------------------------------------------------------------------------ rows
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [64, 100, 515, 2048])
def test_layer_norm_on_outputs_and_on_the_stream(dtype, D):
    from mashbox_b200 import ops
    gen = torch.Generator().manual_seed(D)
    N = 7
    x = rnd(gen, N, D) * 3
    y1, y2 = (rnd(gen, N, D) + 5.0).to(TD[dtype]).double(), rnd(gen, N, D, dtype=dtype, scale=4.0)      # a mean to take off
    w, b = rnd(gen, D) + 1, rnd(gen, D)
    xs = dev(x)
    copy = torch.empty(N, D, device=DEV, dtype=TD[dtype])
    ops.ln_add(xs, dev(y1, dtype), dev(w), dev(b), 1e-5, copy)
    want = x + plain.layer_norm(y1, w, b, 1e-5)
    kernel_close(xs, want, "float32", "stream += ln(output)")
    kernel_close(copy, want, dtype, "the stream in the activation dtype")
    ops.ln_add(xs, dev(y1, dtype), dev(w), dev(b), 1e-5, None, dev(y2, dtype), 0.6, -1.1)
    want = want + plain.layer_norm(0.6 * y1 - 1.1 * y2, w, b, 1e-5)
    kernel_close(xs, want, "float32", "stream += ln(weighted sum of two outputs)")
    rows = [5, 0, 5, 2]
    out = torch.empty(len(rows), D, device=DEV, dtype=TD[dtype])
    ops.layer_norm(xs, i32(rows), dev(w), dev(b), 1e-5, out)
    kernel_close(out, plain.layer_norm(want[rows], w, b, 1e-5), dtype, "ln of chosen rows of the stream")


@pytest.mark.parametrize("dtype", DTYPES)
def test_clamped_gated_unit(dtype):
    from mashbox_b200 import ops
    gen = torch.Generator().manual_seed(1)
    gu = rnd(gen, 6, 2 * 37, dtype=dtype, scale=3.0)
    gu[0, 0], gu[0, 37], gu[1, 1], gu[1, 38] = 9.0, 9.0, -9.0, -9.0
    out = torch.empty(6, 37, device=DEV, dtype=TD[dtype])
    ops.glu_clamped(dev(gu, dtype), out, 1.5)
    g, u = torch.clamp(gu[:, :37], max=1.5), torch.clamp(gu[:, 37:], -1.5, 1.5)
    kernel_close(out, g * torch.sigmoid(1.702 * g) * (u + 1), dtype, "min(gate), clamp(up)")
    assert abs(float(out[1, 1]) - (-9.0 / (1 + math.exp(1.702 * 9.0)) * -0.5)) < 1e-6      # the gate is not clamped from below


def paged_rows(lengths, page, seed):
    """-> (table (S, blocks), pages in all): every sequence's pages in shuffled order"""
    gen = torch.Generator().manual_seed(seed)
    blocks = [-(-n // page) for n in lengths]
    total = sum(blocks) + 3
    perm = torch.randperm(total, generator=gen).tolist()
    table = np.full((len(lengths), max(blocks) + 1), -1, np.int32)
    nxt = 0
    for s, nb in enumerate(blocks):
        for b_ in range(nb):
            table[s, b_] = perm[nxt]
            nxt += 1
    return table, total


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,DK,DV,RD,pairing,gain,normed", [(4, 2, 16, 24, 8, 1, 1.0, True), (3, 1, 12, 20, 12, 0, 1.07, True),
                                                               (2, 2, 64, 32, 0, 1, 1.0, True), (6, 3, 32, 8, 16, 0, 1.0, False)])
def test_head_norms_rotation_and_cache_write(dtype, H, KV, DK, DV, RD, pairing, gain, normed):
    from mashbox_b200 import ops
    gen = torch.Generator().manual_seed(DK)
    lengths, page = [11, 4], 4
    table, pages = paged_rows(lengths, page, 1)
    positions = np.concatenate([np.arange(n) for n in lengths])
    tok_row = np.repeat([0, 1], lengths)
    N = len(positions)
    C = (H + KV) * DK + KV * DV + 5
    rows = rnd(gen, N, C, dtype=dtype)
    qw, kw = rnd(gen, DK) + 1, rnd(gen, DK) + 1
    freqs = torch.tensor([100.0 ** (-2 * i / max(RD, 1)) for i in range(RD // 2)], dtype=torch.float32)
    kpool = torch.zeros(pages, KV, page, DK, device=DEV, dtype=TD[dtype])
    vpool = torch.zeros(pages, KV, page, DV, device=DEV, dtype=TD[dtype])
    r = dev(rows, dtype)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.norm_rope_kv_write(r, dev(qw) if normed else None, dev(kw) if normed else None, 1e-6, dev(freqs) if RD else None, RD,
                           pairing, gain, i32(positions), i32(tok_row), i32(table), kpool, vpool, H, KV, DK, DV, page, pages, err)
    assert int(err.item()) == 0

    def want_heads(x, w):
        x = plain.rms(x, 1e-6, w) if normed else x
        if not RD:
            return x
        a = torch.as_tensor(positions, dtype=F64)[:, None] * freqs.double()[None, :]
        c, s = (torch.cos(a) * gain)[:, None, :], (torch.sin(a) * gain)[:, None, :]
        if pairing == 1:
            u, v = x[..., :RD // 2], x[..., RD // 2:RD]
            return torch.cat([u * c - v * s, v * c + u * s, x[..., RD:]], -1)
        u, v = x[..., 0:RD:2], x[..., 1:RD:2]
        return torch.cat([torch.stack([u * c - v * s, v * c + u * s], -1).reshape(*x.shape[:-1], RD), x[..., RD:]], -1)
    q = want_heads(rows[:, :H * DK].view(N, H, DK), qw)
    k = want_heads(rows[:, H * DK:(H + KV) * DK].view(N, KV, DK), kw)
    v = rows[:, (H + KV) * DK:(H + KV) * DK + KV * DV].view(N, KV, DV)
    kernel_close(r[:, :H * DK], q.reshape(N, -1), dtype, "q in place")
    kernel_close(r[:, (H + KV) * DK:], rows[:, (H + KV) * DK:], dtype, "what lies behind the keys is left alone", 1e-9)
    for n in range(N):
        pg, slot = table[tok_row[n], positions[n] // page], positions[n] % page
        kernel_close(kpool[pg, :, slot], k[n], dtype, f"key of token {n} in its page")
        kernel_close(vpool[pg, :, slot], v[n], dtype, f"value of token {n} in its page", 1e-9)


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_strips_and_wide_rows(dtype):
    """the normed latent goes into the first values of a wider cache row, the rotated key strip behind it; the query's
    unrotated part passes its head's matrix into the first values of a wider query row, its rotated strip behind it"""
    from mashbox_b200 import ops
    gen = torch.Generator().manual_seed(5)
    H, dim, rd, R, rank, qr, page = 3, 6, 10, 6, 14, 9, 4
    lengths = [9, 6]
    table, pages = paged_rows(lengths, page, 2)
    positions = np.concatenate([np.arange(n) for n in lengths])
    tok_row = np.repeat([0, 1], lengths)
    N = len(positions)
    rows = rnd(gen, N, qr + rank + rd, dtype=dtype)
    nq, nkv = rnd(gen, qr) + 1, rnd(gen, rank) + 1
    pool = torch.zeros(pages, 1, page, rank + rd, device=DEV, dtype=TD[dtype])
    cq = torch.empty(N, qr, device=DEV, dtype=TD[dtype])
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.rms_segments_wide(dev(rows, dtype), 0, dev(nq), cq, qr, dev(nkv), pool, i32(positions), i32(tok_row), i32(table), page,
                          pages, 1e-6, err)
    kernel_close(cq, plain.rms(rows[:, :qr], 1e-6, nq), dtype, "query latent")
    q = rnd(gen, N, H * (dim + rd), dtype=dtype)
    wuk = rnd(gen, H * dim, rank, dtype=dtype)
    qa = torch.zeros(N, H * (rank + rd), device=DEV, dtype=TD[dtype])
    ops.head_product_strided(dev(q, dtype), dim, dev(wuk, dtype), qa, rank, H, transposed=True)
    freqs = torch.tensor([50.0 ** (-2 * i / R) for i in range(R // 2)], dtype=torch.float32)
    gain = 1.2
    ops.latent_rope(dev(q, dtype), dim + rd, dim, qa, rank + rd, rank, dev(rows, dtype), qr + rank, pool, rank, dev(freqs), R, rd, 0,
                    gain, i32(positions), i32(tok_row), i32(table), H, page, pages, err)
    assert int(err.item()) == 0
    rot = dict(dims=R, base=50.0)
    pos = torch.as_tensor(positions)
    q3 = q.view(N, H, dim + rd)
    want_q = torch.cat([torch.einsum("nhi,hij->nhj", q3[..., :dim], wuk.view(H, dim, rank)),
                        plain.rotate(q3[..., dim:], pos, rot, "adjacent") * 1.0], -1)
    # the gain multiplies cos and sin: the rotated pairs only
    want_q[..., rank:rank + R] = plain.rotate(q3[..., dim:], pos, rot, "adjacent")[..., :R] * gain
    kernel_close(qa.view(N, H, rank + rd), want_q, dtype, "query rows [matrix applied | strip]")
    kr = plain.rotate(rows[:, None, qr + rank:], pos, rot, "adjacent")[:, 0]
    kr[:, :R] *= gain
    want_row = torch.cat([plain.rms(rows[:, qr:qr + rank], 1e-6, nkv), kr], -1)
    for n in range(N):
        pg, slot = table[tok_row[n], positions[n] // page], positions[n] % page
        kernel_close(pool[pg, 0, slot], want_row[n], dtype, f"cache row of token {n}")


# ------------------------------------------------------------------------------------------------ general attention
def plain_general_attention(q, k, v, scale, cap, sinks, gate, G):
    """q (T, H, DK), k (T, KV, DK), v (T, KV, DV) of one sequence, float64; sinks (H,) or None; gate (T, H) logits or None"""
    T, H, _ = q.shape
    k, v = k.repeat_interleave(G, 1), v.repeat_interleave(G, 1)
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), -math.inf)
    if sinks is None:
        w = torch.softmax(s, -1)
    else:
        w = plain.softmax_with_sink(s, sinks[:, None].expand(H, T))
    o = torch.einsum("hij,jhd->ihd", w, v)
    return o if gate is None else o * torch.sigmoid(gate)[:, :, None]


class GeneralCase:
    """S sequences in shuffled pages; the last q_len positions of each are the step's queries.  `shared`: keys and values
    are one pool whose row is the key, the value its first DV values (then KV = 1)."""

    def __init__(self, dtype, H, KV, DK, DV, lengths, q_lens, page, seed=0, shared=False, loud=None, sinks=True, gate=True,
                 quiet=1.0):
        gen = torch.Generator().manual_seed(seed)
        self.__dict__.update(dtype=dtype, H=H, KV=KV, DK=DK, DV=DV, lengths=lengths, q_lens=q_lens, page=page, shared=shared)
        G = H // KV
        self.q = [rnd(gen, n, H, DK, dtype=dtype) for n in lengths]
        self.k = [rnd(gen, n, KV, DK, dtype=dtype, scale=quiet if shared else 1.0) for n in lengths]
        self.v = [k_[..., :DV].clone() for k_ in self.k] if shared else [rnd(gen, n, KV, DV, dtype=dtype, scale=quiet) for n in lengths]
        for (s, qpos, kpos, amount) in (loud or []):             # one score that stands out: query qpos of sequence s, key kpos
            d = torch.zeros(DK, dtype=F64)
            d[DK - 1] = 1.0
            self.q[s][qpos, :, :] = d * amount
            self.k[s][kpos, :, :] = d * amount
            self.v[s][kpos] = 0.0
            self.v[s][kpos, :, 0] = 8.0                         # ... whose value is loud in its first channel
            if shared:
                self.k[s][kpos, :, :DV] = self.v[s][kpos]
        self.sinks = rnd(gen, H, scale=1.5) if sinks else None
        self.gate = [rnd(gen, n, H, dtype=dtype) for n in lengths] if gate else None
        table, pages = paged_rows(lengths, page, seed + 1)
        krow = DK
        kpool = torch.zeros(pages, KV, page, krow, dtype=F64)
        vpool = torch.zeros(pages, KV, page, DV, dtype=F64)
        for s, n in enumerate(lengths):
            for p in range(n):
                pg, slot = table[s, p // page], p % page
                kpool[pg, :, slot] = self.k[s][p]
                vpool[pg, :, slot] = self.v[s][p]
        self.table, self.pages = i32(table), pages
        self.kpool = dev(kpool, dtype)
        self.vpool = self.kpool if shared else dev(vpool, dtype)
        self.positions = i32(np.concatenate([np.arange(n - ql, n) for n, ql in zip(lengths, q_lens)]))
        self.tok_row = i32(np.repeat(np.arange(len(lengths)), q_lens))
        self.N = sum(q_lens)
        extra = 8                                                # the gates' logits behind the queries, and zero padding
        rows = torch.zeros(self.N, H * DK + extra * ((H + extra - 1) // extra), dtype=F64)
        at = 0
        for s, (n, ql) in enumerate(zip(lengths, q_lens)):
            rows[at:at + ql, :H * DK] = self.q[s][n - ql:].reshape(ql, -1)
            if gate:
                rows[at:at + ql, H * DK:H * DK + H] = self.gate[s][n - ql:]
            at += ql
        self.rows = dev(rows, dtype)
        self.gate_view = self.rows[:, H * DK:H * DK + H] if gate else None

    def want(self, scale, cap):
        out = []
        for s, (n, ql) in enumerate(zip(self.lengths, self.q_lens)):
            o = plain_general_attention(self.q[s], self.k[s], self.v[s], scale, cap, self.sinks,
                                        self.gate[s] if self.gate is not None else None, self.H // self.KV)
            out.append(o[n - ql:].reshape(ql, -1))
        return torch.cat(out)

    def run_plain(self, scale, cap):
        from mashbox_b200 import ops
        out = torch.full((self.N, self.H * self.DV), float("nan"), device=DEV, dtype=TD[self.dtype])
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.attention_general(self.rows, self.rows.stride(0), out, self.positions, self.tok_row, self.table, self.kpool,
                              self.vpool, self.H, self.KV, self.DK, self.DV, self.page, self.pages, None, scale, err, cap,
                              dev(self.sinks) if self.sinks is not None else None, self.gate_view)
        assert int(err.item()) == 0
        return out

    def run_mma(self, scale, cap, splits=1):
        from mashbox_b200 import ops
        H, KV = self.H, self.KV
        dec, pre, part_base, part_tok = mma_items(self, H // KV, splits)
        out = torch.full((self.N, H * self.DV), float("nan"), device=DEV, dtype=torch.bfloat16)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        ms = 16
        n_part = len(part_tok) // 2
        part_o = torch.zeros(max(1, n_part) * H * ms, self.DV, device=DEV)
        part_ml = torch.zeros(max(1, n_part) * H * ms, 2, device=DEV)
        q_start = np.concatenate([[0], np.cumsum(self.q_lens)[:-1]])
        pos0 = [n - ql for n, ql in zip(self.lengths, self.q_lens)]
        sinks = dev(self.sinks) if self.sinks is not None else None
        for items, decode in ((pre, False), (dec, True)):
            if items:
                ops.attention_general_mma(self.rows, self.rows.stride(0), out, self.kpool, self.vpool,
                                          i32(np.asarray(items).reshape(-1)), len(items), decode, i32(q_start), i32(self.q_lens),
                                          i32(pos0), i32(part_base), i32(np.arange(len(self.lengths))), self.table, part_o,
                                          part_ml, ms, H, KV, self.DK, self.DV, self.page, self.pages, None, scale, err, cap,
                                          sinks, self.gate_view)
        if n_part:
            ops.attention_general_merge(part_o, part_ml, i32(part_tok), n_part, out, H, self.DK, self.DV, ms, sinks, self.gate_view)
        assert int(err.item()) == 0
        return out


GENERAL_SHAPES = [("plain", 4, 2, 16, 24, 8), ("plain", 3, 1, 12, 20, 5), ("plain", 5, 1, 40, 24, 16), ("mma", 8, 2, 32, 64, 16),
                  ("mma", 2, 1, 128, 16, 8), ("mma", 4, 4, 16, 16, 16), ("mma", 6, 1, 80, 64, 16), ("mma", 20, 1, 160, 128, 32)]


@pytest.mark.parametrize("kernel,H,KV,DK,DV,page", GENERAL_SHAPES)
def test_general_attention_far_away_at_page_borders_and_after_the_query(kernel, H, KV, DK, DV, page):
    """ONE loud key -- far back among 700, at the last slot of a page and the first of the next, at the query's own
    position, and one position AFTER the query (which must not count) -- in prompt portions and in single decoded tokens,
    with sinks, a cap well above the loud score's reach, gates, and, for one kv head, rows that are key and value at once"""
    shared = KV == 1 and DV <= DK and kernel == "mma" or (kernel, DK) == ("plain", 40)
    dtypes = ("bfloat16",) if kernel == "mma" else DTYPES
    amount = 4.5            # the loud score is 20: e^20 beside hundreds of keys whose scores are 4.5 times a unit normal
    scale, cap = 1.0, 50.0
    for dtype in dtypes:
        for lengths, q_lens, loud in (([700, 40], [1, 1], [(0, 699, 3, amount), (1, 39, 39, amount)]),
                                      ([700, 2 * page + 2], [30, page + 2], [(0, 680, 7, amount), (1, page + 1, page - 1, amount)]),
                                      ([3 * page, 2 * page + 1], [2, 1], [(0, 3 * page - 2, 3 * page - 1, amount), (1, 2 * page, page, amount)]),
                                      ([90, 300], [90, 300], [(0, 50, 51, amount), (1, 299, 0, amount)])):
            case = GeneralCase(dtype, H, KV, DK, DV, lengths, q_lens, page, seed=len(lengths) + page, shared=shared, loud=loud,
                               gate=False, quiet=0.25)
            want = case.want(scale, cap)
            got = case.run_plain(scale, cap) if kernel == "plain" else case.run_mma(scale, cap)
            kernel_close(got, want, dtype, f"{kernel} {lengths} {q_lens}", 3e-2 if dtype == "bfloat16" else None)
            # where the loud key is seen the first value channel is loud (its value there is 8, the others' a quarter of a
            # unit normal); where it lies after the query it is not
            at = 0
            for s, (n, ql) in enumerate(zip(lengths, q_lens)):
                for (ls, qpos, kpos, _) in loud:
                    if ls == s and qpos >= n - ql:
                        row = want[at + qpos - (n - ql)].view(H, DV)[:, 0].abs().min()
                        assert (row > 2.0) == (kpos <= qpos), (lengths, qpos, kpos, float(row))
                at += ql


@pytest.mark.parametrize("kernel", ["plain", "mma"])
def test_sinks_caps_and_gates_each_change_the_result_as_they_should(kernel):
    dtype = "bfloat16" if kernel == "mma" else "float32"
    run = lambda c, scale, cap: c.run_plain(scale, cap) if kernel == "plain" else c.run_mma(scale, cap)
    for sinks, gate, cap, scale in ((True, False, None, 0.3), (False, True, None, 0.3), (False, False, 1.5, 2.0), (True, True, 4.0, 1.0)):
        case = GeneralCase(dtype, 4, 2, 32, 16, [70, 9], [70, 1], 16, seed=9, sinks=sinks, gate=gate)
        kernel_close(run(case, scale, cap), case.want(scale, cap), dtype, f"sinks {sinks} gate {gate} cap {cap}", 3e-2 if kernel == "mma" else None)
    # a sink far above every score takes the whole weight: the result vanishes; far below: the plain softmax
    case = GeneralCase(dtype, 2, 2, 16, 16, [20], [20], 8, seed=1, gate=False)
    case.sinks = torch.tensor([40.0, -40.0], dtype=F64)
    got = run(case, 0.1, None).float().cpu().view(20, 2, 16)
    assert float(got[:, 0].abs().max()) < 1e-6
    kernel_close(got[:, 1], plain_general_attention(case.q[0], case.k[0], case.v[0], 0.1, None, None, None, 1)[:, 1], dtype, "no sink")
    # the first token of a sequence sees itself and the sink: its weight is e^s / (e^sink + e^s)
    case = GeneralCase(dtype, 1, 1, 16, 16, [1], [1], 8, seed=2, gate=False)
    case.sinks = torch.zeros(1, dtype=F64)
    s = float((case.q[0][0, 0] * case.k[0][0, 0]).sum()) * 0.25
    got = run(case, 0.25, None).float().cpu()[0]
    kernel_close(got, case.v[0][0, 0] * (math.exp(s) / (1 + math.exp(s))), dtype, "one key and a sink of score zero")


@pytest.mark.parametrize("splits", [1, 2, 4, 16])
def test_general_decode_form_cut_along_the_keys(splits):
    case = GeneralCase("bfloat16", 8, 2, 32, 64, [700, 130, 17], [1, 2, 1], 16, seed=splits, loud=[(0, 699, 5, 3.0)])
    kernel_close(case.run_mma(0.2, 10.0, splits), case.want(0.2, 10.0), "bfloat16", f"{splits} splits", 3e-2)
    case = GeneralCase("bfloat16", 6, 1, 80, 64, [500, 64], [1, 1], 16, seed=splits, shared=True)
    kernel_close(case.run_mma(0.1, None, splits), case.want(0.1, None), "bfloat16", f"{splits} splits, shared rows", 3e-2)


# ------------------------------------------------------------------------------------------------ the model in the engine
def runner_for(tmp, name, dtype, max_tokens, options=None, max_requests=4, config=None):
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


@pytest.mark.parametrize("name", ["P", "Q", "Z"])
def test_layer_by_layer(tmp_path_factory, name):
    """float32: the model cut after its first, second, ... layer (a tensor's values depend on its name and the seed alone,
    so the shorter models are the longer one's beginnings) against the plain implementation cut alike"""
    import dataclasses
    import json
    import os
    from mashbox_b200.engine.replay import make_runner
    from mashbox_b200.weights.random_init import write_model_folder
    from tests.plain.llama import read_model
    cfg, seed, page = S.CONFIGS[name]
    tmp = tmp_path_factory.mktemp("layers")
    (p,) = S.prompts_for(name, (45,))
    for n in range(1, len(cfg.layers) + 1):
        d = os.path.join(str(tmp), f"first{n}")
        write_model_folder(d, dataclasses.replace(cfg, layers=cfg.layers[:n]), seed, dtype=torch.float32, std=cfg.width ** -0.5,
                           norm_std=0.1, std_by_name=S.STD_BY_NAME)
        c, W = read_model(d)
        assert len(json.load(open(os.path.join(d, "config.json")))["layers"]) == n
        want = plain.forward(c, W, p).numpy()
        runner = make_runner(d, "float32", 64, page_size=page)
        got = replay(runner, cut_steps("a", p, [len(p)]))[0]
        S.assert_close(got, want, "float32", f"{name}: the first {n} layers ({cfg.layers[n - 1].type} last)")


@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random(tmp_path_factory, seed):
    """2 to 5 layers of any kind in any order with sizes drawn from small sets: a whole prompt, then the same prompt in
    portions and single tokens through a pool of four pages' slack, float32 against the plain model and bfloat16 against
    float32's bars for bfloat16"""
    import os
    from mashbox_b200.engine.replay import make_runner
    from mashbox_b200.weights.random_init import write_model_folder
    from tests.plain.llama import read_model
    cfg = S.random_config(seed)
    page = (4, 8, 16, 5)[seed % 4]
    tmp = tmp_path_factory.mktemp("r")
    rng = np.random.default_rng(seed)
    p = rng.integers(0, cfg.vocab, 75).tolist()
    for dtype in DTYPES:
        d = os.path.join(str(tmp), dtype)
        write_model_folder(d, cfg, 500 + seed, dtype=TD[dtype], std=cfg.width ** -0.5, norm_std=0.1, std_by_name=S.STD_BY_NAME)
        c, W = read_model(d)
        want = plain.forward(c, W, p).numpy()
        runner = make_runner(d, dtype, 128, page_size=page)
        whole = replay(runner, cut_steps("a", p, [len(p)]))[0]
        S.assert_close(whole, want, dtype, f"random configuration {seed}: {[l.type for l in cfg.layers]}, whole")
        cuts = [33, 2, 1, 17, 1, 1, 20]
        out = replay(runner, cut_steps("b", p, cuts))
        S.assert_close(np.concatenate([out[i] for i in range(len(cuts))]), want, dtype, f"random configuration {seed}, in portions")
        runner.cache.check()


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


@pytest.mark.parametrize("name,dtype,options", [("R", "bfloat16", dict(plain_attention=True)),
                                                ("R", "bfloat16", dict(attention_splits=4)),
                                                ("R", "bfloat16", dict(attention_target_blocks=1)),
                                                ("P", "bfloat16", dict(plain_attention=True))])
def test_every_kernel_form_gives_the_same_model(tmp_path_factory, name, dtype, options):
    """the forms the engine chooses between, forced: the plain attention kernel beside the tensor-core one, decode keys
    cut four ways and not at all"""
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), name, dtype, 512, options=options)
    (p,) = S.prompts_for(name, (300,), seed=7)
    want = S.plain_logits(folder, p)
    out = replay(runner, cut_steps("a", p, [200, 70] + [1] * 30))
    got = np.concatenate([out[i] for i in range(32)])
    S.assert_close(got, want, dtype, f"{name} with {options}")


def test_tensor_core_attention_is_what_bfloat16_runs(tmp_path_factory):
    from mashbox_b200 import ops
    folder, runner = runner_for(tmp_path_factory.mktemp("m"), "R", "bfloat16", 128)
    (p,) = S.prompts_for("R", (70,), seed=8)
    replay(runner, cut_steps("a", p, [69, 1]))
    loaded = [k[0] for k in ops._fn_cache]
    for pair in ("32_64", "80_64", "128_16", "160_128", "16_16"):
        assert f"attention_general_mma_{pair}" in loaded, (pair, loaded)


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("P", "bfloat16"), ("R", "bfloat16"), ("S", "float32"),
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


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("Q", "float32"), ("R", "bfloat16"), ("S", "float32")])
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
