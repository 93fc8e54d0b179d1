"""The kernels and the whole path of the Tibepel design on the GPU, against the plain implementation
(plain_tibepel.py): every mechanism alone - with planted keys and values where random numbers would hide a fault -, then
trace replay under the four schedules in both number formats, generation through the entry point and its scheduler,
and long decoding."""
import io
import math

import pytest
import torch

import plain_tibepel as P
import tibepel_tools as X
import trace_tools as TT
from gpu_tools import rel_err
from model_tools import random_requests

pytestmark = pytest.mark.gpu
F64 = torch.float64
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.6e-2}


@pytest.fixture(scope="module")
def K():
    from rvllm_b200.kernels import get_library
    return get_library("cuda:0")


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64) * scale


def i32(values):
    return torch.tensor(values, dtype=torch.int32).cuda()


# ---------------------------------------------------------------------------------------- row kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [45, 256, 1032])
def test_scaled_embeddings_plus_position_vector(K, dtype, cols):
    """Late positions are as exact as early ones: the angle is formed in double precision."""
    pos = [0, 1, 2, 119, 120, 4095, 100000, 131071]
    x = rnd(len(pos), cols, seed=1).to(dtype)
    freq = torch.tensor([10000.0 ** (-2.0 * i / cols) for i in range((cols + 1) // 2)], dtype=F64)
    got = K.scale_add_sinusoid(x.cuda(), i32(pos), freq.cuda(), 3.5)
    want = x.double() * 3.5 + P.sinusoid(pos, cols)
    assert got.dtype == torch.float32 and float((got.double().cpu() - want).abs().max()) < 3e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [45, 352, 4096 + 24])
def test_stream_sum_and_the_next_sublayers_input(K, dtype, cols):
    x, y, w = rnd(6, cols, seed=2, scale=3.0).float(), rnd(6, cols, seed=3).float(), rnd(cols, seed=4, scale=0.3).float()
    tol = 4e-6 if dtype == torch.float32 else 5e-3
    s = x.double() + y.double()
    xs = x.clone().cuda()
    out, nxt = K.stream_add_norm(xs, y.cuda(), ((w + 1.0).cuda(), 1e-5), dtype)
    assert out is xs and rel_err(out, s) < 1e-7 and nxt.dtype == dtype and rel_err(nxt, P.offset_norm(s, w.double(), 1e-5)) < tol
    out, nxt = K.stream_add_norm(x.clone().cuda(), y.cuda(), None, dtype)
    assert rel_err(out, s) < 1e-7 and rel_err(nxt, s) < tol
    out, nxt = K.stream_add_norm(x.clone().cuda(), y.cuda(), None, None)
    assert nxt is None and rel_err(out, s) < 1e-7
    # the norm of the stream alone, as the first sublayer of a layer and the output read it
    got = K.rmsnorm(x.cuda(), (w + 1.0).cuda(), 1e-6, out_dtype=dtype)
    assert got.dtype == dtype and rel_err(got, P.offset_norm(x.double(), w.double(), 1e-6)) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_steps_around_the_mixers(K, dtype):
    tol = 4e-6 if dtype == torch.float32 else 5e-3
    gu = rnd(9, 2 * 37, seed=5, scale=3.0).float()
    for limit in (0.7, 2.5):
        g, u = torch.clamp(gu[:, :37].double(), max=limit), torch.clamp(gu[:, 37:].double(), -limit, limit)
        got = K.act_mul(gu.cuda(), "swiglu_clamp", dtype, limit=limit, alpha=1.702)
        assert got.dtype == dtype and rel_err(got, g * torch.sigmoid(1.702 * g) * (u + 1.0)) < tol
    g, rows = rnd(7, 5, seed=6, scale=2.0).float(), rnd(7, 23, seed=7).to(dtype)
    got = K.gelu_mul_columns(g.cuda(), rows.cuda(), 15, dtype)
    assert rel_err(got, P.gelu_tanh(g.double()) * rows[:, 15:20].double()) < tol
    wide = rnd(5, 29, seed=8).float()
    assert rel_err(K.column_slice(wide.cuda(), 3, 11, dtype), wide[:, 3:14].double()) < tol
    a, b = rnd(4, 33, seed=9).float(), rnd(4, 33, seed=10).float()
    first = K.scaled_sum(None, 1.0, b.cuda(), -0.6)
    assert rel_err(first, -0.6 * b.double()) < 1e-7
    acc = a.clone().cuda()
    assert K.scaled_sum(acc, 1.0, b.cuda(), 1.3) is acc and rel_err(acc, a.double() + 1.3 * b.double()) < 1e-6
    # per-head norm with a weight shared by the heads, then the gate read from the middle of a wider row
    for heads, vd in ((3, 20), (4, 64), (1, 7), (2, 200)):
        o, gamma, proj = rnd(6, heads * vd, seed=11, scale=4.0).float(), (rnd(vd, seed=12) + 1.0).to(dtype), rnd(6, 13 + heads * vd + 2, seed=13).float()
        got = K.head_norm_gate(o.cuda(), gamma.cuda(), 1e-5, proj.cuda(), 13, heads, vd, dtype)
        z = proj[:, 13:13 + heads * vd].double().view(6, heads, vd)
        want = P.rms(o.double().view(6, heads, vd), 1e-5) * gamma.double() * P.silu(z)
        assert rel_err(got, want.reshape(6, -1)) < tol


# ---------------------------------------------------------------------------------------- recurrences
def _portions(total, cuts):
    """[(start, stop)] of a sequence of `total` tokens cut at `cuts`."""
    edges = [0, *cuts, total]
    return [(a, b) for a, b in zip(edges[:-1], edges[1:]) if b > a]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,N,taps", [(40, 12, 3), (11, 1, 1), (72, 33, 5), (384, 16, 4), (40, 70, 2), (130, 256, 4)])
def test_convolution_and_channel_scan_carry_their_state(K, dtype, inner, N, taps):
    """Two sequences in changing slots, cut into portions down to one token, side by side in one step: the outputs equal
    those of the whole sequences, and a slot that is handed on zeroed starts a new sequence."""
    T = (37, 22)
    lens_cuts = ([5, 6, 8, 30], [1, 2, 19])
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    A = -torch.exp(rnd(inner, N, seed=20, scale=0.5))
    Dk, dt_bias = rnd(inner, seed=21), rnd(inner, seed=22) - 1.0
    w, b = rnd(inner, taps, seed=23, scale=0.5).to(dtype), rnd(inner, seed=24, scale=0.2).to(dtype)
    seqs = []
    for s, n in enumerate(T):
        xz = rnd(n, 2 * inner + 3, seed=30 + s).float()                       # [3 junk | u | z]
        dt_raw, bc = rnd(n, inner, seed=40 + s).float(), rnd(n, 2 + 2 * N, seed=50 + s).float()   # [2 junk | B | C]
        u = P.silu(P.causal_conv(xz[:, 3:3 + inner].double(), w.double(), b.double()))
        u_kept = u.to(dtype).double()
        y = P.channel_scan(u_kept, P.softplus(dt_raw.double() + dt_bias), A, bc[:, 2:2 + N].double(), bc[:, 2 + N:].double(), Dk)
        seqs.append((xz, dt_raw, bc, u, y * P.silu(xz[:, 3 + inner:].double())))
    floats = inner * N + (taps - 1) * inner
    state = torch.full((5, floats + 4), 9.0).cuda()
    slots = (3, 1)
    state[list(slots), :floats] = 0.0
    parts = [_portions(n, c) for n, c in zip(T, lens_cuts)]
    got_u, got_y = [[], []], [[], []]
    for step in range(max(len(p) for p in parts)):
        live = [s for s in range(2) if step < len(parts[s])]
        pieces = [parts[s][step] for s in live]
        cat = lambda idx: torch.cat([seqs[s][idx][a:b] for s, (a, b) in zip(live, pieces)]).cuda()
        cu = [0]
        for a, b_ in pieces:
            cu.append(cu[-1] + b_ - a)
        token_seq = torch.cat([torch.full((b_ - a,), i, dtype=torch.int32) for i, (a, b_) in enumerate(pieces)]).cuda()
        sl = i32([slots[s] for s in live])
        xz = cat(0)
        u = K.causal_conv_silu(xz, 3, inner, w.cuda(), b.cuda(), token_seq, i32(cu), sl, state, inner * N, dtype)
        y = K.selective_scan(u, cat(1), dt_bias.float().cuda(), A.float().cuda(), cat(2), 2, 2 + N, Dk.float().cuda(), xz, 3 + inner,
                             i32(cu), sl, state, dtype)
        for i, s in enumerate(live):
            got_u[s].append(u[cu[i]:cu[i + 1]])
            got_y[s].append(y[cu[i]:cu[i + 1]])
    for s in range(2):
        assert rel_err(torch.cat(got_u[s]), seqs[s][3]) < tol / 2, s
        assert rel_err(torch.cat(got_y[s]), seqs[s][4]) < tol, s
    assert bool((state[[0, 2, 4]] == 9.0).all()) and bool((state[:, floats:] == 9.0).all())      # nobody else's row is touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,vd", [(4, 2, 12, 20), (1, 1, 5, 3), (4, 4, 32, 64), (6, 2, 34, 9), (2, 1, 128, 32), (3, 3, 64, 130), (2, 2, 200, 40)])
def test_gated_delta_rule_carries_its_state(K, dtype, H, G, d, vd):
    T = (45, 19)
    lens_cuts = ([7, 8, 10, 40], [2, 3, 4])
    tol = 3e-5 if dtype == torch.float32 else 1.5e-2
    a_log, dt_bias = rnd(H, seed=60) - 1.5, rnd(H, seed=61)
    qk = G * d
    seqs = []
    for s, n in enumerate(T):
        qkv = rnd(n, 2 * qk + H * vd, seed=62 + s).to(dtype)
        proj = rnd(n, 3 + 2 * H, seed=70 + s, scale=2.0).float()             # [3 junk | beta logits | decay logits]
        x = qkv.double()
        q = (P.unit(x[:, :qk].view(n, G, d)) * d ** -0.5).repeat_interleave(H // G, dim=1)
        k = P.unit(x[:, qk:2 * qk].view(n, G, d)).repeat_interleave(H // G, dim=1)
        beta = torch.sigmoid(proj[:, 3:3 + H].double())
        g = torch.exp(-torch.exp(a_log) * P.softplus(proj[:, 3 + H:].double() + dt_bias))
        seqs.append((qkv, proj, P.delta_rule(q, k, x[:, 2 * qk:].view(n, H, vd), beta, g).reshape(n, -1)))
    floats = H * d * vd
    state = torch.full((4, floats + 6), 9.0).cuda()
    slots = (2, 0)
    state[list(slots), :floats] = 0.0
    parts = [_portions(n, c) for n, c in zip(T, lens_cuts)]
    got = [[], []]
    for step in range(max(len(p) for p in parts)):
        live = [s for s in range(2) if step < len(parts[s])]
        pieces = [parts[s][step] for s in live]
        cu = [0]
        for a, b in pieces:
            cu.append(cu[-1] + b - a)
        qkv = torch.cat([seqs[s][0][a:b] for s, (a, b) in zip(live, pieces)]).cuda()
        proj = torch.cat([seqs[s][1][a:b] for s, (a, b) in zip(live, pieces)]).cuda()
        o = K.delta_rule(qkv, proj, 3, 3 + H, a_log.float().cuda(), dt_bias.float().cuda(), i32(cu), i32([slots[s] for s in live]), state,
                         H, G, d, vd, 1e-6)
        assert o.dtype == torch.float32
        for i, s in enumerate(live):
            got[s].append(o[cu[i]:cu[i + 1]])
    for s in range(2):
        assert rel_err(torch.cat(got[s]), seqs[s][2]) < tol, s
    assert bool((state[[1, 3]] == 9.0).all()) and bool((state[:, floats:] == 9.0).all())


def test_delta_rule_keeps_a_value_over_a_long_stretch(K):
    """A value written once under a key that no later token touches (orthogonal keys, no decay on that head) is read
    back unchanged 700 tokens later, token by token; the head that decays has forgotten it."""
    H, d, vd, n = 2, 16, 8, 700
    qkv = torch.zeros(n, 2 * H * d + H * vd, dtype=F64)
    for h in range(H):
        qkv[0, H * d + h * d] = 5.0                          # k: first axis
        qkv[0, 2 * H * d + h * vd:2 * H * d + (h + 1) * vd] = torch.arange(1, vd + 1, dtype=F64)
        qkv[1:, H * d + h * d + 1] = 1.0                     # later keys: second axis only
        qkv[n - 1, h * d] = 2.0                              # the last query asks along the first axis
    proj = torch.zeros(n, 2 * H)
    proj[:, :H] = 30.0                                       # beta = 1
    proj[:, H] = -60.0                                       # head 0: softplus -> 0, no decay;  head 1: decay exp(-exp(0) softplus(0))
    a_log = torch.zeros(H)
    state = torch.zeros(1, H * d * vd).cuda()
    cu, slot = i32([0, 1]), i32([0])
    for t in range(n):
        o = K.delta_rule(qkv[t:t + 1].float().cuda(), proj[t:t + 1].cuda(), 0, H, a_log.cuda(), torch.zeros(H).cuda(), cu, slot, state,
                         H, H, d, vd, 1e-6)
    want = torch.arange(1, vd + 1, dtype=F64) * d ** -0.5
    assert rel_err(o[0, :vd], want) < 1e-5
    assert float(o[0, vd:].abs().max()) < 1e-30


# ---------------------------------------------------------------------------------------- attention over the paged cache
def flat_pages(k_seqs, v_seqs, q_lens, page, dtype, chunk=None, seed=0, spare=3):
    """Scatter whole-sequence keys [ctx, G, d] and values [ctx, G, vd] into shuffled pages of a cache whose pages hold
    their key rows and then their value rows.  The last q_len tokens of a sequence are the step's.  Pages that lie wholly
    below the chunk of a sequence's first query have been given back: their table entries are -1 and their keys are
    nowhere.  Slots nobody wrote hold finite junk, as a page that is used again would."""
    from rvllm_b200.kernels import AttentionMeta
    B, (G, d), vd = len(k_seqs), k_seqs[0].shape[1:], v_seqs[0].shape[2]
    ctx = [k.shape[0] for k in k_seqs]
    blocks = [(c + page - 1) // page for c in ctx]
    n_pages = sum(blocks) + spare
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    keys = torch.full((n_pages, G, page, d), 3.0, dtype=torch.float32)
    vals = torch.full((n_pages, G, page, vd), -2.0, dtype=torch.float32)
    table = torch.full((B, max(blocks)), -1, dtype=torch.int32)
    nxt = 0
    for b in range(B):
        first = ctx[b] - q_lens[b]
        first_seen = (first // chunk) * chunk if chunk else 0
        for blk in range(blocks[b]):
            if (blk + 1) * page <= first_seen:
                continue
            pg = perm[nxt]
            nxt += 1
            table[b, blk] = pg
            lo, hi = blk * page, min(ctx[b], (blk + 1) * page)
            keys[pg, :, :hi - lo] = k_seqs[b][lo:hi].transpose(0, 1)
            vals[pg, :, :hi - lo] = v_seqs[b][lo:hi].transpose(0, 1)
    cache = torch.cat([keys.reshape(n_pages, -1), vals.reshape(n_pages, -1)], dim=1)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    seq = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(q_lens)])
    positions = torch.cat([torch.arange(c - n, c, dtype=torch.int32) for c, n in zip(ctx, q_lens)])
    meta = AttentionMeta(table.cuda(), i32(cu), i32(ctx), seq.cuda(), None, B, max(q_lens), max(ctx), page,
                         sum(1 for n in q_lens if n == 1))
    return cache.cuda().to(dtype).contiguous(), meta, positions.cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,vd,chunk,page", [(6, 3, 16, 24, 21, 8), (8, 2, 64, 32, 40, 16), (1, 1, 9, 7, 1, 8), (5, 5, 10, 11, None, 16),
                                                 (4, 1, 24, 8, 50, 8), (16, 4, 128, 64, 33, 32)])
def test_mixed_head_attention_over_pages(K, dtype, H, G, d, vd, chunk, page):
    """Portions of prompts beside single tokens; the first tokens of a sequence; queries on both sides of a chunk's edge
    and of a page's; pages below the chunk given back."""
    ctx, q_lens = (70, 45, 1, 130, 64), (70, 1, 1, 9, 2)
    ks = [rnd(c, G, d, seed=80 + i).to(dtype).double() for i, c in enumerate(ctx)]
    vs = [rnd(c, G, vd, seed=90 + i).to(dtype).double() for i, c in enumerate(ctx)]
    qs = [rnd(n, H, d, seed=100 + i).to(dtype).double() for i, n in enumerate(q_lens)]
    r1, r2 = torch.rand(H, generator=torch.Generator().manual_seed(1), dtype=F64) * 1.5, torch.rand(H, generator=torch.Generator().manual_seed(2), dtype=F64) + 0.1
    talk = torch.eye(H, dtype=F64) + 0.4 * rnd(H, H, seed=3)
    cache, meta, positions = flat_pages(ks, vs, q_lens, page, dtype, chunk)
    q = torch.cat(qs).reshape(sum(q_lens), H * d).to(dtype).cuda()
    for use_bias, use_talk in ((True, True), (False, True), (True, False)):
        got = K.talking_attention(q, cache, meta, positions, H, G, d, vd, 0.3, r1.float().cuda() if use_bias else None,
                                  r2.float().cuda() if use_bias else None, talk.float().cuda() if use_talk else None, chunk)
        at = 0
        for i, n in enumerate(q_lens):
            full_q = torch.zeros(ctx[i], H, d, dtype=F64)
            full_q[ctx[i] - n:] = qs[i]
            want = P.mixed_head_attention(full_q, ks[i], vs[i], 0.3, r1 if use_bias else torch.zeros(H, dtype=F64), r2,
                                          talk if use_talk else torch.eye(H, dtype=F64), chunk or 10 ** 9)[ctx[i] - n:]
            assert rel_err(got[at:at + n], want.reshape(n, -1)) < TOL[dtype], (i, use_bias, use_talk)
            at += n


@pytest.mark.parametrize("H,G,d,vd,chunk,page", [(8, 2, 64, 32, 40, 16), (16, 4, 128, 64, 133, 32), (4, 4, 32, 128, None, 8), (16, 1, 16, 16, 64, 16),
                                                 (8, 8, 48, 96, 97, 16), (2, 1, 128, 128, 31, 8), (12, 6, 64, 32, 70, 16)])
@pytest.mark.parametrize("path", ["tensor", "split", "plain"])
def test_every_build_of_the_mixed_head_attention_gives_the_plain_result(K, H, G, d, vd, chunk, page, path):
    """The tensor-core build (many tokens), the split-key build (few tokens behind many keys) and the plain kernel against
    the slow implementation: portions that start and end inside tiles, chunks and pages, single tokens among them, head
    groups of 1 to 16, key and value widths that differ."""
    dtype = torch.bfloat16
    ctx, q_lens = ((300, 171, 1, 260, 64), (150, 37, 1, 259, 2)) if path != "split" else ((300, 171, 1, 64), (3, 1, 1, 20))
    ks = [rnd(c, G, d, seed=180 + i).to(dtype).double() for i, c in enumerate(ctx)]
    vs = [rnd(c, G, vd, seed=190 + i).to(dtype).double() for i, c in enumerate(ctx)]
    qs = [rnd(n, H, d, seed=200 + i).to(dtype).double() for i, n in enumerate(q_lens)]
    r1, r2 = torch.rand(H, generator=torch.Generator().manual_seed(1), dtype=F64) * 1.5, torch.rand(H, generator=torch.Generator().manual_seed(2), dtype=F64) + 0.1
    talk = torch.eye(H, dtype=F64) + 0.4 * rnd(H, H, seed=3)
    cache, meta, positions = flat_pages(ks, vs, q_lens, page, dtype, chunk)
    q = torch.cat(qs).reshape(sum(q_lens), H * d).to(dtype).cuda()
    old = K.TALKING_MMA, K.TALKING_SPLIT
    K.TALKING_MMA, K.TALKING_SPLIT = path == "tensor", path == "split"
    try:
        for use_bias, use_talk in ((True, True), (False, False)):
            got = K.talking_attention(q, cache, meta, positions, H, G, d, vd, 0.3, r1.float().cuda() if use_bias else None,
                                      r2.float().cuda() if use_bias else None, talk.float().cuda() if use_talk else None, chunk)
            at = 0
            for i, n in enumerate(q_lens):
                full_q = torch.zeros(ctx[i], H, d, dtype=F64)
                full_q[ctx[i] - n:] = qs[i]
                want = P.mixed_head_attention(full_q, ks[i], vs[i], 0.3, r1 if use_bias else torch.zeros(H, dtype=F64), r2,
                                              talk if use_talk else torch.eye(H, dtype=F64), chunk or 10 ** 9)[ctx[i] - n:]
                assert rel_err(got[at:at + n], want.reshape(n, -1)) < TOL[dtype], (i, use_bias, use_talk)
                at += n
    finally:
        K.TALKING_MMA, K.TALKING_SPLIT = old


def test_a_large_batch_of_single_tokens_takes_the_split_keys(K):
    """Seventy sequences of unequal lengths, one token each: more tokens than the tensor-core build is preferred from, yet
    all of them single, so the keys are split (into fewer ranges than for a small batch); against the slow implementation."""
    H, G, d, vd, chunk, page, dtype = 4, 2, 32, 16, 90, 16, torch.bfloat16
    ctx = [3 + (37 * i) % 230 for i in range(70)]
    q_lens = [1] * 70
    ks = [rnd(c, G, d, seed=300 + i).to(dtype).double() for i, c in enumerate(ctx)]
    vs = [rnd(c, G, vd, seed=400 + i).to(dtype).double() for i, c in enumerate(ctx)]
    qs = [rnd(1, H, d, seed=500 + i).to(dtype).double() for i in range(70)]
    r1, r2 = torch.rand(H, generator=torch.Generator().manual_seed(1), dtype=F64) * 1.5, torch.rand(H, generator=torch.Generator().manual_seed(2), dtype=F64) + 0.1
    talk = torch.eye(H, dtype=F64) + 0.4 * rnd(H, H, seed=3)
    cache, meta, positions = flat_pages(ks, vs, q_lens, page, dtype, chunk)
    q = torch.cat(qs).reshape(70, H * d).to(dtype).cuda()
    got = K.talking_attention(q, cache, meta, positions, H, G, d, vd, 0.3, r1.float().cuda(), r2.float().cuda(), talk.float().cuda(), chunk)
    for i in range(70):
        full_q = torch.zeros(ctx[i], H, d, dtype=F64)
        full_q[-1:] = qs[i]
        want = P.mixed_head_attention(full_q, ks[i], vs[i], 0.3, r1, r2, talk, chunk)[-1:]
        assert rel_err(got[i:i + 1], want.reshape(1, -1)) < TOL[dtype], i


def test_a_planted_key_reaches_the_tensor_core_build(K):
    """As the planted key below, in a long portion: the key at the first position of the last query's chunk takes the whole
    weight, one position lower it is not seen."""
    H, G, d, vd, page, dtype, q_len = 8, 2, 32, 64, 16, torch.bfloat16, 200
    for chunk, ctx in ((320, 600), (250, 499), (48, 300)):
        start = ((ctx - 1) // chunk) * chunk
        v = rnd(ctx, G, vd, seed=5).to(dtype).double()
        for key in (start, start - 1, ctx - 1):
            k, q = torch.zeros(ctx, G, d, dtype=F64), torch.zeros(q_len, H, d, dtype=F64)
            k[key, :, 3], q[-1, :, 3] = 8.0, 8.0
            cache, meta, positions = flat_pages([k], [v], [q_len], page, dtype, chunk, seed=key)
            got = K.talking_attention(q.reshape(q_len, H * d).to(dtype).cuda(), cache, meta, positions, H, G, d, vd, 1.0, None, None, None, chunk)
            for h in range(H):
                want = v[key, h // 4] if key >= start else v[start:, h // 4].mean(0)
                assert float((got[-1, h * vd:(h + 1) * vd].double().cpu() - want).abs().max()) < 2e-2, (chunk, key, h)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_len", [1, 7])
def test_a_planted_key_at_the_edges_of_a_chunk(K, dtype, q_len):
    """One key matches the last query strongly, all others are zero.  At the first position of the query's chunk - also
    where that is the first slot of a page or the last slot of the page before - it takes the whole weight, hundreds of
    positions back; one position lower it is not seen at all (the weights are then even over the chunk)."""
    H, G, d, vd, page = 4, 2, 16, 8, 16
    for chunk, ctx in ((320, 600), (250, 499), (48, 100), (17, 300)):
        start = ((ctx - 1) // chunk) * chunk
        v = rnd(ctx, G, vd, seed=5).to(dtype).double()
        for key in (start, start - 1, ctx - 1, start + 1):
            k, q = torch.zeros(ctx, G, d, dtype=F64), torch.zeros(q_len, H, d, dtype=F64)
            k[key, :, 3], q[-1, :, 3] = 8.0, 8.0
            cache, meta, positions = flat_pages([k], [v], [q_len], page, dtype, chunk, seed=key)
            got = K.talking_attention(q.reshape(q_len, H * d).to(dtype).cuda(), cache, meta, positions, H, G, d, vd, 1.0, None, None, None, chunk)
            for h in range(H):
                want = v[key, h // 2] if key >= start else v[start:, h // 2].mean(0)
                assert float((got[-1, h * vd:(h + 1) * vd].double().cpu() - want).abs().max()) < (1e-4 if dtype == torch.float32 else 2e-2), (chunk, key, h)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_keys_values_and_queries_find_their_places(K, dtype):
    """q rounded, k as it is and v under its per-head norm in the token's slot; slot -1 writes nothing; nothing else is touched."""
    H, G, d, vd, page, n_pages, T = 6, 3, 16, 24, 8, 5, 7
    proj = rnd(T, H * d + G * (d + vd), seed=7, scale=2.0).float()
    slots = [0, 1, 17, 18, -1, 39, 8]
    tol = 1e-6 if dtype == torch.float32 else 5e-3
    for eps in (1e-5, None):
        cache = torch.full((n_pages, G * page * (d + vd)), 7.0, dtype=dtype).cuda()
        q = K.kv_prepare(proj.cuda(), i32(slots), cache, H, G, d, vd, eps, dtype)
        assert q.dtype == dtype and rel_err(q, proj[:, :H * d].double()) < tol
        keys = cache[:, :G * page * d].view(n_pages, G, page, d)
        vals = cache[:, G * page * d:].view(n_pages, G, page, vd)
        k_want = proj[:, H * d:H * d + G * d].double().view(T, G, d)
        v_want = proj[:, H * d + G * d:].double().view(T, G, vd)
        if eps is not None:
            v_want = P.rms(v_want, eps)
        for t, s in enumerate(slots):
            if s >= 0:
                assert rel_err(keys[s // page, :, s % page], k_want[t]) < tol and rel_err(vals[s // page, :, s % page], v_want[t]) < tol
        written = {s for s in slots if s >= 0}
        for s in range(n_pages * page):
            if s not in written:
                assert bool((keys[s // page, :, s % page] == 7.0).all()) and bool((vals[s // page, :, s % page] == 7.0).all())
        only_q = K.kv_prepare(proj.cuda(), None, None, H, G, d, vd, eps, dtype, write_kv=False)
        assert torch.equal(only_q, q)


# ---------------------------------------------------------------------------------------- the whole path
LENGTHS = {"a": (45, 170, 33, 81, 1, 138), "b": (90, 37, 300, 64, 151, 2)}
SCHEDULES = {"whole": TT.schedule_whole, "bulk_tail": TT.schedule_bulk_tail, "portions": TT.schedule_portions,
             "mixed": TT.schedule_mixed}
_cache = {}


def _reference(which):
    if which not in _cache:
        from rvllm_b200 import load_config
        folder = X.write_folder({"a": X.small_a, "b": X.small_b}[which](), seed=6, edit=X.lively)
        vocab = load_config(folder).vocab_size
        reqs = random_requests(vocab, LENGTHS[which], seed=4)
        _cache[which] = (folder, vocab, reqs, X.plain_logits(folder, reqs), X.plain_logits(folder, reqs, rounded=True))
    return _cache[which][:4]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("which", ["a", "b"])
def test_replay_matches_plain(tmp_path, which, schedule, dtype):
    from rvllm_b200.engine import trace as trace_mod
    folder, vocab, reqs, ref = _reference(which)
    trace = SCHEDULES[schedule](reqs)
    block = 8 if which == "a" else 16
    if schedule == "whole":                      # once per configuration as a user runs it: a process of its own
        TT.run_trace_tool(folder, dtype, trace, str(tmp_path), block)
    else:
        engine = trace_mod.build_engine(folder, dtype, trace.max_tokens, block, graphs=schedule == "bulk_tail")
        trace_mod.replay(engine, io.StringIO(trace.lines()), str(tmp_path), io.StringIO())
        engine.cache.check()
        assert not engine.cache.requests
    got = TT.read_logits(str(tmp_path), trace, vocab)
    what = f"{which}/{schedule}/{dtype}"
    if dtype == "float32":
        TT.compare(got, ref, 1e-4, what)
    else:
        TT.compare_bfloat16(got, ref, _cache[which][4], what)
        TT.compare(got, ref, 0.2, what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_odd_shapes_whole_and_mixed(tmp_path, dtype):
    """Sizes off every fast path (see tibepel_tools.odd_shapes), whole prompts and the mixed schedule."""
    from rvllm_b200 import load_config
    from rvllm_b200.engine import trace as trace_mod
    folder = X.write_folder(X.odd_shapes(), seed=8, edit=X.lively)
    vocab = load_config(folder).vocab_size
    reqs = random_requests(vocab, (70, 150, 9, 33, 130), seed=6)
    ref = X.plain_logits(folder, reqs)
    rounded = X.plain_logits(folder, reqs, rounded=True) if dtype == "bfloat16" else None
    for name, make in (("whole", TT.schedule_whole), ("mixed", TT.schedule_mixed)):
        out = tmp_path / name
        trace = make(reqs)
        engine = trace_mod.build_engine(folder, dtype, trace.max_tokens, 16)
        trace_mod.replay(engine, io.StringIO(trace.lines()), str(out), io.StringIO())
        engine.cache.check()
        got = TT.read_logits(str(out), trace, vocab)
        if dtype == "float32":
            TT.compare(got, ref, 1e-4, f"odd/{name}")
        else:
            TT.compare_bfloat16(got, ref, rounded, f"odd/{name}")
        del engine


def test_generation_through_the_entry_point():
    """Greedy tokens through LLM.generate and its scheduler (decode steps from CUDA graphs, prompts in portions,
    more requests than slots): float32 equals the plain implementation token for token; bfloat16 may differ only
    where the plain logits' two best lie closer together than its rounding."""
    from rvllm_b200 import LLM, SamplingParams
    folder, vocab, reqs, ref = _reference("b")
    cfg, w = X.read_folder(folder)
    prompts = [reqs["r1"], reqs["r5"], reqs["r3"], reqs["r0"][:50], reqs["r4"][:100]]
    for dtype in ("float32", "bfloat16"):
        llm = LLM(folder, dtype=dtype, block_size=16, num_blocks=40, max_model_len=256, max_num_seqs=3,
                  max_num_batched_tokens=48, max_prefill_chunk=33)
        assert llm.engine.model.graph_safe
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True))
        assert llm.engine.runner._graphs, "decode steps were not replayed from graphs"
        for p, o in zip(prompts, outs):
            got = o.outputs[0].token_ids
            ids = list(p)
            for tok in got:
                logits = P.forward(cfg, w, ids)[-1]
                top = torch.topk(logits, 2).values
                if dtype == "float32":
                    assert tok == int(logits.argmax())
                else:
                    assert float(top[0] - top[1]) / float(logits.abs().max()) <= 6e-2 or tok == int(logits.argmax())
                ids.append(tok)
        assert not llm.engine.cache.requests
        del llm


def test_long_decoding_over_many_chunks():
    """A short prompt, then 400 tokens one by one (graphs), over several chunks of both attention layers and with the
    recurrent states carried all the way: the logits equal those of the whole sequence."""
    from rvllm_b200.engine import trace as trace_mod
    from rvllm_b200.engine.step import StepEntry
    folder, vocab, reqs, ref = _reference("a")
    toks = random_requests(vocab, (420,), seed=9)["r0"]
    want = X.plain_logits(folder, {"x": toks})["x"]
    engine = trace_mod.build_engine(folder, "float32", 512, 8, graphs=True)
    engine.runner.step([StepEntry("x", toks[:20], [])])
    for i in range(20, 420):
        logits = engine.runner.step([StepEntry("x", toks[i:i + 1], [0])])
        if i % 21 in (0, 20) or i % 50 in (0, 49) or i == 419:
            assert rel_err(logits[0], want[i]) < 1e-4, i
