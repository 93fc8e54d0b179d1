"""The kernels and the whole path of the Tugodra design on the GPU, against the plain implementation
(plain_tugodra.py): every mechanism alone, then trace replay under the four schedules in both number formats,
generation through the entry point and its scheduler, and long decoding."""
import io
import math

import pytest
import torch

import plain_tugodra as P
import trace_tools as TT
import tugodra_tools as X
from gpu_tools import paged_setup, rel_err
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


def dev32(t):
    return t.float().cuda().contiguous()


# ---------------------------------------------------------------------------------------- norms and rows
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cols", [44, 45, 352, 4096 + 24])
def test_dynamic_tanh_alone_and_with_the_sum(K, dtype, cols):
    y, r = rnd(6, cols, seed=1, scale=3.0).float().double(), rnd(6, cols, seed=2).float().double()
    n1 = {"n": rnd(cols, seed=3) + 1.0, "n.b": rnd(cols, seed=4, scale=0.2), "n.alpha": torch.tensor(0.37, dtype=F64)}
    n2 = {"n": rnd(cols, seed=5) + 1.0, "n.b": rnd(cols, seed=6, scale=0.2), "n.alpha": torch.tensor(1.3, dtype=F64)}
    n1, n2 = ({k: v.float().double() for k, v in n.items()} for n in (n1, n2))
    as_dyt = lambda n: (dev32(n["n.alpha"].reshape(1)), dev32(n["n"]), dev32(n["n.b"]))
    out = K.dynamic_tanh(y.to(dtype).cuda(), *as_dyt(n1), out_dtype=dtype)
    assert out.dtype == dtype and rel_err(out, P.dynamic_tanh(y.to(dtype).double(), n1, "n")) < (2e-6 if dtype == torch.float32 else 5e-3)
    stream = r + P.dynamic_tanh(y, n1, "n")
    res = dev32(r)
    got, nxt = K.residual_dynamic_tanh(dev32(y), as_dyt(n1), res, as_dyt(n2), dtype)
    assert got is res and rel_err(got, stream) < 2e-6
    assert nxt.dtype == dtype and rel_err(nxt, P.dynamic_tanh(stream, n2, "n")) < (4e-6 if dtype == torch.float32 else 5e-3)
    got2, none = K.residual_dynamic_tanh(dev32(y), as_dyt(n1), dev32(r), None, None)
    assert none is None and rel_err(got2, stream) < 2e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scaled_rows_and_squared_relu(K, dtype):
    x = rnd(7, 93, seed=8).to(dtype)
    assert K.scale_rows(x.cuda(), 13.25).dtype == torch.float32 and rel_err(K.scale_rows(x.cuda(), 13.25), x.double() * 13.25) < 1e-6
    for cols in (77, 96, 2048 + 4):                           # rows off and on the four-column path
        u, s = rnd(5, cols, seed=9, scale=2.0).float(), torch.rand(5, generator=torch.Generator().manual_seed(2))
        assert rel_err(K.act_rows(u.cuda(), "relu2", dtype), torch.relu(u.double()) ** 2) < TOL[dtype] / 2
        assert rel_err(K.act_rows(u.cuda(), "relu2", dtype, row_scale=s.cuda()), torch.relu(u.double()) ** 2 * s.double()[:, None]) < TOL[dtype] / 2


# ---------------------------------------------------------------------------------------- queries and keys of the window attention
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("halves", [False, True])
@pytest.mark.parametrize("H,G,D,V,dims", [(6, 2, 24, 16, 16), (4, 4, 8, 12, 4), (3, 3, 10, 7, 6), (8, 2, 64, 64, 64), (6, 2, 6, 18, 2), (2, 1, 128, 256, 128)])
def test_rotation_unit_norm_and_cache_write(K, dtype, halves, H, G, D, V, dims):
    T, page, slot_dim, eps = 11, 8, max(D, V), 1e-5
    proj = rnd(T, H * D + G * (D + V) + H, seed=10, scale=2.0).float()
    pos = torch.tensor([0, 1, 2, 7, 8, 30, 31, 32, 500, 900, 1023], dtype=torch.int32)
    inv = torch.tensor([50.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    ang = torch.arange(1024, dtype=F64)[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    slots = torch.tensor([5, 6, 7, 16, 17, 40, 41, -1, 3, 2, 1], dtype=torch.int32)
    cache = torch.full((8, 2, G, page, slot_dim), 7.0, dtype=dtype).cuda()
    q, gate = K.qk_unit_prepare(proj.cuda(), eps, pos.cuda(), cos, sin, slots.cuda(), cache, H, G, D, V, slot_dim, dtype, halves=halves)
    turn = P.turn_halves if halves else P.turn_neighbours
    x = proj.double()
    want_q = P.unit_rms(turn(x[:, :H * D].view(T, H, D), pos, dims, 50.0), eps)
    want_k = P.unit_rms(turn(x[:, H * D:H * D + G * D].view(T, G, D), pos, dims, 50.0), eps)
    want_v = x[:, H * D + G * D:H * D + G * (D + V)].view(T, G, V)
    tol = 3e-6 if dtype == torch.float32 else 5e-3
    qv = q.view(T, H, slot_dim)
    assert rel_err(qv[:, :, :D], want_q) < tol and float(qv[:, :, D:].abs().max() if slot_dim > D else 0.0) == 0.0
    assert rel_err(gate, torch.sigmoid(x[:, -H:])) < 2e-6
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        kk, vv = cache[s // page, 0, :, s % page], cache[s // page, 1, :, s % page]
        assert rel_err(kk[:, :D], want_k[t]) < tol and rel_err(vv[:, :V], want_v[t]) < tol
        assert float(kk[:, D:].abs().max() if slot_dim > D else 0.0) == 0.0 and float(vv[:, V:].abs().max() if slot_dim > V else 0.0) == 0.0
    written = {s for s in slots.tolist() if s >= 0}
    untouched = [s for s in range(8 * page) if s not in written]
    assert all(float((cache[s // page, :, :, s % page] - 7.0).abs().max()) == 0.0 for s in untouched)     # slot -1 wrote nothing
    # a borrowing layer: queries and gates only
    only_q = torch.cat([proj[:, :H * D], proj[:, -H:]], dim=1).contiguous()
    q2, gate2 = K.qk_unit_prepare(only_q.cuda(), eps, pos.cuda(), cos, sin, None, None, H, G, D, V, slot_dim, dtype, halves=halves, write_kv=False)
    assert torch.equal(q2, q) and torch.equal(gate2, gate)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,page", [(64, 16), (24, 8), (128, 16)])
@pytest.mark.parametrize("window", [5, 40, 96, 700])
def test_one_key_at_the_window_edge(K, dtype, hd, page, window):
    """Unit-norm queries and keys with a large scale: the key that equals the query takes all the weight.  Planted at the last
    position the window still holds it is the result; one position lower it is not seen - for a decoded token, the last
    token of a portion, and both in one step, with the pages below the window given back."""
    H, G, ctx, scale = 4, 2, 900, 40.0 / hd ** 0.5
    unit = lambda v: v / torch.sqrt((v * v).mean(-1, keepdim=True))
    for q_lens, ctxs in (((1,), (ctx,)), ((70,), (ctx,)), ((1, 33), (ctx, 850)), ((1, 1, 1), (ctx, 64, 3))):
        for inside in (True, False):
            keys = [unit(rnd(c, G, hd, seed=50 + i)).to(dtype).double() for i, c in enumerate(ctxs)]
            vals = [rnd(c, G, hd, seed=60 + i).to(dtype).double() for i, c in enumerate(ctxs)]
            T = sum(q_lens)
            q = unit(rnd(T, H, hd, seed=70)).to(dtype)
            at = ctxs[0] - window + (0 if inside else -1)          # the oldest key the first sequence's last query sees, or the one before
            probe = q_lens[0] - 1
            if at >= 0:
                keys[0][at, 1] = unit(q[probe, 3].double()).to(dtype).double()      # head 3 reads kv head 1
            gate = torch.rand(T, H, generator=torch.Generator().manual_seed(3))
            cache, meta = paged_setup(keys, vals, q_lens, page, dtype, seed=window, window=window)
            got = K.paged_attention(q.view(T, H * hd).cuda(), cache, meta, H, G, hd, scale, window, gate=gate.cuda()).view(T, H, hd)
            want, t = [], 0
            for kk, vv, n in zip(keys, vals, q_lens):
                c = kk.shape[0]
                for i in range(n):
                    p_ = c - n + i
                    lo = max(0, p_ - window + 1)
                    rows = []
                    for h in range(H):
                        s = (kk[lo:p_ + 1, h // 2] @ q[t, h].double()) * scale
                        rows.append(torch.softmax(s, 0) @ vv[lo:p_ + 1, h // 2] * gate[t, h].double())
                    want.append(torch.stack(rows))
                    t += 1
            want = torch.stack(want)
            assert rel_err(got, want) < (3e-5 if dtype == torch.float32 else 2e-2), (q_lens, inside)
            if at >= 0:
                hit = rel_err(got[probe, 3], vals[0][at, 1] * gate[probe, 3].double()) < (1e-3 if dtype == torch.float32 else 2e-2)
                assert hit == inside, (q_lens, inside)
    K.raise_on_abort()


# ---------------------------------------------------------------------------------------- latent attention: pairs and sink
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Rd,dims,R", [(3, 24, 16, 16, 40), (4, 8, 12, 8, 20), (1, 9, 6, 6, 35), (6, 32, 32, 32, 128)])
def test_latent_rows_with_half_split_pairs(K, dtype, H, D, Rd, dims, R):
    T, page, eps = 9, 8, 1e-5
    proj = rnd(T, H * (D + Rd) + R + Rd, seed=11, scale=2.0).float()
    gamma = (rnd(R, seed=12) + 1.0).to(dtype)
    pos = torch.tensor([0, 1, 5, 8, 31, 32, 100, 700, 1023], dtype=torch.int32)
    inv = torch.tensor([10000.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    ang = torch.arange(1024, dtype=F64)[:, None] * inv[None, :]
    slots = torch.tensor([0, 1, 2, 9, 10, -1, 30, 31, 17], dtype=torch.int32)
    cache = torch.full((4, 1, 1, page, R + Rd), 7.0, dtype=dtype).cuda()
    q_plain, q_row, gate = K.latent_prepare(proj.cuda(), gamma.cuda(), eps, pos.cuda(), torch.cos(ang).float().cuda(),
                                            torch.sin(ang).float().cuda(), slots.cuda(), cache, H, D, Rd, R, dtype, with_gate=False, halves=True)
    assert gate is None
    x = proj.double()
    q = x[:, :H * (D + Rd)].view(T, H, D + Rd)
    tol = 3e-6 if dtype == torch.float32 else 5e-3
    assert rel_err(q_plain, q[:, :, :D]) < tol and rel_err(q_row[:, :, R:], P.turn_halves(q[:, :, D:], pos, dims, 10000.0)) < tol
    c = P.unit_rms(x[:, H * (D + Rd):H * (D + Rd) + R], eps) * gamma.double()
    r = P.turn_halves(x[:, H * (D + Rd) + R:], pos, dims, 10000.0)
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            assert rel_err(cache[s // page, 0, 0, s % page], torch.cat([c[t], r[t]])) < tol
    assert float((cache[3, 0, 0, 5] - 7.0).abs().max()) == 0.0          # slot -1 wrote nothing, a free slot stays


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,row,vd,page", [(6, 160, 128, 16), (3, 56, 40, 8), (4, 96, 64, 16), (1, 300, 260, 16), (5, 64, 48, 32)])
@pytest.mark.parametrize("q_lens,ctx", [((1, 1, 1), (257, 64, 1)), ((70, 5), (70, 133)), ((1, 40, 1, 2), (100, 300, 17, 2))])
def test_latent_attention_with_a_sink(K, dtype, H, row, vd, page, q_lens, ctx):
    """exp(sink) joins the denominator, in every build of the kernel (tcgen05 for portions, mma.sync, plain): decoded tokens
    with split keys, portions behind a prefix, both in one step; a first token whose only key competes with its sink."""
    from test_vipelix_gpu import latent_pages
    rows = [rnd(c, row, seed=20 + i).to(dtype).double() for i, c in enumerate(ctx)]
    T = sum(q_lens)
    q = rnd(T, H, row, seed=30, scale=1.5).to(dtype)
    sink = torch.linspace(-2.0, 4.0, H)
    cache, meta = latent_pages(rows, q_lens, page, dtype)

    def plain():
        out, t = [], 0
        for rr, n in zip(rows, q_lens):
            c = rr.shape[0]
            for i in range(n):
                s = q[t].double() @ rr[:c - n + i + 1].T * 0.11
                p = torch.softmax(torch.cat([s, sink.double()[:, None]], dim=1), -1)[:, :-1]
                out.append(p @ rr[:c - n + i + 1, :vd])
                t += 1
        return torch.stack(out)

    want = plain()
    got = K.latent_attention(q.cuda(), cache, meta, H, row, vd, 0.11, sinks=sink.cuda())
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    assert got.shape == (T, H, vd) and rel_err(got, want) < tol
    if dtype == torch.bfloat16 and row <= 256:
        K.LATENT_TCGEN05 = False
        try:
            flash = K.latent_attention(q.cuda(), cache, meta, H, row, vd, 0.11, sinks=sink.cuda())
            K.LATENT_FLASH = False
            slow = K.latent_attention(q.cuda(), cache, meta, H, row, vd, 0.11, sinks=sink.cuda())
        finally:
            K.LATENT_FLASH = K.LATENT_TCGEN05 = True
        assert rel_err(flash, want) < tol and rel_err(slow, want) < tol
        K.raise_on_abort()


# ---------------------------------------------------------------------------------------- the matrix memory
def mlstm_weights(width, H, D, V, seed, lively=True):
    w = {"q": rnd(H * D, width, seed=seed), "k": rnd(H * D, width, seed=seed + 1), "v": rnd(H * V, width, seed=seed + 2),
         "g": rnd(H * V, width, seed=seed + 3), "i": rnd(H, width, seed=seed + 4, scale=1.5 if lively else 0.1),
         "f": rnd(H, width, seed=seed + 5, scale=1.5 if lively else 0.1), "i.b": rnd(H, seed=seed + 6), "f.b": rnd(H, seed=seed + 7) + 2.0,
         "norm": rnd(H * V, seed=seed + 8) + 1.0, "o": torch.eye(H * V, dtype=F64)}
    return {k: v.float().double() for k, v in w.items()}


def run_mlstm(K, w, hs, cuts, slots, H, D, V, cap, eps, state, dtype=torch.float32):
    """hs: per sequence [T_s, width]; cuts: per step, per sequence, how many tokens it brings.  Returns per sequence the
    outputs [T_s, H * V] of the kernels, the state rows carried from step to step."""
    done = [0] * len(hs)
    outs = [[] for _ in hs]
    wcat = torch.cat([w["q"], w["k"], w["v"], w["g"], w["i"], w["f"]], dim=0)
    for step in cuts:
        parts, cu, live = [], [0], []
        for s, n in enumerate(step):
            if n:
                parts.append(hs[s][done[s]:done[s] + n])
                cu.append(cu[-1] + n)
                live.append(s)
        proj = (torch.cat(parts) @ wcat.T).float().cuda().contiguous()
        seq = torch.cat([torch.full((cu[i + 1] - cu[i],), i, dtype=torch.int32) for i in range(len(live))]).cuda()
        cu_t = torch.tensor(cu, dtype=torch.int32).cuda()
        sl = torch.tensor([slots[s] for s in live], dtype=torch.int32).cuda()
        gate_col = 2 * H * D + H * V
        raw, top = K.mlstm_scan(proj, gate_col + H * V, gate_col + H * V + H, dev32(w["i.b"]), dev32(w["f.b"]), cu_t, sl, state, H, D, V, cap)
        y = K.mlstm_output(raw, top, dev32(w["norm"]), eps, 1e-6, proj, gate_col, H, D, V, dtype, seq, cu_t, sl, state)
        for i, s in enumerate(live):
            outs[s].append(y[cu[i]:cu[i + 1]].float().cpu())
            done[s] += step[s]
    return [torch.cat(o) if o else None for o in outs]


@pytest.mark.parametrize("H,D,V", [(3, 12, 20), (1, 5, 3), (5, 40, 9), (2, 32, 64), (2, 128, 128), (1, 200, 70), (4, 64, 31)])
def test_matrix_memory_in_portions_against_the_whole_sequence(K, H, D, V):
    width, cap, eps = 24, 9.0, 1e-5
    w = mlstm_weights(width, H, D, V, seed=100 + D)
    m = {"heads": H, "dim": D, "vdim": V, "gate_cap": cap}
    hs = [rnd(61, width, seed=1).float().double(), rnd(40, width, seed=2).float().double(), rnd(5, width, seed=3).float().double()]
    want = [P.mlstm(h, w, "", m, eps) for h in hs]
    state = torch.zeros((4, H * D * (V + 1) + H), dtype=torch.float32, device="cuda")
    state[1].fill_(9.0)                                       # a slot nobody holds stays as it is
    # sequence 2 sits in no slot (a padding row): nothing is read or written for it
    cuts = [(17, 1, 5), (2, 16, 0), (1, 1, 0), (33, 0, 0), (1, 20, 0), (7, 2, 0)]
    got = run_mlstm(K, w, hs, cuts, [2, 0, -1], H, D, V, cap, eps, state)
    assert rel_err(got[0], want[0]) < 3e-5 and rel_err(got[1], want[1]) < 3e-5
    assert float((state[1] - 9.0).abs().max()) == 0.0 and float(state[3].abs().max()) == 0.0
    # token by token from an empty state gives the same
    state.zero_()
    single = run_mlstm(K, w, hs[:1], [(1,)] * 61, [3], H, D, V, cap, eps, state)
    assert rel_err(single[0], want[0]) < 3e-5
    # what the state row holds is the memory, its normaliser in the last column, and the running maximum
    top = 0.0
    li = cap * torch.tanh((hs[0] @ w["i"].T + w["i.b"]) / cap)
    lf = torch.nn.functional.logsigmoid(cap * torch.tanh((hs[0] @ w["f"].T + w["f.b"]) / cap))
    for t in range(61):
        top = max(float(lf[t, 0]) + top, float(li[t, 0]))
    assert abs(float(state[3, H * D * (V + 1)]) - top) < 1e-4 * max(1.0, abs(top))


def test_matrix_memory_keeps_a_value_over_a_long_stretch(K):
    """One token writes with a wide-open input gate, every later one with a closed input gate and a forget gate near one:
    hundreds of tokens later the memory still answers with that token's value - in one portion, and decoded one by one."""
    H, D, V, width, cap, eps, T = 2, 16, 24, 20, 15.0, 1e-6, 400
    w = mlstm_weights(width, H, D, V, seed=7)
    for name in ("i", "f"):
        w[name] = torch.zeros_like(w[name])
    w["i"][:, 0], w["i.b"] = 30.0, torch.full((H,), -15.0, dtype=F64)          # input 0 of a token opens its input gate
    w["f.b"] = torch.full((H,), 15.0, dtype=F64)
    h = rnd(T, width, seed=8).float().double()
    h[:, 0] = 0.0
    h[3, 0] = 1.0
    m = {"heads": H, "dim": D, "vdim": V, "gate_cap": cap}
    want = P.mlstm(h, w, "", m, eps)
    v3 = (h[3] @ w["v"].T).view(H, V)
    direction = P.unit_rms(want[-1].view(H, V) / (w["norm"].view(H, V) * torch.sigmoid(h[-1] @ w["g"].T).view(H, V)), 0.0)
    assert float((direction.abs() - P.unit_rms(v3, 0.0).abs()).abs().max()) < 1e-3          # the oracle itself remembers token 3
    state = torch.zeros((1, H * D * (V + 1) + H), dtype=torch.float32, device="cuda")
    whole = run_mlstm(K, w, [h], [(T,)], [0], H, D, V, cap, eps, state)[0]
    state.zero_()
    decoded = run_mlstm(K, w, [h], [(10,)] + [(1,)] * (T - 10), [0], H, D, V, cap, eps, state)[0]
    assert rel_err(whole, want) < 1e-4 and rel_err(decoded, want) < 1e-4


# ---------------------------------------------------------------------------------------- router and experts
@pytest.mark.parametrize("E,top,groups,keep", [(12, 4, 3, 2), (6, 2, 3, 2), (4, 1, 1, 1), (4, 3, 4, 3), (8, 4, 2, 1), (64, 6, 8, 3), (40, 40, 1, 1), (3, 3, 3, 3)])
def test_router_choice_and_weights(K, E, top, groups, keep):
    T = 70
    logits = rnd(T, E + 1, seed=E, scale=2.5).float()
    corr = rnd(E, seed=top, scale=0.5).float()
    w = {"router": torch.eye(E, dtype=F64), "correction": corr.double()}
    chosen, weights, gate = K.moe_route_top(logits.cuda(), corr.cuda(), E, top, groups, keep, 1e-20, shared_gate=True)
    want_c, want_w = P.route(logits[:, :E].double(), w, "", {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}})
    assert torch.equal(chosen.cpu().sort(-1).values.long(), want_c.sort(-1).values)
    order_got, order_want = chosen.cpu().long().argsort(-1), want_c.argsort(-1)
    assert rel_err(weights.cpu().gather(1, order_got), want_w.gather(1, order_want)) < 1e-5
    assert rel_err(gate, torch.sigmoid(logits[:, E].double())) < 1e-6
    chosen2, weights2, none = K.moe_route_top(logits[:, :E].contiguous().cuda(), corr.cuda(), E, top, groups, keep, 1e-20)
    assert none is None and torch.equal(chosen2, chosen) and torch.equal(weights2, weights)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,width,ff,E,top", [(1, 48, 24, 5, 2), (9, 44, 9, 4, 4), (70, 384, 88, 12, 3), (300, 64, 40, 3, 1), (260, 192, 96, 12, 4),
                                              (130, 44, 9, 6, 2)])
def test_squared_relu_experts_with_weights(K, dtype, T, width, ff, E, top):
    """Few tokens (weights streamed per token) and many (sorted by expert, grouped products), with a weight per (token,
    slot) and something to add to."""
    x = rnd(T, width, seed=1).to(dtype)
    up, down = rnd(E, ff, width, seed=2, scale=width ** -0.5).to(dtype), rnd(E, width, ff, seed=3, scale=ff ** -0.5).to(dtype)
    g = torch.Generator().manual_seed(4)
    chosen = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if T >= 128:
        chosen[: T // 2] = chosen[0]                           # one expert gets many blocks
    weights = torch.rand(T, top, generator=g)
    add = rnd(T, width, seed=5).float()
    got = K.moe_experts(x.cuda(), chosen.cuda(), up.cuda(), down.cuda(), 1.0, add=add.cuda(), out_dtype=torch.float32, weights=weights.cuda(),
                        activation="relu2")
    want = add.double().clone()
    for t in range(T):
        for j, e in enumerate(chosen[t].tolist()):
            a = torch.relu(up[e].double() @ x[t].double()) ** 2
            want[t] += weights[t, j].double() * (down[e].double() @ a)
    assert got.dtype == torch.float32 and rel_err(got, want) < TOL[dtype]
    K.raise_on_abort()


# ---------------------------------------------------------------------------------------- whole models
LENGTHS = {"a": (45, 170, 33, 81, 1, 138), "b": (90, 37, 300, 64, 151, 2)}
SCHEDULES = {"whole": TT.schedule_whole, "bulk_tail": TT.schedule_bulk_tail, "portions": TT.schedule_portions,
             "mixed": TT.schedule_mixed}
_cache = {}


def _reference(which):
    if which not in _cache:
        from rvllm_b200 import load_config
        folder = X.write_folder({"a": X.small_a, "b": X.small_b}[which](), seed=5, edit=X.lively)
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_odd_shapes_whole_and_mixed(tmp_path, dtype):
    """Sizes off every fast path (see tugodra_tools.odd_shapes), whole prompts and the mixed schedule."""
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
            if dtype == "float32":
                assert got == P.greedy(cfg, w, p, 20)
            else:
                ids = list(p)
                for tok in got:
                    logits = P.forward(cfg, w, ids)[-1]
                    top = torch.topk(logits, 2).values
                    assert float(top[0] - top[1]) / float(logits.abs().max()) <= 6e-2 or tok == int(logits.argmax())
                    ids.append(tok)
        assert not llm.engine.cache.requests
        del llm


def test_long_decoding_past_every_window():
    """A short prompt, then 400 tokens one by one (graphs): windows pass over decoded tokens, window pages come back, the
    matrix memories run on; the logits equal those of the whole sequence."""
    from rvllm_b200.engine import trace as trace_mod
    from rvllm_b200.engine.step import StepEntry
    folder, vocab, reqs, ref = _reference("a")
    toks = random_requests(vocab, (420,), seed=9)["r0"]
    want = X.plain_logits(folder, {"x": toks})["x"]
    engine = trace_mod.build_engine(folder, "float32", 512, 8, graphs=True)
    engine.runner.step([StepEntry("x", toks[:20], [])])
    for i in range(20, 420):
        logits = engine.runner.step([StepEntry("x", toks[i:i + 1], [0])])
        if i % 57 == 0 or i == 419:
            assert rel_err(logits[0], want[i]) < 1e-4, i
    assert engine.runner._graphs
