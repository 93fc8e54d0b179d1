"""The Tugodra design on the engine's host side, without a GPU: configuration, tensor names, the plain mechanisms
themselves, and the real step function, cache manager, scheduler, trace replay and entry point driven with the torch
stand-ins for the kernels (emulated_kernels.py) against the plain implementation (plain_tugodra.py).  What is checked here is
the bookkeeping - a cache shared by a lending and a borrowing layer and kept as long as the wider window needs, window pages
that come back while a request runs, state rows that start at zero, pages and slots used again, portions cut anywhere; the
kernels themselves are checked by the GPU tests."""
import io
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_tugodra as P
import trace_tools as TT
import tugodra_tools as X
from emulated_kernels import EmulatedKernels
from model_tools import random_requests

from rvllm_b200 import ConfigError, LLM, SamplingParams, config_from_dict, kernels as kernel_pkg, load_config
from rvllm_b200.engine import trace as trace_mod
from rvllm_b200.engine.step import StepEntry
from rvllm_b200.models.decoder import DecoderModel, expected_tensors
from rvllm_b200.parts.base import KvCacheNeed, StateNeed


@pytest.fixture
def emulated():
    kernel_pkg.set_library(EmulatedKernels())
    yield
    kernel_pkg.set_library(None)


# ---------------------------------------------------------------------------------------- configuration
def test_config_round_trip_and_spec():
    cfg = config_from_dict(X.small_a())
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.to_spec()
    assert spec.residual_dtype == "float32" and spec.lm_head_name == "head" and not spec.validate()
    assert [h.kind for h in spec.embedding_hooks] == ["embedding_scale"] and spec.embedding_hooks[0].params["scale"] == 5.5
    # a borrowing layer runs on its lender's cache slot and writes nothing
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.run_order] == \
        [(0, 0, True), (1, 1, True), (2, 2, True), (3, 3, True), (4, 1, False), (5, 3, False), (6, 6, True), (7, 7, True)]
    shapes = {n: ts.shape for n, ts in expected_tensors(spec).items()}
    assert shapes["head"] == (131, 48) and shapes["final.norm"] == (48,) and shapes["final.norm.alpha"] == () and shapes["l3.norm1b.b"] == (48,)
    assert shapes["l0.mix.q"] == (36, 48) and shapes["l0.mix.v"] == (60, 48) and shapes["l0.mix.g"] == (60, 48) and shapes["l0.mix.i"] == (3, 48)
    assert shapes["l0.mix.f.b"] == (3,) and shapes["l0.mix.norm"] == (60,)
    assert shapes["l1.mix.k"] == (48, 48) and shapes["l1.mix.v"] == (32, 48) and shapes["l1.mix.g"] == (6, 48) and shapes["l1.mix.o"] == (48, 96)
    assert "l4.mix.k" not in shapes and "l4.mix.v" not in shapes and shapes["l4.mix.q"] == (144, 48)
    assert shapes["l2.mix.dkv"] == (56, 48) and shapes["l2.mix.sink"] == (3,) and "l2.mix.g" not in shapes
    assert shapes["l0.mlp.router"] == (6, 48) and shapes["l0.mlp.correction"] == (6,) and shapes["l0.mlp.shared.sg"] == (1, 48)
    assert shapes["l0.mlp.e5.down"] == (48, 24) and "l0.mlp.e6.up" not in shapes and "l1.mlp.shared.up" not in shapes
    assert "l3.norm2" not in shapes and "l3.mlp.router" not in shapes
    needs = DecoderModel(spec).cache_needs()
    # the lender's cache keeps what the wider of the two windows needs; a slot is as wide as the larger of key and value
    assert needs[1] == KvCacheNeed(2, 24, 29) and needs[3] == KvCacheNeed(4, 12, None)
    assert needs[2] == KvCacheNeed(1, 56, None, planes=1) and needs[0] == StateNeed((3 * 12 * 21 + 3,), "float32")
    assert sorted(needs) == [0, 1, 2, 3, 6, 7]
    kinds = [spec.layers[i].parts["mixer"].params.get("pairs") for i in (1, 2)]
    assert kinds == ["neighbours", "halves"]


def test_config_errors_are_collected():
    bad = X.small_a()
    bad["layers"][4]["mixer"]["kv_from"] = 2                 # not an attention layer
    bad["layers"][5]["mixer"]["heads"] = 8                   # differs from its lender
    bad["layers"][0]["mlp"]["router"]["groups"] = {"count": 4, "keep": 2}      # 6 experts in 4 groups
    bad["layers"][2]["mixer"]["rot"]["dims"] = 18            # beyond the rotated block
    del bad["embedding"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    text = str(e.value)
    for piece in ("layers[4]", "layers[5]", "layers[0]", "rot.dims", "embedding"):
        assert piece in text, (piece, text)
    chain = X.small_a()
    chain["layers"][5]["mixer"]["kv_from"] = 4               # a borrower lends nothing
    with pytest.raises(ConfigError):
        config_from_dict(chain)


# ---------------------------------------------------------------------------------------- the plain mechanisms
def test_plain_dynamic_tanh_and_rotations():
    w = {"n": torch.tensor([2.0, -1.0], dtype=torch.float64), "n.b": torch.tensor([0.5, 0.25], dtype=torch.float64),
         "n.alpha": torch.tensor(0.3, dtype=torch.float64)}
    x = torch.tensor([[1.0, -4.0]], dtype=torch.float64)
    want = torch.tensor([[2.0 * math.tanh(0.3) + 0.5, -1.0 * math.tanh(-1.2) + 0.25]], dtype=torch.float64)
    assert torch.allclose(P.dynamic_tanh(x, w, "n"), want)
    g = torch.Generator().manual_seed(0)
    v = torch.randn(5, 2, 8, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 3, 4, 9, 100])
    for turn, pair in ((P.turn_neighbours, (0, 1)), (P.turn_halves, (0, 3))):
        out = turn(v, pos, 6, 50.0)
        assert torch.equal(out[0], v[0]) and torch.equal(out[..., 6:], v[..., 6:])        # position 0 and the tail stay
        a, b = pair
        ang = 3.0                                                                          # pair 0 turns by the position itself
        assert torch.allclose(out[1, 0, a], v[1, 0, a] * math.cos(ang) - v[1, 0, b] * math.sin(ang))
        assert torch.allclose(out[1, 0, b], v[1, 0, b] * math.cos(ang) + v[1, 0, a] * math.sin(ang))
        # a score depends on the distance only
        q, k = torch.randn(1, 1, 8, generator=g, dtype=torch.float64), torch.randn(1, 1, 8, generator=g, dtype=torch.float64)
        s1 = (turn(q, torch.tensor([7]), 6, 50.0) * turn(k, torch.tensor([2]), 6, 50.0)).sum()
        s2 = (turn(q, torch.tensor([45]), 6, 50.0) * turn(k, torch.tensor([40]), 6, 50.0)).sum()
        assert torch.allclose(s1, s2)
    assert not torch.allclose(P.turn_neighbours(v, pos, 6, 50.0), P.turn_halves(v, pos, 6, 50.0))


def _attention_weights(T=40, width=16, m=None, seed=1):
    g = torch.Generator().manual_seed(seed)
    m = m or {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.7, "mask": {"size": 9}, "rot": {"dims": 4, "base": 20.0}}
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"q": rnd(m["heads"] * m["dim"], width), "k": rnd(m["kv_heads"] * m["dim"], width), "v": rnd(m["kv_heads"] * m["vdim"], width),
         "g": rnd(m["heads"], width), "o": rnd(width, m["heads"] * m["vdim"])}
    return m, w, rnd(T, width)


def test_plain_window_edge_and_unit_norm():
    """A query sees itself and the window - 1 keys before it: changing the input of a token just outside changes nothing,
    just inside it does.  Scaling a token's input leaves its key unchanged (unit norm) but not its value."""
    m, w, h = _attention_weights()
    pos = torch.arange(h.shape[0])
    run = lambda hh: P.window_attention(hh, w, "", m, 1e-6, pos, *P.window_keys(hh, w, "", m, 1e-6, pos))
    base = run(h)
    outside, inside = h.clone(), h.clone()
    outside[30 - 9] += 1.0
    inside[30 - 8] += 1.0
    assert torch.allclose(run(outside)[30], base[30], atol=1e-12) and not torch.allclose(run(inside)[30], base[30], atol=1e-6)
    assert not torch.allclose(run(outside)[29], base[29], atol=1e-6)
    k1, v1 = P.window_keys(h, w, "", m, 0.0, pos)
    k2, v2 = P.window_keys(3.0 * h, w, "", m, 0.0, pos)
    assert torch.allclose(k1, k2) and torch.allclose(3.0 * v1, v2)
    assert torch.allclose((k1 * k1).mean(-1), torch.ones_like(k1[..., 0]))
    # a borrowing layer: other queries and window, the lender's keys and values
    m2 = dict(m, scale=0.2, mask={"size": 20})
    keys, values = P.window_keys(h, w, "", m, 1e-6, pos)
    far = h.clone()
    far[30 - 15] += 1.0                                       # outside the lender's window, inside the borrower's
    k_far, v_far = P.window_keys(far, w, "", m, 1e-6, pos)
    assert not torch.allclose(P.window_attention(h, w, "", m2, 1e-6, pos, k_far, v_far)[30],
                              P.window_attention(h, w, "", m2, 1e-6, pos, keys, values)[30], atol=1e-6)


def test_plain_latent_sink_and_absorbed_form():
    g = torch.Generator().manual_seed(3)
    T, width, m = 11, 20, {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 7, "scale": 0.4, "rot": {"dims": 4, "base": 30.0}}
    H, D, Rd, V, R = 3, 6, 4, 5, 7
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"q": rnd(H * (D + Rd), width), "dkv": rnd(R + Rd, width), "dkv.norm": rnd(R), "uk": rnd(H * D, R), "uv": rnd(H * V, R),
         "sink": torch.tensor([0.5, -1.0, 2.0], dtype=torch.float64), "o": rnd(width, H * V)}
    h, pos = rnd(T, width), torch.arange(T)
    want = P.latent_attention(h, w, "", m, 1e-5, pos)
    q = (h @ w["q"].T).view(T, H, D + Rd)
    down = h @ w["dkv"].T
    row = torch.cat([P.unit_rms(down[:, :R], 1e-5) * w["dkv.norm"], P.turn_halves(down[:, R:], pos, 4, 30.0)], dim=1)   # what is cached
    outs = []
    for i in range(H):
        qi = torch.cat([q[:, i, :D] @ w["uk"][i * D:(i + 1) * D], P.turn_halves(q[:, i, D:], pos, 4, 30.0)], dim=1)
        s = (qi @ row.T * 0.4).masked_fill(pos[None, :] > pos[:, None], float("-inf"))
        e = torch.exp(s)
        p = e / (e.sum(-1, keepdim=True) + math.exp(float(w["sink"][i])))
        outs.append((p @ row[:, :R]) @ w["uv"][i * V:(i + 1) * V].T)
    assert torch.allclose(torch.cat(outs, 1) @ w["o"].T, want, atol=1e-10)
    # the sink takes weight and gives nothing: a huge one empties the result, a tiny one is plain softmax
    assert float(P.latent_attention(h, dict(w, sink=torch.full((3,), 600.0, dtype=torch.float64)), "", m, 1e-5, pos).abs().max()) < 1e-12
    none = P.latent_attention(h, dict(w, sink=torch.full((3,), -800.0, dtype=torch.float64)), "", m, 1e-5, pos)
    first = torch.cat([row[0, :R] @ w["uv"][i * V:(i + 1) * V].T for i in range(H)]) @ w["o"].T      # the first token sees itself only
    assert torch.allclose(none[0], first, atol=1e-10)


def test_plain_mlstm_against_the_unstabilised_sum():
    """With small gates the memory can be written without the running maximum: C_t = sum_j exp(i_j + sum_{l > j} f_l) k_j v_j^T,
    and the result is C^T q / (max(|n . q|, 1) + 1e-6 exp(m)) up to the factor exp(-m) on numerator and bound."""
    g = torch.Generator().manual_seed(5)
    T, width, m = 9, 10, {"heads": 2, "dim": 4, "vdim": 3, "gate_cap": 5.0}
    H, D, V = 2, 4, 3
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = {"q": rnd(H * D, width), "k": rnd(H * D, width), "v": rnd(H * V, width), "g": rnd(H * V, width), "i": 0.3 * rnd(H, width),
         "f": 0.3 * rnd(H, width), "i.b": rnd(H), "f.b": rnd(H), "norm": rnd(H * V), "o": torch.eye(H * V, dtype=torch.float64)}
    h = rnd(T, width)
    got = P.mlstm(h, w, "", m, 1e-6)
    q = (h @ w["q"].T).view(T, H, D) / 2.0
    k, v = (h @ w["k"].T).view(T, H, D), (h @ w["v"].T).view(T, H, V)
    li = 5.0 * torch.tanh((h @ w["i"].T + w["i.b"]) / 5.0)
    lf = torch.nn.functional.logsigmoid(5.0 * torch.tanh((h @ w["f"].T + w["f.b"]) / 5.0))
    out = torch.zeros(T, H, V, dtype=torch.float64)
    for i in range(H):
        top = 0.0
        for t in range(T):
            top = max(float(lf[t, i]) + top, float(li[t, i]))
            C = sum(math.exp(float(li[j, i] + lf[j + 1:t + 1, i].sum())) * torch.outer(k[j, i], v[j, i]) for j in range(t + 1))
            n = sum(math.exp(float(li[j, i] + lf[j + 1:t + 1, i].sum())) * k[j, i] for j in range(t + 1))
            out[t, i] = (C.T @ q[t, i]) / (max(abs(float(n @ q[t, i])), 1.0) + 1e-6 * math.exp(top))
    want = (P.unit_rms(out, 1e-6).reshape(T, H * V) * w["norm"]) * torch.sigmoid(h @ w["g"].T)
    assert torch.allclose(got, want, atol=1e-6)
    # the running maximum starts at 0: a first token whose gates are very negative is divided by exp(-0) = 1, not by |n . q|
    w2 = dict(w, **{"i.b": torch.full((H,), -30.0, dtype=torch.float64), "i": torch.zeros(H, width, dtype=torch.float64)})
    m2 = dict(m, gate_cap=40.0)
    raw = P.mlstm(h[:1], dict(w2, norm=torch.ones(H * V, dtype=torch.float64)), "", m2, 0.0)
    assert torch.isfinite(raw).all()


def test_plain_router_groups_and_weights():
    width = 4
    w = {"router": torch.zeros(8, width, dtype=torch.float64), "correction": torch.zeros(8, dtype=torch.float64)}
    h = torch.ones(1, width, dtype=torch.float64)
    logits = torch.tensor([3.0, -3.0, 0.5, 0.4, 2.0, 1.9, -1.0, 2.5], dtype=torch.float64)
    w["router"][:, 0] = logits
    r = {"experts": 8, "top": 3, "groups": {"count": 4, "keep": 2}}
    # groups (0,1) (2,3) (4,5) (6,7): sums of two sigmoids; the best are (4,5) and (6,7)?  s = .953 .047 | .622 .599 | .881 .870 | .269 .924
    chosen, weights = P.route(h, w, "", r)
    s = torch.sigmoid(logits)
    assert sorted(chosen[0].tolist()) == [4, 5, 2] or sorted(chosen[0].tolist()) == [2, 4, 5]      # groups (4,5) and (2,3): expert 0 and 7 are shut out
    assert torch.allclose(weights.sum(), torch.tensor(1.0, dtype=torch.float64))
    picked = chosen[0].tolist()
    assert torch.allclose(weights[0], s[picked] / s[picked].sum())
    # a correction changes the choice but not the weights' source; choice scores may be negative
    w["correction"] = torch.tensor([0.0, 0.0, -5.0, -5.0, -5.0, -5.0, -3.0, -3.0], dtype=torch.float64)
    chosen, weights = P.route(h, w, "", r)
    assert sorted(chosen[0].tolist()) == [0, 1, 7]            # groups (0,1) and (6,7); expert 6 is worse than 1
    assert torch.allclose(weights[0], s[chosen[0]] / s[chosen[0]].sum())
    # one group keeps everything; experts are squared relus
    chosen, _ = P.route(h, dict(w, correction=torch.zeros(8, dtype=torch.float64)), "", {"experts": 8, "top": 2})
    assert sorted(chosen[0].tolist()) == [0, 7]
    e = {"up": torch.tensor([[1.0, 0, 0, 0], [-1.0, 0, 0, 0]], dtype=torch.float64), "down": torch.tensor([[1.0, 1.0]] * 4, dtype=torch.float64)}
    assert torch.allclose(P.expert(3.0 * h, e, ""), torch.full((1, 4), 9.0, dtype=torch.float64))


# ---------------------------------------------------------------------------------------- replay through the engine
LENGTHS = (41, 70, 23, 88, 1, 37)
SCHEDULES = {"whole": TT.schedule_whole, "bulk_tail": TT.schedule_bulk_tail, "portions": TT.schedule_portions,
             "mixed": TT.schedule_mixed}
_cache = {}


def _reference(which):
    if which not in _cache:
        folder = X.write_folder({"a": X.small_a, "b": X.small_b, "odd": X.odd_shapes}[which](), seed=5, edit=X.lively)
        vocab = load_config(folder).vocab_size
        reqs = random_requests(vocab, LENGTHS, seed=4)
        _cache[which] = (folder, vocab, reqs, X.plain_logits(folder, reqs))
    return _cache[which]


@pytest.mark.parametrize("which", ["a", "b"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
def test_replay_matches_plain_under_every_cut(emulated, tmp_path, which, schedule):
    folder, vocab, reqs, ref = _reference(which)
    trace = SCHEDULES[schedule](reqs)
    if schedule == "portions":
        assert min(len(e["tokens"]) for s in trace.steps for e in s["entries"]) <= 2
    if schedule == "mixed":
        assert max(len(s["entries"]) for s in trace.steps) == 4 and trace.preemptions == 1     # pages and slots are used again
    engine = trace_mod.build_engine(folder, "float32", trace.max_tokens, block_size=8, device="cpu")
    n = trace_mod.replay(engine, io.StringIO(trace.lines()), str(tmp_path), io.StringIO())
    assert n == len(trace.steps)
    got = TT.read_logits(str(tmp_path), trace, vocab)
    assert TT.compare(got, ref, 2e-5, f"{which}/{schedule}") < 2e-5
    engine.cache.check()
    assert not engine.cache.requests and engine.cache.slots.num_free == 4


def test_streams_after_every_layer(emulated):
    folder, vocab, reqs, _ = _reference("a")
    cfg, w = X.read_folder(folder)
    toks = reqs["r2"]
    want = []
    P.forward(cfg, w, toks, streams=want)
    engine = trace_mod.build_engine(folder, "float32", 64, block_size=8, device="cpu")
    seen = []

    def recording(block):
        def run(x, ctx, cache, write=True):
            y = block(x, ctx, cache, write)
            seen.append(y.clone())           # (the next layer adds into y in place)
            return y
        return run

    for layer in engine.model.layers:
        layer.block = recording(layer.block)
    engine.runner.step([StepEntry("x", toks, [0])])
    assert len(seen) == len(want) == 8
    for k, (a, b) in enumerate(zip(seen, want)):
        assert float((a.double() - b).abs().max() / b.abs().max()) < 1e-5, f"layer {k}"


def test_window_pages_come_back_and_states_start_at_zero(emulated):
    folder, vocab, reqs, ref = _reference("a")
    engine = trace_mod.build_engine(folder, "float32", 192, block_size=8, device="cpu")
    cache = engine.cache
    windowed = [i for i, g in enumerate(cache.groups) if g.need.window is not None]
    assert len(windowed) == 1 and cache.groups[windowed[0]].need.window == 29          # the lender keeps the borrower's window
    toks = reqs["r3"]
    rows = [engine.runner.step([StepEntry("x", toks[:50], list(range(50)))])]
    table = cache.block_table("x", windowed[0])
    assert table[0] == -1 and table[1] == -1 and table[2] >= 0                         # keys below 50 - 29 + 1 = 22 are gone: pages 0 and 1
    for p in range(50, len(toks)):
        rows.append(engine.runner.step([StepEntry("x", toks[p:p + 1], [0])]))
    got = torch.cat(rows).double()
    assert float((got - ref["r3"]).abs().max() / ref["r3"].abs().max()) < 2e-5
    engine.runner.finish("x")
    # the slot's state rows hold what the request left; the next request in the same slot starts from zeros all the same
    states = [t for t in cache._state.values()]
    assert states and any(float(t[0].abs().max()) > 0 for t in states)
    again = engine.runner.step([StepEntry("y", reqs["r0"], list(range(len(reqs["r0"]))))]).double()
    assert cache.state_slot("y") == 0
    assert float((again - ref["r0"]).abs().max() / ref["r0"].abs().max()) < 2e-5
    engine.runner.finish("y")
    cache.check()


def test_odd_sizes_in_portions(emulated):
    folder, vocab, reqs, ref = _reference("odd")
    engine = trace_mod.build_engine(folder, "float32", 128, block_size=8, device="cpu")
    toks = reqs["r1"]
    got = torch.cat([engine.runner.step([StepEntry("x", toks[:9], list(range(9)))]),
                     engine.runner.step([StepEntry("x", toks[9:11], [0, 1])]),
                     engine.runner.step([StepEntry("x", toks[11:69], list(range(58)))]),
                     engine.runner.step([StepEntry("x", toks[69:], [0])])]).double()
    assert float((got - ref["r1"]).abs().max() / ref["r1"].abs().max()) < 2e-5
    engine.runner.finish("x")
    engine.cache.check()


def test_generate_greedy_matches_plain(emulated):
    folder, vocab, reqs, ref = _reference("a")
    cfg, w = X.read_folder(folder)
    prompts = [reqs["r2"], reqs["r4"], reqs["r0"][:30]]
    llm = LLM(folder, dtype="float32", device="cpu", block_size=8, num_blocks=24, max_model_len=64, max_num_seqs=2,
              max_num_batched_tokens=16, max_prefill_chunk=7)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.outputs[0].token_ids == P.greedy(cfg, w, p, 6)
    assert not llm.engine.cache.requests


def test_command_line_info_and_random_weights(tmp_path):
    """`rvllm random-weights` writes a folder for the design from a config.json; `rvllm info` reads it back."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(X.small_a()))
    out = tmp_path / "model"
    run = lambda *a: subprocess.run([sys.executable, os.path.join(root, "bin", "rvllm"), *a], capture_output=True, text=True, timeout=300)
    p = run("random-weights", "--config", str(cfg_file), "--out", str(out), "--seed", "3")
    assert p.returncode == 0, p.stderr
    p = run("info", "--model", str(out))
    assert p.returncode == 0, p.stderr
    info = json.loads(p.stdout)
    assert info["architecture"] == "Tugodra" and info["config"]["layers"][4]["mixer"]["kv_from"] == 1
    cfg, w = X.read_folder(str(out))
    assert w["l0.norm1.alpha"].shape == () and P.forward(cfg, w, [1, 2, 3]).shape == (3, 131)


def test_steps_ask_the_kernel_library_for_strict_launches(emulated):
    """The design's specification switches programmatic dependent launch off, and the step function tells the kernel library,
    which the engines of a process share, before every step - and switches it back on for a model that allows it."""
    from model_tools import model_folder

    class Recording(EmulatedKernels):
        calls = []

        def set_pdl(self, allowed):
            self.calls.append(bool(allowed))

    kernel_pkg.set_library(Recording())
    folder, vocab, reqs, ref = _reference("a")
    assert load_config(folder).to_spec().programmatic_launch is False
    engine = trace_mod.build_engine(folder, "float32", 64, block_size=8, device="cpu")
    engine.runner.step([StepEntry("x", reqs["r2"][:5], [4])])
    assert Recording.calls and Recording.calls[-1] is False
    other = trace_mod.build_engine(model_folder("tiny_llama"), "float32", 64, block_size=8, device="cpu")
    other.runner.step([StepEntry("y", [1, 2, 3], [2])])
    assert Recording.calls[-1] is True
