"""The Tibepel design on the engine's host side, without a GPU: configuration, tensor names, the plain mechanisms
themselves, and the real step function, cache manager, scheduler, trace replay and entry point driven with the torch
stand-ins for the kernels (emulated_kernels.py) against the plain implementation (plain_tibepel.py).  What is checked
here is the bookkeeping - a cache view per member of a mixer made of two, pages of a chunk group given back and used
again, state rows zeroed for a new request, portions cut anywhere; the kernels themselves are checked by the GPU tests."""
import io
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_tibepel as P
import tibepel_tools as X
import trace_tools as TT
from emulated_kernels import EmulatedKernels
from model_tools import random_requests

from rvllm_b200 import ConfigError, LLM, SamplingParams, config_from_dict, kernels as kernel_pkg, load_config
from rvllm_b200.engine import trace as trace_mod
from rvllm_b200.engine.step import StepEntry
from rvllm_b200.models.decoder import DecoderModel, expected_tensors
from rvllm_b200.parts.base import CompositeNeed, KvCacheNeed, StateNeed

F64 = torch.float64


@pytest.fixture
def emulated():
    kernel_pkg.set_library(EmulatedKernels())
    yield
    kernel_pkg.set_library(None)


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64) * scale


# ---------------------------------------------------------------------------------------- configuration
def test_config_round_trip_and_spec():
    cfg = config_from_dict(X.small_a())
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = cfg.to_spec()
    assert spec.residual_dtype == "float32" and spec.lm_head_name == "head" and not spec.validate()
    assert [(e.layer, e.cache) for e in spec.run_order] == [(0, 0), (1, 1), (2, 2), (3, 3)]
    shapes = {n: ts.shape for n, ts in expected_tensors(spec).items()}
    assert shapes["embed"] == (131, 48) and shapes["head"] == (131, 48) and shapes["side.embed"] == (131, 4 * 6)
    assert shapes["l0.mix.in"] == (80, 48) and shapes["l0.mix.x"] == (5 + 2 * 12, 40) and shapes["l0.mix.dt"] == (40, 5)
    assert shapes["l0.mix.conv"] == (40, 3) and shapes["l0.mix.A_log"] == (40, 12) and shapes["l0.mix.D"] == (40,)
    assert shapes["l1.mix.left.q"] == (6 * 16, 48) and shapes["l1.mix.left.v"] == (3 * 24, 48) and shapes["l1.mix.left.v.b"] == (72,)
    assert shapes["l1.mix.left.talk"] == (6, 6) and shapes["l1.mix.left.r1"] == (6,) and shapes["l1.mix.left.o"] == (48, 6 * 24)
    assert shapes["l1.mix.right.q"] == (2 * 12, 48) and shapes["l1.mix.right.v"] == (4 * 20, 48) and shapes["l1.mix.right.v.conv"] == (80, 3)
    assert shapes["l1.mix.right.b"] == (4, 48) and shapes["l1.mix.right.norm"] == (20,) and shapes["l1.mix.right.g"] == (80, 48)
    assert shapes["l1.mlp.gate.b"] == (40,) and shapes["l1.side.proj"] == (48, 6) and shapes["l3.side.norm"] == (48,)
    assert "l2.norm2" not in shapes and "l2.mlp.up" not in shapes and "l2.side.gate" in shapes        # no feed-forward in layer 2
    needs = DecoderModel(spec).cache_needs()
    assert needs[0] == StateNeed((40 * 12 + 2 * 40,), "float32")
    assert needs[1] == CompositeNeed((KvCacheNeed(3, 16, None, 2, 24, 21), StateNeed((4 * 12 * 20 + 2 * (24 + 24 + 80),), "float32")))
    assert needs[2].parts[0] == KvCacheNeed(1, 24, None, 2, 8, 50)
    bare = config_from_dict(X.small_b()).to_spec()
    assert not bare.logit_hooks and not bare.embedding_hooks and "side.embed" not in expected_tensors(bare)
    assert [h.kind for h in config_from_dict(X.odd_shapes()).to_spec().logit_hooks] == ["logit_softcap"]


def test_config_problems_are_collected():
    bad = X.small_a()
    bad["layers"][0]["mixer"]["state"] = 0
    bad["layers"][1]["mixer"]["left"]["kv_heads"] = 4            # 6 heads
    bad["layers"][1]["mixer"]["left"]["mask"] = {}
    bad["layers"][1]["mixer"]["right"]["conv"] = "three"
    bad["layers"][2]["type"] = "attention"
    bad["layers"][3]["mlp"] = {"kind": "wide"}
    bad["logit_softcap"] = -1
    del bad["norm"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    text = str(e.value)
    for piece in ("`state`", "multiple of `kv_heads`", "`size`", "`conv`", "'attention'", "wide", "logit_softcap", "`eps`"):
        assert piece in text, (piece, text)


# ---------------------------------------------------------------------------------------- the plain mechanisms
def test_plain_position_vector_and_norm():
    pe = P.sinusoid([0, 3], 5)
    assert torch.allclose(pe[0], torch.tensor([0.0, 1.0, 0.0, 1.0, 0.0], dtype=F64))
    w1 = 10000.0 ** (-2.0 / 5)
    assert torch.allclose(pe[1], torch.tensor([torch.sin(torch.tensor(3.0)), torch.cos(torch.tensor(3.0)), torch.sin(torch.tensor(3 * w1)),
                                               torch.cos(torch.tensor(3 * w1)), torch.sin(torch.tensor(3 * w1 * w1))], dtype=F64))
    x = rnd(2, 7, seed=1)
    assert torch.allclose(P.offset_norm(x, torch.zeros(7, dtype=F64), 0.0), x / x.pow(2).mean(-1, keepdim=True).sqrt())
    assert torch.allclose(P.offset_norm(x, torch.full((7,), -1.0, dtype=F64), 1e-5), torch.zeros(2, 7, dtype=F64))


def test_plain_attention_chunks_bias_and_mixing():
    """A planted key: the query at position i matches one key strongly.  Inside the query's chunk it takes all the
    weight, one position below the chunk's start it takes none; the distance penalty moves weight to near keys; the
    mixing matrix lets one head read with another head's weights."""
    T, H, G, d, dv, chunk = 14, 4, 2, 6, 3, 5
    v = rnd(T, G, dv, seed=2)
    zero, one = torch.zeros(H, dtype=F64), torch.ones(H, dtype=F64)
    for key, seen in ((10, True), (9, False), (12, True)):           # the query sits at 12: its chunk is 10 .. 14
        q, k = torch.zeros(T, H, d, dtype=F64), torch.zeros(T, G, d, dtype=F64)
        q[12, :, 0], k[key, :, 0] = 30.0, 30.0
        out = P.mixed_head_attention(q, k, v, 1.0, zero, one, torch.eye(H, dtype=F64), chunk)
        for h in range(H):
            want = v[key, h // 2] if seen else v[10:13, h // 2].mean(0)
            assert torch.allclose(out[12, h], want, atol=1e-9), (key, h)
    # the same with the sequence's positions starting at 3: chunks are counted from position 0, so position 12 is index 9
    q, k = torch.zeros(T, H, d, dtype=F64), torch.zeros(T, G, d, dtype=F64)
    out = P.mixed_head_attention(q, k, v, 1.0, zero, one, torch.eye(H, dtype=F64), chunk, start=3)
    assert torch.allclose(out[9, 0], v[7:10, 0].mean(0)) and torch.allclose(out[1, 0], v[0:2, 0].mean(0))
    # penalty r1 ln(1 + r2 dist): with equal scores the weights are (1 + r2 dist)^(-r1)
    r1, r2 = torch.tensor([2.0, 0, 0, 0], dtype=F64), torch.tensor([0.5, 1, 1, 1], dtype=F64)
    out = P.mixed_head_attention(q, k, v, 1.0, r1, r2, torch.eye(H, dtype=F64), 100)
    wts = torch.tensor([(1 + 0.5 * (3 - j)) ** -2.0 for j in range(4)], dtype=F64)
    assert torch.allclose(out[3, 0], (wts / wts.sum()) @ v[:4, 0])
    # mixing: head 3 (kv head 1) reads with head 0's weights, head 0 with the difference of two heads' weights
    talk = torch.zeros(H, H, dtype=F64)
    talk[3, 0], talk[0, 0], talk[0, 1] = 1.0, 1.0, -1.0
    out = P.mixed_head_attention(q, k, v, 1.0, r1, r2, talk, 100)
    assert torch.allclose(out[3, 3], (wts / wts.sum()) @ v[:4, 1])
    assert torch.allclose(out[3, 0], (wts / wts.sum() - 0.25) @ v[:4, 0]) and torch.allclose(out[3, 1], torch.zeros(dv, dtype=F64))


def test_plain_delta_rule_and_scan_properties():
    # beta = 1, no decay, orthonormal keys: the state stores each value exactly and a later write to the same key replaces it
    d, dv = 4, 3
    keys = torch.eye(d, dtype=F64)[[0, 1, 2, 0]][:, None, :]
    vals = rnd(4, 1, dv, seed=3)
    one = torch.ones(4, 1, dtype=F64)
    o = P.delta_rule(keys, keys, vals, one, one)
    assert torch.allclose(o, vals)                                   # the read-out sees the current token's write
    q = torch.eye(d, dtype=F64)[[3, 0, 1, 1]][:, None, :]
    o = P.delta_rule(q, keys, vals, one, one)
    assert torch.allclose(o[0], torch.zeros(1, dv, dtype=F64)) and torch.allclose(o[1], vals[0]) and torch.allclose(o[3], vals[1])
    # with decay g the stored value fades by g per step; beta scales the correction
    g = torch.full((4, 1), 0.5, dtype=F64)
    o = P.delta_rule(q, keys, vals, one, g)
    assert torch.allclose(o[1], 0.5 * vals[0]) and torch.allclose(o[3], 0.25 * vals[1])
    o = P.delta_rule(keys, keys, vals, 0.25 * one, one)
    assert torch.allclose(o[0], 0.25 * vals[0]) and torch.allclose(o[3], 0.25 * vals[0] + 0.25 * (vals[3] - 0.25 * vals[0]))
    # the channel scan: with B = C = 1 on one state and constant dt, y is a geometric sum
    T, dt, a = 5, 0.3, -2.0
    u = torch.ones(T, 1, dtype=F64)
    y = P.channel_scan(u, torch.full((T, 1), dt, dtype=F64), torch.tensor([[a]], dtype=F64), torch.ones(T, 1, dtype=F64),
                       torch.ones(T, 1, dtype=F64), torch.tensor([0.5], dtype=F64))
    decay = torch.exp(torch.tensor(dt * a, dtype=F64))
    want = torch.stack([dt * sum(decay ** j for j in range(t + 1)) + 0.5 for t in range(T)])
    assert torch.allclose(y[:, 0], want)
    # the convolution's last column multiplies the current token; before the start there are zeros
    taps = torch.tensor([[1.0, 10.0, 100.0]], dtype=F64)
    out = P.causal_conv(torch.tensor([[1.0], [2.0], [3.0]], dtype=F64), taps, torch.tensor([0.5], dtype=F64))
    assert out[:, 0].tolist() == [100.5, 210.5, 321.5]


def test_plain_feed_forward_clamps():
    w = {"gate": torch.eye(3, dtype=F64), "up": torch.eye(3, dtype=F64), "down": torch.eye(3, dtype=F64),
         "gate.b": torch.zeros(3, dtype=F64), "up.b": torch.tensor([0.0, 0.0, 0.25], dtype=F64), "down.b": torch.tensor([1.0, 0, 0], dtype=F64)}
    h = torch.tensor([[5.0, -5.0, 0.5]], dtype=F64)
    out = P.clamped_glu(h, w, "", 2.0)[0]
    sig = lambda z: 1.0 / (1.0 + torch.exp(torch.tensor(-1.702 * z, dtype=F64)))
    assert torch.allclose(out, torch.stack([2.0 * sig(2.0) * 3.0 + 1.0, -5.0 * sig(-5.0) * (-2.0 + 1.0), 0.5 * sig(0.5) * 1.75]))


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
        assert max(len(s["entries"]) for s in trace.steps) == 4 and trace.preemptions == 1     # pages are freed and used again
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
    P.forward(cfg, w, toks, layers_out=want)
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
    assert len(seen) == len(want) == 4
    for k, (a, b) in enumerate(zip(seen, want)):
        assert float((a.double() - b).abs().max() / b.abs().max()) < 1e-5, f"layer {k}"


def test_chunk_pages_come_back_while_a_request_runs(emulated):
    """Chunks of 21 and 50 positions over pages of 8: once the next query's chunk starts above a page, the page is free
    again, so a request longer than the pool still runs, and its logits are those of the whole sequence."""
    folder, vocab, _, _ = _reference("a")
    toks = random_requests(vocab, (150,), seed=8)["r0"]
    want = X.plain_logits(folder, {"x": toks})["x"]
    from rvllm_b200.config import EngineConfig
    from rvllm_b200.engine.core import Engine
    engine = Engine(folder, engine_config=EngineConfig(dtype="float32", block_size=8, num_blocks=12, max_model_len=256, max_num_seqs=2,
                                                       max_num_batched_tokens=64, enforce_eager=True, device="cpu"))   # 12 pages for 150 tokens
    rows, at = [], 0
    for n in (19, 2, 3, 30, 1, 1, 1, 30, 2, 27, 3, 31):
        rows.append(engine.runner.step([StepEntry("x", toks[at:at + n], list(range(n)))]))
        at += n
        held = [sum(1 for p in t if p >= 0) for t in engine.cache.requests["x"].tables]
        assert all(h <= 12 for h in held)
    assert at == 150
    got = torch.cat(rows).double()
    assert float((got - want).abs().max() / want.abs().max()) < 2e-5
    engine.runner.finish("x")
    engine.cache.check()
    assert all(n == 12 for n in engine.cache.num_free_pages())


def test_state_rows_start_at_zero_for_a_new_request(emulated):
    """Five requests through two slots: a slot's recurrent state and convolution inputs are those of the new request."""
    folder, vocab, reqs, ref = _reference("b")
    engine = trace_mod.build_engine(folder, "float32", 256, block_size=8, device="cpu", max_live=2)
    for rid in ("r2", "r5", "r0", "r2", "r4"):
        toks = reqs[rid]
        half = len(toks) // 2
        rows = [engine.runner.step([StepEntry(rid, toks[:half], list(range(half)))])] if half else []
        rows.append(engine.runner.step([StepEntry(rid, toks[half:], list(range(len(toks) - half)))]))
        engine.runner.finish(rid)
        assert float((torch.cat(rows).double() - ref[rid]).abs().max() / ref[rid].abs().max()) < 2e-5, rid


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
        ids = list(p)
        for _ in range(6):
            ids.append(int(P.forward(cfg, w, ids)[-1].argmax()))
        assert o.outputs[0].token_ids == ids[len(p):]
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
    assert info["architecture"] == "Tibepel" and info["config"]["layers"][1]["mixer"]["left"]["mask"] == {"size": 21}
    # keys and values of the two attention members: 3 x (16 + 24) and 1 x (24 + 8) elements of two bytes per token
    assert info["kv_bytes_per_token_bf16"] == 2 * (3 * 40 + 32)
    cfg, w = X.read_folder(str(out))
    assert P.forward(cfg, w, [1, 2, 3]).shape == (3, 131)
