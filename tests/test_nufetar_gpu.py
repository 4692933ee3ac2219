"""Nufetar through the engine against the plain implementation (tests/plain_nufetar.py): whole prompts, prefill
against token-by-token decoding, portions down to two tokens, mixed batches with pages and state slots that are
used again, each mechanism alone, weights made so that a key lost or one too many at the edge of a window or of a
run of positions would show, long decoding, sizes that differ in every place, and greedy generation through the
entry points."""
import copy

import numpy as np
import pytest
import torch

import plain_nufetar as plain
from helpers import Trace, max_live_tokens, mixed_schedule, run_trace
from lelatar_cases import run_engine, tokens, worst
from nufetar_cases import (CONFIG_A, CONFIG_B, CONFIG_C, CONFIG_ODD, CONFIG_W, ONLY_ATTENTION, ONLY_LATENT, ONLY_WKV, make_dir,
                           sharpen, with_mask)

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C, "W": CONFIG_W, "odd": CONFIG_ODD, "attention": ONLY_ATTENTION,
           "latent": ONLY_LATENT, "wkv": ONLY_WKV}
# Largest |difference| as a fraction of max(1, largest |logit| of the row).  float32: sums in another order.
# bfloat16: the rounding of every product's inputs.  Measured on a B200: at most 1.0e-6 and 0.007 over all cases below; a key
# lost or one too many at an edge moves the sharpened models' logits by 0.06 and more.
TOL = {"float32": 5e-6, "bfloat16": 0.02}


def reference(config, weights, requests):
    return {name: plain.forward(config, weights, toks, dtype=torch.float64).float() for name, toks in requests.items()}


def load(path, dtype):
    from mlx_lm_b200.weights import load_model
    return load_model(str(path), dtype=dtype)[0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts(name, dtype, tmp_path):
    """One step per prompt, all logits: also the first tokens of a sequence (lengths 1, 2, 3: the token before the
    first is zeros, the states start at zero, the first run and the first window are not full)."""
    config = CONFIGS[name]
    weights = make_dir(tmp_path, config, seed=11)
    reqs = {f"r{n}": tokens(n, config["vocab"], n) for n in (1, 2, 3, 37, 150)}
    tr = Trace()
    for rid, toks in reqs.items():
        tr.whole(rid, toks)
    got = run_engine(load(tmp_path, dtype), tr)
    w = worst(got, reference(config, weights, reqs))
    print(f"whole {name} {dtype}: {w:.3g}")
    assert w < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cutting_gives_the_same_logits(name, dtype, tmp_path):
    """Prefill then 40 tokens one by one; portions of many sizes (two tokens, one, sizes around the 16 tokens the
    recurrence stages at a time, around 32 and 64 rows, more than 128); mixed batches of unequal requests in a pool
    with three state slots and few pages, so that both are used again by later requests."""
    config = CONFIGS[name]
    weights = make_dir(tmp_path, config, seed=5)
    V = config["vocab"]
    reqs = {"a": tokens(70, V, 1), "b": tokens(131, V, 2), "c": tokens(23, V, 3), "d": tokens(300, V, 4), "e": tokens(5, V, 5)}
    tr = Trace()
    for rid, toks in reqs.items():
        tr.bulk_then_single(f"{rid}:tail", toks, tail=40)
    for rid, toks in reqs.items():
        tr.portions(f"{rid}:portions", toks, sizes=(2, 1, 15, 2, 16, 17, 3, 33, 2, 37, 64, 2, 130, 1, 31))
    mixed_schedule(tr, [(f"{rid}:mixed", toks) for rid, toks in reqs.items()], seed=1, max_live=3)
    mixed_schedule(tr, [(f"{rid}:mixed2", toks) for rid, toks in reversed(list(reqs.items()))], seed=2, max_live=3,
                   sizes=(2, 1, 1, 48, 1, 16, 1, 2, 37, 1, 1, 9, 130, 1))
    pool = max_live_tokens(tr, round_to=16)
    got = run_engine(load(tmp_path, dtype), tr, page_size=16, n_pages=pool // 16, max_requests=3, max_len=512)
    assert len(got) == 4 * sum(len(t) for t in reqs.values())
    w = worst(got, reference(config, weights, reqs))
    print(f"cuttings {name} {dtype}: {w:.3g}")
    assert w < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["run of positions", "window"])
def test_keys_at_the_edges_of_runs_and_windows(case, dtype, tmp_path):
    """Sharp attention: single scores stand out.  The plain model with a run or a window one position longer or
    shorter gives other logits (so a key lost or one too many at the edge shows), and the engine gives the plain
    model's: in prompts cut at, just before and just after the edges, and in tokens decoded one by one across them."""
    if case == "run of positions":
        config, layer, size = copy.deepcopy(ONLY_ATTENTION), 0, 40
    else:
        config, layer, size = copy.deepcopy(ONLY_LATENT), 0, 30
    weights = make_dir(tmp_path, config, seed=21, edit=lambda w: sharpen(w, 12.0))
    V = config["vocab"]
    reqs = {"a": tokens(135, V, 31), "b": tokens(90, V, 32)}
    ref = reference(config, weights, reqs)
    for other in (size - 1, size + 1):
        moved = plain.forward(with_mask(config, layer, other), weights, reqs["a"]).float()
        assert float((moved - ref["a"]).abs().max()) > 0.3, other
    tr = Trace()
    tr.whole("a:w", reqs["a"])
    tr.portions("a:1", reqs["a"], sizes=(size - 1, 1, 1, size - 2, 2, 2, size, 3))
    tr.portions("b:1", reqs["b"], sizes=(size, size - 1, 2, 2))
    tr.bulk_then_single("a:2", reqs["a"], tail=135 - size + 3)           # decodes across every edge after the first
    tr.bulk_then_single("b:2", reqs["b"], tail=12)
    got = run_engine(load(tmp_path, dtype), tr)
    w = worst(got, ref)
    print(f"edges of a {case} {dtype}: {w:.3g}")
    assert w < 2 * TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_and_page_borders(dtype, tmp_path):
    """Runs and windows of hundreds of positions with sharp attention: keys far back, across many pages and across
    the 64-key blocks the kernel walks, in portions that end at and next to those borders and in decoding."""
    config = copy.deepcopy(CONFIG_A)
    config["layers"][0]["mixer"]["mask"]["size"] = 333
    config["layers"][1]["mixer"]["mask"]["size"] = 290
    config["layers"][3]["mixer"]["mask"]["size"] = 256
    weights = make_dir(tmp_path, config, seed=22, edit=lambda w: sharpen(w, 8.0))
    V = config["vocab"]
    reqs = {"a": tokens(400, V, 31), "b": tokens(260, V, 32)}
    ref = reference(config, weights, reqs)
    dull = make_dir(tmp_path / "dull", config, seed=22)
    assert float((plain.forward(config, dull, reqs["b"]).float() - ref["b"]).abs().max()) > 0.5
    tr = Trace()
    tr.portions("a:1", reqs["a"], sizes=(127, 1, 2, 126, 16, 15, 1, 112))
    tr.portions("b:1", reqs["b"], sizes=(129, 127, 2, 2))
    tr.bulk_then_single("b:2", reqs["b"], tail=8)
    tr.bulk_then_single("a:2", reqs["a"], tail=80)
    got = run_engine(load(tmp_path, dtype), tr)
    w = worst(got, ref)
    print(f"far keys {dtype}: {w:.3g}")
    assert w < 2 * TOL[dtype]


def test_each_option_of_the_attention_matters_and_is_there(tmp_path):
    """The plain model without the score mix, the value norm, the head gate or a bias gives other logits; the engine
    gives those of the full one."""
    config = ONLY_ATTENTION
    weights = make_dir(tmp_path, config, seed=3)
    toks = tokens(60, config["vocab"], 1)
    ref = reference(config, weights, {"a": toks})
    H = config["layers"][0]["mixer"]["heads"]
    for name, value in (("l0.mix.talk", torch.eye(H)), ("l0.mix.g", None), ("l0.mix.o.b", None), ("l0.mix.k.b", None)):
        changed = dict(weights)
        changed[name] = torch.zeros_like(weights[name].float()) if value is None else value
        assert float((plain.forward(config, changed, toks).float() - ref["a"]).abs().max()) > 0.05, name
    tr = Trace()
    tr.whole("a:w", toks)
    tr.bulk_then_single("a:t", toks, tail=25)
    w = worst(run_engine(load(tmp_path, "float32"), tr), ref)
    assert w < TOL["float32"], w


def test_state_is_per_request_and_starts_at_zero(tmp_path):
    """A slot that a long request left is given to the next one: neither the recurrence's state nor the token
    before may leak.  The same prompt, run after another request in the same slot, gives what it gives alone."""
    config = ONLY_WKV
    weights = make_dir(tmp_path, config, seed=2)
    V = config["vocab"]
    a, b = tokens(120, V, 1), tokens(9, V, 2)
    ref = reference(config, weights, {"a": a, "b": b})
    tr = Trace()
    tr.whole("a:1", a)
    tr.portions("b:1", b, sizes=(2, 1, 3))
    tr.whole("a:2", a)
    got = run_engine(load(tmp_path, "float32"), tr, max_requests=1, n_pages=16)
    assert worst(got, ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype, tmp_path):
    """A short prompt and then 500 tokens one by one beside a second request: windows and runs pass over decoded
    tokens many times, pages are given back and taken again, the state is carried 500 times."""
    config = CONFIG_A
    weights = make_dir(tmp_path, config, seed=8)
    V = config["vocab"]
    reqs = {"a": tokens(510, V, 1), "b": tokens(200, V, 2)}
    ref = reference(config, weights, reqs)
    tr = Trace()
    tr.step([("a", reqs["a"][:10], "all"), ("b", reqs["b"][:3], "all")])
    for t in range(10, 510):
        e = [("a", reqs["a"][t:t + 1], "all")]
        tb = t - 7
        if tb < 200:
            e.append(("b", reqs["b"][tb:tb + 1], "all"))
        tr.step(e, end=(["b"] if tb == 199 else []) + (["a"] if t == 509 else []))
    got = run_engine(load(tmp_path, dtype), tr, n_pages=24, max_requests=2, max_len=640)
    w = worst(got, ref)
    print(f"long decoding {dtype}: {w:.3g}")
    assert w < TOL[dtype]


def test_trace_replay_with_few_slots_and_pages(tmp_path):
    """The command-line replay on this design: mixed steps in a pool that forces pages and slots to be used again."""
    config = CONFIG_B
    weights = make_dir(tmp_path / "m", config, seed=13)
    V = config["vocab"]
    reqs = {f"r{i}": tokens(n, V, 40 + i) for i, n in enumerate((50, 3, 129, 64, 18, 77))}
    ref = reference(config, weights, reqs)
    tr = Trace()
    mixed_schedule(tr, list(reqs.items()), seed=5, max_live=4)
    for dtype in DTYPES:
        got = run_trace(str(tmp_path / "m"), tr, dtype, str(tmp_path / f"out-{dtype}"), extra=("--max-requests", "4"))
        w = worst(got, ref)
        print(f"replay {dtype}: {w:.3g}")
        assert w < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_points(dtype, tmp_path):
    """``generate``, ``stream_generate`` and ``batch_generate`` (scheduler, decode graphs, device sampler) give the
    plain model's greedy tokens."""
    from mlx_lm_b200 import batch_generate, generate, load, stream_generate
    config = CONFIG_A
    weights = make_dir(tmp_path, config, seed=23, calmed=False, edit=lambda w: w.__setitem__("embed", w["embed"] * 0.25))
    V = config["vocab"]
    prompts = [tokens(7, V, 0), tokens(21, V, 1), tokens(2, V, 2)]

    def greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(plain.forward(config, weights, seq)[-1].argmax()))
        return seq[len(prompt):]

    def agrees(got, ref, prompt):
        for i, (a, b) in enumerate(zip(got, ref)):
            if a != b:
                lg = plain.forward(config, weights, prompt + ref[:i])[-1]
                top = torch.topk(lg, 2).values
                return dtype == "bfloat16" and float(top[0] - top[1]) < 0.05 * float(lg.abs().max())
        return len(got) == len(ref)

    want = [greedy(p, 30) for p in prompts]
    model, tokenizer = load(str(tmp_path), dtype=dtype)
    for p, w in zip(prompts, want):
        got = [int(t) for t in generate(model, tokenizer, p, max_tokens=30).split()]
        assert agrees(got, w, p), (got, w)
        streamed = [r.token for r in stream_generate(model, tokenizer, p, max_tokens=30, prefill_step_size=5)]
        assert agrees(streamed, w, p), (streamed, w)
    out = batch_generate(model, tokenizer, prompts, max_tokens=30, return_token_ids=True)
    for got, w, p in zip(out.token_ids, want, prompts):
        assert agrees(got, w, p), (got, w)


def test_command_line_and_sampling(tmp_path):
    """`python -m mlx_lm_b200 generate` on a model folder gives the Python entry point's tokens; the random-weights
    mode builds the design from a config.json alone; samplers with filters run on its logits; and what is drawn
    with a temperature does not depend on what else is in the batch."""
    import json
    import subprocess
    import sys
    from helpers import ROOT
    from mlx_lm_b200 import generate, load
    from mlx_lm_b200.generate import BatchGenerator
    from mlx_lm_b200.sampling import make_sampler
    config = CONFIG_C
    make_dir(tmp_path / "m", config, seed=31, calmed=False, edit=lambda w: w.__setitem__("embed", w["embed"] * 0.25))
    model, tokenizer = load(str(tmp_path / "m"), dtype="float32")
    want = generate(model, tokenizer, [5, 17, 3], max_tokens=12)
    run = lambda *a: subprocess.run([sys.executable, "-m", "mlx_lm_b200", "generate", *a], cwd=ROOT, capture_output=True,
                                    text=True, timeout=300)
    r = run("--model", str(tmp_path / "m"), "--prompt", "5 17 3", "-m", "12", "--dtype", "float32", "--verbose", "F")
    assert r.returncode == 0, r.stderr
    assert r.stdout.split() == want.split()
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(config))
    r = run("--random-weights", "11", "--config", str(cfg), "--prompt", "5 17 3", "-m", "12", "--temp", "0.7",
            "--top-p", "0.9", "--min-p", "0.01", "--top-k", "20", "--seed", "4", "--verbose", "F")
    assert r.returncode == 0 and len(r.stdout.split()) == 12, r.stderr
    prompts = [tokens(n, config["vocab"], n) for n in (5, 31, 64)]

    def drawn(**kw):
        gen = BatchGenerator(model, max_tokens=20, sampler=make_sampler(0.8, top_p=0.95), seed=1, **kw)
        uids = gen.insert(prompts)
        out = {u: [] for u in uids}
        while gen.scheduler.has_work():
            for resp in gen.next_generated():
                out[resp.uid].append(resp.token)
        return [out[u] for u in uids]
    together = drawn(completion_batch_size=8, prefill_batch_size=8)
    assert all(len(t) == 20 for t in together)
    assert drawn(completion_batch_size=1, prefill_batch_size=1) == together
    assert drawn(completion_batch_size=2, prefill_batch_size=1, prefill_step_size=7, max_tokens_per_step=9) == together
