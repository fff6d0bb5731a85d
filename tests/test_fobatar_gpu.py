"""Fobatar through the engine: the step function, the cache manager and the runtime against the plain
implementation (``plain_fobatar``), on five tiny configurations that differ in every size, in both
dtypes: whole prompts, token-by-token decoding, portions down to two tokens, batches of unequal
requests over pools whose pages and slots are used again, long decoding over page and chunk borders,
the stream after every layer run, and greedy generation through the entry point and its scheduler."""
import numpy as np
import pytest
import torch

import plain_fobatar as P
from gpu_util import (DTYPES, TOL_ORACLE, assert_close, mixed_trace, model_dir, new_runner, oracle_bound,
                      plain_logits, plain_model, random_tokens, replay_in_process, run_portions, run_whole)
from tiny_configs import TINY, vocab_of

pytestmark = pytest.mark.gpu
NAMES = ("FA", "FB", "FC")
ALL = NAMES + ("FD", "FE")


@pytest.mark.parametrize("name", ALL)
@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompts(name, dtype):
    runner = new_runner(name, dtype)
    for n in (1, 2, 3, 37, 38, 64, 65, 71, 131, 200):
        tokens = random_tokens(name, n, seed=n)
        assert_close(run_whole(runner, f"w{n}", tokens), plain_logits(name, dtype, tokens),
                     oracle_bound(name, dtype, tokens), f"{name} {dtype} whole prompt of {n}")
    runner.check_health()


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_against_token_by_token_decoding(name, dtype):
    runner = new_runner(name, dtype)
    tokens = random_tokens(name, 140, seed=5)
    whole = run_whole(runner, "whole", tokens)
    single = run_portions(runner, "single", tokens, [1])
    want = plain_logits(name, dtype, tokens)
    bound = oracle_bound(name, dtype, tokens)
    assert_close(single, want, bound, "token by token")
    assert_close(single, whole, 2e-5 if dtype == "float32" else bound, "token by token against the whole prompt")
    late = run_portions(runner, "late", tokens, [100] + [1] * 40)
    assert_close(late, want, bound, "a prompt, then decoding")


@pytest.mark.parametrize("name", ALL)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(2,), (3, 2, 7, 1, 64, 2, 33), (63, 2, 64, 1, 1, 65), (128, 2), (36, 1, 1, 2)])
def test_portions_of_any_size(name, dtype, sizes):
    runner = new_runner(name, dtype)
    tokens = random_tokens(name, 197, seed=11)
    want = plain_logits(name, dtype, tokens)
    assert_close(run_portions(runner, "p", tokens, list(sizes)), want, oracle_bound(name, dtype, tokens),
                 f"portions {sizes}")


@pytest.mark.parametrize("name", ALL)
@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_over_a_small_pool(name, dtype):
    """Up to four live requests, portions beside single tokens, requests left out of steps; the pool
    has fewer pages than the requests need together, so pages and state slots are used again, and a
    stale recurrent state, a stale source of mixed values or a cache row of an earlier owner would show."""
    lengths = [150, 40, 97, 1, 130, 64, 2, 70, 129]
    steps, tokens = mixed_trace(lengths, vocab_of(TINY[name]), num_pages=7, max_live=4, seed=4, tail=20)
    runner = new_runner(name, dtype, num_pages=7, num_slots=4, max_model_len=256)
    got = replay_in_process(runner, steps)
    for rid, ids in tokens.items():
        assert_close(got[rid], plain_logits(name, dtype, ids), oracle_bound(name, dtype, ids),
                     f"{name} {dtype} request {rid}")
    assert all(group.pool.n_used == 0 for group in runner.cache.groups)
    runner.check_health()


@pytest.mark.parametrize("name", ("FA", "FB", "FE"))
def test_a_slot_and_pages_used_again_hold_nothing_of_their_last_owner(name):
    dtype = "float32"
    runner = new_runner(name, dtype, num_pages=3, num_slots=1, max_model_len=192)
    first = random_tokens(name, 180, seed=1)
    second = random_tokens(name, 150, seed=2)
    run_whole(runner, "first", first)
    got = run_portions(runner, "second", second, [70, 1, 1, 50, 28])
    assert_close(got, plain_logits(name, dtype, second), TOL_ORACLE[dtype], "second owner")


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_page_and_chunk_borders(name, dtype):
    """Three requests decode together for 200 steps from prompts of different lengths: every page border
    is crossed by a decoded token and every chunk's border is crossed by decoded tokens, in a replayed graph once the shape has settled."""
    prompts = [random_tokens(name, n, seed=30 + n) for n in (1, 60, 127)]
    cont = [random_tokens(name, 200, seed=40 + i) for i in range(3)]
    runner = new_runner(name, dtype, num_pages=16, num_slots=4, max_model_len=512)
    rows = [[runner.step([(f"d{i}", p, list(range(len(p))))]).cpu().numpy()] for i, p in enumerate(prompts)]
    for step in range(200):
        out = runner.step([(f"d{i}", [cont[i][step]], [0]) for i in range(3)]).cpu().numpy()
        for i in range(3):
            rows[i].append(out[i:i + 1])
    assert runner.graph_replays > 0
    for i in range(3):
        assert_close(np.concatenate(rows[i]), plain_logits(name, dtype, prompts[i] + cont[i]),
                     oracle_bound(name, dtype, prompts[i] + cont[i]), f"{name} {dtype} request {i}")
    runner.check_health()


@pytest.mark.parametrize("name", ("FA", "FB", "FC"))
def test_the_stream_after_every_layer(name):
    """float32, layer by layer: the engine's residual stream behind each layer against the plain one, so a
    fault shows in the first layer that has it and not only in the logits."""
    dtype = "float32"
    tokens = random_tokens(name, 90, seed=8)
    cfg, w = plain_model(name, dtype)
    want = []
    P.forward(cfg, w, tokens, layers_out=want)
    runner = new_runner(name, dtype)
    model = runner.model
    seen = []
    hooks = []
    for layer in model.layers:             # (a layer that runs several times is hooked once and seen each time)
        original = layer.forward

        def wrapped(ctx, x, pending, cache, _f=original):
            out = _f(ctx, x, pending, cache)
            assert out[1] is None
            seen.append(out[0].detach().to(torch.float64).cpu().clone())
            return out
        layer.forward = wrapped
        hooks.append((layer, original))
    try:
        run_whole(runner, "layers", tokens)
    finally:
        for layer, original in hooks:
            layer.forward = original
    assert len(seen) == len(want) == len(P.layer_runs(cfg))
    for index, (got, plain) in enumerate(zip(seen, want)):
        assert_close(got.numpy(), plain.numpy(), 2e-5, f"{name} stream behind layer run {index}")


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_runtime(name):
    from flyweight_b200 import Model
    cfg, w = plain_model(name, "float32")
    prompts = [random_tokens(name, n, seed=50 + n) for n in (1, 9, 70)]
    with Model(model_dir(name, "float32"), dtype="float32").native_runtime(
            context_limit=192, parallel_sequences=3) as runtime:
        alone = runtime.generate(prompts[1], 24)
        assert alone == P.greedy_generate(cfg, w, prompts[1], 24)
        for prompt, result in zip(prompts, runtime.generate_batch(prompts, 24)):
            assert list(result.generated_ids) == P.greedy_generate(cfg, w, prompt, 24)
        assert runtime.info["cache"]["groups"][0]["pages_in_use"] == 0


def test_bfloat16_generation_with_more_requests_than_slots():
    """Requests queue for slots and pages, are admitted as others end, and every generated token is
    (within the bfloat16 bound) the best of the plain implementation's logits at its place."""
    from flyweight_b200 import Model
    name, dtype = "FC", "bfloat16"
    prompts = [random_tokens(name, n, seed=70 + n) for n in (3, 40, 66, 12, 90, 5)]
    with Model(model_dir(name, dtype), dtype=dtype).native_runtime(
            context_limit=128, parallel_sequences=2) as runtime:
        results = runtime.generate_batch(prompts, 20)
    for prompt, result in zip(prompts, results):
        made = list(result.generated_ids)
        assert len(made) == 20
        logits = plain_logits(name, dtype, prompt + made)
        scale = max(1.0, np.abs(logits).max())
        for i, token in enumerate(made):
            row = logits[len(prompt) - 1 + i]
            assert row.max() - row[token] <= 2 * oracle_bound(name, dtype, prompt + made) * scale


def test_the_model_folder_round_trip_the_command_line_and_the_trace_runner(tmp_path):
    """`make-random` writes a Fobatar folder from a configuration file, `inspect` and `generate` read it,
    and the trace runner replays steps over it."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY["FA"]))
    folder = tmp_path / "model"
    run = lambda *args: subprocess.run([sys.executable, "-m", "flyweight_b200", *args], cwd=root,
                                       capture_output=True, text=True, timeout=600)
    made = run("make-random", str(config), "--out", str(folder), "--seed", "5", "--preset", "unit",
               "--dtype", "float32")
    assert made.returncode == 0, made.stderr
    seen = run("inspect", str(folder))
    assert seen.returncode == 0 and "Fobatar" in seen.stdout, seen.stderr
    prompt = random_tokens("FA", 6, seed=1)
    out = run("generate", str(folder), "--dtype", "float32", "--prompt", ",".join(map(str, prompt)),
              "--max-tokens", "8", "--temperature", "0")
    assert out.returncode == 0, out.stderr[-2000:]
    cfg, w = P.load_model_dir(folder)
    assert [int(t) for t in out.stdout.split()] == P.greedy_generate(cfg, w, prompt, 8)
    tokens = random_tokens("FA", 75, seed=2)
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:70], "want": [0, 69]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[70:72], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": tokens[72:], "want": [2]}], "end": ["a"]}]
    replay = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out",
                             str(tmp_path / "out"), "--max-tokens", "128"], cwd=root, capture_output=True, text=True,
                            timeout=600, input="".join(json.dumps(line) + "\n" for line in lines))
    assert replay.returncode == 0, replay.stderr[-2000:]
    assert [l for l in replay.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = np.asarray(P.forward(cfg, w, tokens))
    got = np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(2, -1)
    assert_close(got, want[[0, 69]], TOL_ORACLE["float32"], "step 0")
    assert not (tmp_path / "out" / "1.f32").exists()
    got = np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(1, -1)
    assert_close(got, want[[74]], TOL_ORACLE["float32"], "step 2")


# ------------------------------------------------------------------ wider layers, longer prompts
def _wider_config(v):
    ramp = lambda factor, original, fast, slow: {"factor": factor, "original": original, "fast": fast, "slow": slow}
    if v == 0:
        att = {"heads": 4, "kv_heads": 4, "dim": 64, "vdim": 128, "scale": 0.11, "conv": 4, "mask": {"size": 100},
               "rot": {"base": 10000.0, "dims": 32, "scaling": ramp(4.0, 128, 16.0, 1.0)}}
        att_wide = {"heads": 6, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.2, "conv": 2, "mask": {"size": 300}}
        lat = {"heads": 8, "dim": 64, "rot_dim": 32, "vdim": 32, "kv_rank": 192, "scale": 0.125,
               "rot": {"base": 10000.0, "dims": 32, "scaling": ramp(2.0, 256, 32.0, 2.0)}}
        mlp = {"kind": "moe", "expert": {"ff": 96, "limit": 1.5}, "router": {"experts": 5, "top": 2},
               "shared": {"ff": 160, "limit": 2.5}}
        layers = [{"type": "latent_attention", "mixer": lat, "mlp": mlp},
                  {"type": "attention", "mixer": att, "mlp": None},
                  {"type": "attention", "mixer": att_wide, "mlp": mlp},
                  {"type": "latent_attention", "mixer": lat, "mlp": None},
                  {"type": "attention", "mixer": att, "mlp": mlp}]
        return {"architecture": "Fobatar", "vocab": 1000, "width": 256, "norm": {"eps": 1e-6},
                "embedding": {"scale": 2.0}, "residual_mult": 0.4, "loop": {"start": 2, "stop": 5, "times": 2},
                "layers": layers}
    att = {"heads": 12, "kv_heads": 3, "dim": 128, "vdim": 64, "scale": 0.09, "conv": 3, "mask": {"size": 257},
           "rot": {"base": 500000.0, "dims": 80, "scaling": ramp(32.0, 2048, 64.0, 4.0)}}
    lat = {"heads": 5, "dim": 24, "rot_dim": 8, "vdim": 56, "kv_rank": 72, "scale": 0.1, "rot": {"base": 300.0, "dims": 8}}
    mlp = {"kind": "moe", "expert": {"ff": 200, "limit": 3.0}, "router": {"experts": 9, "top": 4}}
    layers = [{"type": "attention", "mixer": att, "mlp": mlp},
              {"type": "latent_attention", "mixer": lat, "mlp": mlp},
              {"type": "latent_attention", "mixer": lat, "mlp": mlp},
              {"type": "attention", "mixer": att, "mlp": mlp}]
    return {"architecture": "Fobatar", "vocab": 777, "width": 320, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
            "residual_mult": 0.8, "loop": {"start": 0, "stop": 1, "times": 3}, "layers": layers}


@pytest.mark.parametrize("variant", (0, 1))
@pytest.mark.parametrize("dtype", DTYPES)
def test_wider_layers_and_longer_prompts(variant, dtype, tmp_path):
    """Two configurations with heads of 24 to 128 channels (values wider than keys and narrower, as many key heads
    as query heads and a quarter, rotation of a part of a head, latent rows of 80 and of 224 entries, experts of
    widths that are and are not multiples of 8, layers without a feed-forward, loops over the last layers and over
    the first alone): 700 tokens whole, in portions that end on and off the borders of pages and chunks, and as
    a prompt of 600 followed by 100 single tokens."""
    from tiny_configs import make_model_dir
    from flyweight_b200.engine import ModelRunner, load_model
    config = _wider_config(variant)
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = make_model_dir(str(tmp_path / "model"), config, seed=7 + variant, dtype=stored)
    cfg, w = P.load_model_dir(folder)
    rng = np.random.default_rng(variant)
    tokens = [int(t) for t in rng.integers(0, config["vocab"], size=700)]
    want = np.asarray(P.forward(cfg, w, tokens))
    bound = 2e-4
    if dtype == "bfloat16":
        rounded = np.asarray(P.forward(cfg, w, tokens, rnd=P.bf16))
        bound = max(TOL_ORACLE[dtype], 3.0 * float(np.abs(rounded - want).max()) / max(1.0, float(np.abs(want).max())))
    runner = ModelRunner(load_model(folder, dtype), num_pages=16, num_slots=4, max_model_len=1024,
                         max_batched_tokens=4096)
    for what, sizes in (("whole", [700]), ("portions", [300, 2, 1, 257, 64, 1, 1, 74]), ("decoding", [600] + [1] * 100)):
        assert_close(run_portions(runner, what, tokens, sizes), want, bound, f"variant {variant} {dtype} {what}")
    runner.check_health()
