"""Fogizen decoders on a device: the scenarios of tests/fogizen_scenarios.py (the engine against the float64 oracle, and each
side of the mixer, the token shift, the router, the experts, the embedding and the block's residual kernel alone with inputs made so that a fault shows) through the CUDA kernels in
float32 and bfloat16, long decoding, graph replay against eager launches, sampling, a checkpoint folder through pipeline() and
bin/trace_run as a process."""
import numpy as np
import pytest
import torch

import fogizen_cases as LC
import fogizen_scenarios as S

pytestmark = pytest.mark.gpu

TOL = {"f32": 2e-5, "bf16": 6e-2}
# Whole decoders in bfloat16: the test configurations have heads of 4 to 12 dimensions, and a unit norm over so few values now and
# then divides by a small root mean square, which multiplies the rounding of what it norms; a lone position reaches a tenth of the
# logits' size.  Each mechanism alone keeps the tight bound.
TOL_ENGINE = {"f32": 2e-5, "bf16": 0.12}


def _make(dtype):
    make = lambda cfg, tensors, **kw: LC.build_engine(cfg, tensors, device="cuda", dtype=dtype, **kw)
    make.all_experts = dtype == "bf16"          # see fogizen_scenarios._config: a rounded stream flips close router choices
    return make


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("scenario", S.ALL, ids=lambda f: f.__name__)
def test_engine_scenario(scenario, dtype):
    scenario(_make(dtype), (TOL if scenario in S.MECHANISMS else TOL_ENGINE)[dtype])


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_long_decoding_over_several_pages(dtype):
    S.prefill_then_decode(_make(dtype), TOL_ENGINE[dtype], n=310, tail=250)


def test_key_ranges_of_a_short_step_agree_with_one_range():
    """A step of few rows cuts its keys into ranges; the scores of all ranges are mixed across heads between the passes and the
    sink joins the denominator once, after the ranges are merged."""
    cfg = LC.config(layers=[LC.layer(LC.left(heads=8, kv_heads=2, dim=32, vdim=32, chunk=0, rot_dims=16, scale=0.2))], width=64)
    w = LC.random_tensors(cfg, seed=41)
    P = LC.prompts_for(cfg, {"a": 330})
    eng = _make("f32")(cfg, w)
    seen = []
    real = eng.model.window_splits
    eng.model.window_splits = lambda n, window, max_pos: seen.append(real(n, window, max_pos)) or seen[-1]
    got = LC.replay(eng, P, [[("a", 300)]] + [[("a", 1)]] * 30)
    assert seen[0] < 8 and max(seen) >= 8
    S._check(got["a"], LC.oracle_logits(cfg, w, P["a"]), 2e-5, "key ranges")


def test_do_sample_through_the_engine_is_a_function_of_the_seed():
    """Sampling requests run the framework's device sampling stage on this decoder's logits; a greedy request beside them is
    not affected by the seed."""
    from lmdeploy_b200.messages import GenerationConfig
    from lmdeploy_b200.turbomind.engine import batched_generate
    cfg = LC.config()
    w = LC.random_tensors(cfg, seed=9)
    P = LC.prompts_for(cfg, {"a": 9, "b": 20})
    run = lambda seed: [list(s.generated) for s in batched_generate(
        LC.build_engine(cfg, w, device="cuda", dtype="bf16"), [P["a"], P["b"]],
        [GenerationConfig(max_new_tokens=12, ignore_eos=True, do_sample=True, top_k=20, temperature=1.5, random_seed=seed),
         GenerationConfig(max_new_tokens=12, ignore_eos=True)])]
    a, b, c = run(1), run(1), run(2)
    assert a == b and a[0] != c[0] and a[1] == c[1]


def test_graph_replay_generates_what_eager_launches_generate(monkeypatch):
    from lmdeploy_b200.messages import GenerationConfig
    from lmdeploy_b200.turbomind.engine import batched_generate
    cfg = LC.config()
    w = LC.random_tensors(cfg, seed=11)
    P = LC.prompts_for(cfg, {"a": 9, "b": 70, "c": 33})
    out = {}
    for graphs in ("0", "1"):
        monkeypatch.setenv("B200_ENGINE_GRAPHS", graphs)
        eng = LC.build_engine(cfg, w, device="cuda", dtype="f32")
        seqs = batched_generate(eng, [P[k] for k in "abc"], GenerationConfig(max_new_tokens=80, ignore_eos=True))
        out[graphs] = [list(s.generated) for s in seqs]
        assert bool(eng._hybrid_graphs) == (graphs == "1")
    assert out["0"] == out["1"]


def _write_checkpoint(folder, cfg, tensors):
    """config.json + model.safetensors (bfloat16) as a Fogizen checkpoint is laid out."""
    import json
    from safetensors.torch import save_file
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))


def test_pipeline_serves_a_checkpoint_folder(tmp_path):
    """pipeline(<folder>) picks the model class by config.json, loads the safetensors and generates what an engine built from
    the same tensors generates; a checkpoint that lacks a tensor is refused by name."""
    import lmdeploy_b200 as lmdeploy
    from lmdeploy_b200.turbomind.engine import batched_generate
    cfg = LC.config()
    w = LC.random_tensors(cfg, seed=12)
    _write_checkpoint(tmp_path, cfg, w)
    P = LC.prompts_for(cfg, {"a": 9, "b": 70})
    gen = lmdeploy.GenerationConfig(max_new_tokens=8, ignore_eos=True)
    ecfg = lmdeploy.TurbomindEngineConfig(max_batch_size=2, session_len=256, cache_max_entry_count=8)
    pipe = lmdeploy.pipeline(str(tmp_path), ecfg)
    assert pipe.engine.hybrid and pipe.engine.spec.arch == "fogizen" and pipe.engine.spec.dtype == "bf16"
    got = [r.token_ids for r in pipe([P["a"], P["b"]], gen)]
    want = [list(s.generated) for s in batched_generate(LC.build_engine(cfg, w, device="cuda", dtype="bf16"), [P["a"], P["b"]], gen)]
    assert got == want and all(len(x) == 8 for x in got)
    bad = tmp_path / "bad"
    bad.mkdir()
    _write_checkpoint(bad, cfg, {k: v for k, v in w.items() if k != "l2.mix.right.w0"})
    with pytest.raises(KeyError, match="l2.mix.right.w0"):
        lmdeploy.pipeline(str(bad), ecfg)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 6e-2)])
def test_trace_runner_replays_a_schedule(tmp_path, dtype, tol):
    """bin/trace_run as a process: three requests over a pool of three pages, portions beside single tokens, a request that sits a
    step out, pages and slots given back at "end" and used again; the logits it writes against the oracle."""
    import json
    import os
    import subprocess
    import sys
    cfg = LC.config()
    w = LC.random_tensors(cfg, seed=13)
    model, out = tmp_path / "model", tmp_path / "out"
    model.mkdir()
    import copy
    bare = copy.deepcopy(cfg)                     # without the decay's inner size: the loader reads it from the tensor's shape
    for e in bare["layers"]:
        del e["mixer"]["right"]["rank"]
    _write_checkpoint(model, bare, w)
    P = LC.prompts_for(cfg, {"a": 100, "b": 6, "c": 64})
    steps = [[("a", 62, [0, 61]), ("b", 2, [1])], [("a", 3, [0, 1, 2]), ("b", 1, [0])], [("b", 3, [2])], [("a", 35, [34]), ("c", 2, [])],
             [("c", 62, [0, 61])], [("b2", 6, [5])]]
    at, lines, asked = {}, [], []
    for k, step in enumerate(steps):
        entries, end = [], []
        for name, count, want in step:
            toks = P[name.rstrip("2")]
            lo = at.get(name, 0)
            at[name] = lo + count
            entries.append({"id": name, "tokens": toks[lo:lo + count], "want": want})
            asked += [(k, name.rstrip("2"), lo + x) for x in want]
            if at[name] == len(toks):
                end.append(name)
        lines.append(json.dumps({"step": k, "entries": entries, "end": end}))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "192"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [x for x in r.stdout.split("\n") if x.startswith("done")] == [f"done {k}" for k in range(len(steps))]
    oracle = {name: LC.oracle_logits(cfg, w, toks) for name, toks in P.items()}
    rows = {}
    for k in range(len(steps)):
        want_here = [(n, p) for kk, n, p in asked if kk == k]
        path = out / f"{k}.f32"
        if not want_here:
            assert not path.exists()
            continue
        got = np.fromfile(path, dtype="<f4").reshape(len(want_here), cfg["vocab"])
        for (n, p), row in zip(want_here, got):
            rows.setdefault(n, []).append((row, oracle[n][p]))
    for n, pairs in rows.items():
        err = LC.rel_error(np.stack([a for a, _ in pairs]), np.stack([b for _, b in pairs]))
        assert err.max() <= tol, (n, err)
