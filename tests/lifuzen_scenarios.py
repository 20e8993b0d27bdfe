"""Scenarios every engine serving a Lifuzen decoder must pass, whatever runs its operators: `make(cfg, tensors, **kw)` builds
the engine (lifuzen_cases.build_engine with a device, dtype and library chosen by the caller), `tol` bounds
hybrid_cases.rel_error against the float64 oracle.  Run on the CPU through the numpy stand-in (tests/test_lifuzen_cpu.py: host
logic -- runs of looped layers, pages, slots, row addressing, scheduling) and on a GPU through the CUDA kernels
(tests/test_lifuzen_gpu.py)."""
import numpy as np
import torch

import lifuzen_cases as LC
from oracle import lifuzen as L


def _check(got, want, tol, what):
    err = LC.rel_error(got, want)
    assert err.max() <= tol, f"{what}: relative error {err.max():.3g} at position {int(err.argmax())} (bound {tol})"


def _config(make, **kw):
    """LC.config for an engine built by `make`.  A bfloat16 engine's stream differs from the float64 oracle's by rounding, and
    rounding flips a router's choice wherever two logits are close: among hundreds of (position, run) pairs with random weights
    some always are, and a flip moves the logits by their whole size without being a fault.  So engines that say so
    (make.all_experts) get configurations in which every router takes ALL its experts -- the scores still scale the experts'
    inputs --, and the choice itself is tested at that precision on exact inputs (routed_experts_alone) and in float32 everywhere."""
    cfg = LC.config(**kw)
    if getattr(make, "all_experts", False):
        for entry in cfg["layers"]:
            if entry["mlp"] is not None:
                entry["mlp"]["router"]["top"] = entry["mlp"]["router"]["experts"]
    return cfg


def whole_prompt(make, tol):
    """Whole prompts: longer than two pages, a single token, a few tokens."""
    cfg = _config(make)
    w = LC.random_tensors(cfg)
    P = LC.prompts_for(cfg, {"a": 150, "b": 1, "c": 5})
    got = LC.replay(make(cfg, w), P, [[("a", 150)], [("b", 1)], [("c", 5)]])
    for k in P:
        _check(got[k], LC.oracle_logits(cfg, w, P[k]), tol, f"whole prompt {k}")


def layer_by_layer(make, tol):
    """The residual stream after every run (a looped layer counts once per pass) against the oracle's."""
    cfg = _config(make)
    w = LC.random_tensors(cfg, seed=2)
    P = LC.prompts_for(cfg, {"a": 80})
    eng = make(cfg, w)
    eng.layer_trace = []
    LC.replay(eng, P, [[("a", 80)]])
    want = []
    LC.oracle_logits(cfg, w, P["a"], trace=want)
    assert len(eng.layer_trace) == len(want) == 8                     # 1 + 3 x 2 + 1 runs
    for r, (g, x) in enumerate(zip(eng.layer_trace, want)):
        err = float((g.double().cpu() - x).abs().max() / x.abs().max())
        assert err <= tol, f"stream after run {r}: {err:.3g} of its largest value (bound {tol})"


def prefill_then_decode(make, tol, n=200, tail=120):
    """Most of a prompt in one step, the rest token by token: decoded tokens cross page borders (127 -> 128, 191 -> 192), the
    recurrent state is carried over more than a hundred single-token steps."""
    cfg = _config(make)
    w = LC.random_tensors(cfg, seed=3)
    P = LC.prompts_for(cfg, {"a": n})
    got = LC.replay(make(cfg, w), P, [[("a", n - tail)]] + [[("a", 1)]] * tail)
    _check(got["a"], LC.oracle_logits(cfg, w, P["a"]), tol, "prefill then decode")


def token_by_token(make, tol, n=70):
    """Every token alone from the first: the first tokens meet empty conv histories, a zero state and a lone key beside the sink."""
    cfg = _config(make)
    w = LC.random_tensors(cfg, seed=4)
    P = LC.prompts_for(cfg, {"a": n})
    got = LC.replay(make(cfg, w), P, [[("a", 1)]] * n)
    _check(got["a"], LC.oracle_logits(cfg, w, P["a"]), tol, "token by token")


def portions(make, tol):
    """Portions of several sizes down to one and two tokens (shorter than every convolution), cut inside pages and at their borders."""
    cfg = _config(make)
    w = LC.random_tensors(cfg, seed=5)
    cuts = [2, 3, 1, 2, 56, 2, 1, 61, 2, 64, 5, 9, 2, 33]
    P = LC.prompts_for(cfg, {"a": sum(cuts)})
    got = LC.replay(make(cfg, w), P, [[("a", c)] for c in cuts])
    _check(got["a"], LC.oracle_logits(cfg, w, P["a"]), tol, "portions")


def unequal_batch(make, tol):
    """Requests of unequal length in one batch -- portions beside single tokens -- against each alone."""
    cfg = _config(make)
    w = LC.random_tensors(cfg, seed=6)
    P = LC.prompts_for(cfg, {"a": 90, "b": 7, "c": 66, "d": 2})
    sched = [[("a", 30), ("b", 3)], [("b", 1), ("c", 64), ("a", 2)], [("a", 50), ("d", 2), ("c", 1), ("b", 1)],
             [("c", 1), ("a", 1), ("b", 2)], [("a", 7)]]
    got = LC.replay(make(cfg, w), P, sched)
    for k in P:
        _check(got[k], LC.oracle_logits(cfg, w, P[k]), tol, f"batched {k}")


def reuse_of_pages_and_slots(make, tol):
    """A pool of 3 pages and 2 state slots serves requests one after another and side by side: every page and slot is handed
    out again, and a request repeated in a used slot (whose state another request left) gives what it gave in a fresh one."""
    cfg = _config(make)
    w = LC.random_tensors(cfg, seed=7)
    P = LC.prompts_for(cfg, {"a": 100, "b": 20, "c": 64})
    eng = make(cfg, w, blocks=3, max_batch=2)
    sched = [[("a", 64), ("b", 20)], [("a", 36), ("c", 10)], [("c", 54), ("b#2", 5)], [("b#2", 15), ("a#2", 30)], [("a#2", 70)],
             [("c#2", 64), ("b#3", 20)]]
    got = LC.replay(eng, P, sched)
    assert eng.scheduler.alloc.num_free == 3 and sorted(eng.scheduler.slots) == [0, 1]
    for k, v in got.items():
        _check(v, LC.oracle_logits(cfg, w, P[k.split("#")[0]]), tol, f"reuse {k}")


def other_sizes(make, tol):
    """Sizes that a given model may make equal or 1: no loop, a loop of one pass, a loop over every layer, a loop from the first
    layer; one head, as many key/value heads as heads, no convolution (taps 1), every dimension rotated, none rotated; one group,
    as many groups as heads, one norm group, a state narrower than a warp and one wider; one expert, all experts chosen, no
    feed-forward; no cap on the logits, a residual factor of one; a lone layer of each kind."""
    A, M, E = LC.attention, LC.ssm, LC.moe
    stacks = [
        dict(layers=[dict(A(heads=1, kv_heads=1, dim=4, taps=1, rot_dims=0), mlp=None)], width=16, vocab=9, loop=None, softcap=0.0, mult=1.0),
        dict(layers=[dict(M(heads=1, vdim=8, state=3, groups=1, norm_groups=1, taps=1), mlp=E(experts=1, top=1, ff=8))], width=16, vocab=9,
             loop=(0, 1, 1)),
        dict(layers=[dict(A(heads=5, kv_heads=5, dim=6, taps=5, rot_dims=6), mlp=E(experts=4, top=4, ff=12)),
                     dict(M(heads=6, vdim=8, state=33, groups=6, norm_groups=6, taps=3), mlp=None)], width=40, vocab=33, loop=(0, 2, 3)),
        dict(layers=[dict(M(), mlp=E(ff=16)), dict(A(heads=8, kv_heads=2, dim=4, rot_dims=2), mlp=E(experts=7, top=3, ff=10)),
                     dict(M(heads=2, vdim=20, state=70, groups=2, norm_groups=4, taps=2), mlp=None)], width=24, vocab=20, loop=(1, 2, 2)),
        dict(layers=[dict(A(), mlp=None), dict(A(heads=2, kv_heads=1, dim=10, rot_dims=4, taps=2), mlp=E())], width=32, vocab=50, loop=(0, 1, 4)),
    ]
    for k, kw in enumerate(stacks):
        cfg = _config(make, **kw)
        w = LC.random_tensors(cfg, seed=10 + k)
        P = LC.prompts_for(cfg, {"a": 131, "b": 4})
        got = LC.replay(make(cfg, w), P, [[("a", 3)], [("a", 62), ("b", 2)], [("a", 1), ("b", 1)], [("a", 1)], [("a", 62), ("b", 1)], [("a", 1)],
                                          [("a", 1)]])
        for name in P:
            _check(got[name], LC.oracle_logits(cfg, w, P[name]), tol, f"sizes {k} {name}")


def wider_sizes(make, tol):
    """Sizes of the order of a real layer's heads: 16 query heads on 2 key/value heads, head dimensions of 64 and 128 (16-byte
    key reads) and an odd one (scalar reads, a lone last dimension), a state of 128 with value heads of 64, expert widths that are and are not
    multiples of eight (16-byte and scalar weight reads), prompts long enough for the grouped expert GEMMs and for key ranges."""
    A, M, E = LC.attention, LC.ssm, LC.moe
    stacks = [
        dict(layers=[dict(A(heads=16, kv_heads=2, dim=64, taps=4, rot_dims=32, scale=0.125), mlp=E(experts=4, top=2, ff=64)),
                     dict(M(heads=4, vdim=64, state=128, groups=2, norm_groups=2, taps=4), mlp=E(experts=3, top=1, ff=40))],
             width=128, vocab=77, loop=(0, 2, 2)),
        dict(layers=[dict(A(heads=4, kv_heads=4, dim=128, taps=2, rot_dims=64, scale=0.09), mlp=None),
                     dict(M(heads=5, vdim=9, state=17, groups=1, norm_groups=5, taps=3), mlp=E(experts=6, top=2, ff=21)),
                     dict(A(heads=3, kv_heads=1, dim=33, taps=3, rot_dims=10, scale=0.2), mlp=E(experts=2, top=1, ff=32))],
             width=66, vocab=50, loop=None),
    ]
    for k, kw in enumerate(stacks):
        cfg = _config(make, **kw)
        w = LC.random_tensors(cfg, seed=20 + k)
        P = LC.prompts_for(cfg, {"a": 380, "b": 5})
        got = LC.replay(make(cfg, w, blocks=8), P, [[("a", 310), ("b", 2)], [("a", 60), ("b", 1)], [("a", 1), ("b", 2)]] + [[("a", 1)]] * 9)
        for name in P:
            _check(got[name], LC.oracle_logits(cfg, w, P[name]), tol, f"wider sizes {k} {name}")


def greedy_generation(make, tol, new=10):
    """batched_generate (the scheduler's own admission, chunking and retirement, greedy sampling on the device) against the
    oracle generating greedily; a position whose two best oracle logits are closer than the tolerance may differ."""
    from lmdeploy_b200.messages import GenerationConfig
    from lmdeploy_b200.turbomind.engine import batched_generate
    cfg = _config(make)
    w = LC.random_tensors(cfg, seed=8)
    P = LC.prompts_for(cfg, {"a": 9, "b": 70, "c": 1})
    eng = make(cfg, w, blocks=4, max_batch=2, prefill_tokens=32)       # prompts longer than a step's token budget are chunked
    seqs = batched_generate(eng, [P[k] for k in "abc"], GenerationConfig(max_new_tokens=new, ignore_eos=True))
    assert eng.scheduler.alloc.num_free == 4 and sorted(eng.scheduler.slots) == [0, 1]
    for k, s in zip("abc", seqs):
        assert len(s.generated) == new and s.finish_reason == "length"
        toks = list(P[k])
        for i, t in enumerate(s.generated):
            lg = LC.oracle_logits(cfg, w, toks)[-1]
            if int(lg.argmax()) != t:
                assert lg.max() - lg[t] <= 4 * tol * np.abs(lg).max(), f"{k}: token {i} is {t}, oracle {int(lg.argmax())}"
            toks.append(t)


# ------------------------------------------------------------------------------------------------ one mechanism at a time
def _step_arrays(eng, start, n, pages, slot=1):
    """Step arrays of ONE sequence feeding rows [start, start + n), its pages in the given (shuffled) order."""
    from lmdeploy_b200.turbomind.hybrid import StepArrays
    dev = eng.model.device
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    ptrs = torch.tensor([eng.pool.base + b * eng.pool.block_bytes for b in pages], dtype=torch.int64, device=dev)
    return StepArrays(n=n, batch=1, tok_seq=i32([0] * n), tok_pos=i32(list(range(start, start + n))), cu_q=i32([0, n]), seq_slot=i32([slot]),
                      block_ptrs=ptrs, cu_blocks=i32([0, len(pages)]), state=eng.state, max_pos=start + n - 1)


def _close(got, want, tol, what):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert err <= tol, f"{what}: {err:.3g} of the largest value (bound {tol})"


def _mix64(w, i):
    return {k[len(f"l{i}.mix."):]: v.double() for k, v in w.items() if k.startswith(f"l{i}.mix.")}


def _in_portions(eng, h, cuts, pages, run):
    """Feed rows h to a mixer method in portions; -> the output projection's result of all rows."""
    model, at, got = eng.model, 0, []
    eng.state.reset(1)
    for c in cuts:
        c = min(c, h.shape[0] - at)
        if c <= 0:
            break
        x = h[at:at + c].to(model.device, model.T).contiguous()
        y = run(model, x, _step_arrays(eng, at, c, pages))
        got.append(torch.mm(y.float(), model.w["l0.o"].float().t()).cpu())
        at += c
    assert at == h.shape[0]
    return torch.cat(got)


def far_keys_first_tokens_and_the_sink(make, tol, cuts=((330,), (61, 3, 64, 1, 1, 2, 120, 48) + (1,) * 30)):
    """The attention mixer alone, with weights and inputs made so that single scores stand out.  No convolution (taps 1); heads of
    12 dimensions of which the first 4 turn.  Input channels 0..3 are markers: a row marked on channel c (with either sign) gets
    a KEY along dimension 4 + c and a QUERY along dimension 4 + (c + 1) % 4 of every head, so after the unit norm it gives the one
    earlier key marked on channel c + 1 with its sign some nineteen units of score, every other marked key about zero.  All other
    rows carry channel 4, which makes their keys and queries opposite along dimension 8: they give each other some nineteen units
    BELOW zero and marked keys about zero, so their weights are shared between the few marked keys and the sink -- a softmax
    without the sink changes them by a fifth, and the second token's output by half.  A found key's VALUE is the key before the norm,
    whose size differs from mark to mark.  Marked keys sit at the first token and at page borders (63, 64, 127, 128); the queries
    that must find them come hundreds of keys later, in a prompt and decoded alone."""
    cfg = LC.config(layers=[dict(LC.attention(heads=4, kv_heads=2, dim=12, taps=1, rot_dims=4, scale=1.6), mlp=None)], loop=None)
    w = LC.random_tensors(cfg, seed=31)
    m = cfg["layers"][0]["mixer"]
    W = cfg["width"]
    wq, wk = w["l0.mix.q"].view(4, 12, W), w["l0.mix.k"].view(2, 12, W)
    wq *= 0.05
    wk *= 0.05
    wq[:, :, :5] = 0.0
    wk[:, :, :5] = 0.0
    for c in range(4):
        wk[:, 4 + c, c] = 0.5
        wq[:, 4 + (c + 1) % 4, c] = 0.5
    wk[:, 8, 4], wq[:, 8, 4] = 0.5, -0.5
    for k in ("q", "k"):
        w[f"l0.mix.{k}"] = w[f"l0.mix.{k}"].to(torch.bfloat16).float()
        w[f"l0.mix.{k}.conv"].fill_(1.0)
    # (position, channel, size): keys first, then the queries that find them (300 -> 0, 301 -> 63, 302 -> 64, 303 -> 127, 304 -> 128, 329 -> 300)
    marks = [(0, 1, 40.0), (63, 2, 44.0), (64, 3, 36.0), (127, 1, -48.0), (128, 2, -52.0),
             (300, 0, 40.0), (301, 1, 40.0), (302, 2, 40.0), (303, 0, -40.0), (304, 1, -40.0), (329, 3, 40.0)]
    n = 330
    h = 0.2 * torch.randn(n, W, generator=torch.Generator().manual_seed(5))
    h[:, :5] = 0.0
    h[:, 4] = 30.0
    for pos, ch, size in marks:
        h[pos, 4] = 0.0
        h[pos, ch] = size
    h = h.to(torch.bfloat16).to(torch.float32)
    want = L.attention_mixer(h.double(), _mix64(w, 0), m, cfg["norm"]["eps"], list(range(n)), L.new_attention_state(m))
    # the oracle itself: position 300 reads the value of key 0 (0.5 * 40 along dimension 5 of the key's head), nothing else to 1e-3
    st = L.new_attention_state(m)
    L.attention_mixer(h.double(), dict(_mix64(w, 0), o=torch.eye(48, dtype=torch.float64)), m, cfg["norm"]["eps"], list(range(n)), st)
    assert abs(float(st["v"][0, 0, 5]) - 20.0) < 0.1 and abs(float(st["v"][127, 1, 5]) + 24.0) < 0.1
    heads = L.attention_mixer(h.double(), dict(_mix64(w, 0), o=torch.eye(48, dtype=torch.float64)), m, cfg["norm"]["eps"], list(range(n)),
                              L.new_attention_state(m)).reshape(n, 4, 12)
    assert float((heads[300, :, 5] - 20.0).abs().max()) < 0.05 and float((heads[303, :, 5] + 24.0).abs().max()) < 0.05
    assert float((heads[1, :, 5] - 10.0).abs().max()) < 0.3             # the second token: key 0 and the sink share the weight
    for cut in cuts:
        eng = make(cfg, w)
        got = _in_portions(eng, h, cut, [2, 0, 1, 5, 3, 4], lambda model, x, c: model.conv_attention_mixer(0, x, c))
        _close(got, want, tol, f"marked keys, portions {cut[:3]}...")


def recurrence_in_portions(make, tol):
    """The state-space mixer alone over 300 rows: heads whose decay is slow (the state remembers hundreds of rows) and fast,
    step sizes from tiny to large, as one prompt, in portions shorter than the convolution and token by token at the end."""
    cfg = LC.config(layers=[dict(LC.ssm(heads=4, vdim=6, state=40, groups=2, norm_groups=2, taps=4), mlp=None)], loop=None)
    w = LC.random_tensors(cfg, seed=32)
    w["l0.mix.A_log"] = torch.tensor([-6.0, -2.0, 0.5, 1.0]).to(torch.bfloat16).float()
    w["l0.mix.dt_bias"] = torch.tensor([-4.0, 0.0, 1.0, 1.5]).to(torch.bfloat16).float()
    m = cfg["layers"][0]["mixer"]
    n = 300
    h = torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).float()
    want = L.ssm_mixer(h.double(), _mix64(w, 0), m, cfg["norm"]["eps"], L.new_ssm_state(m))
    for cut in ((300,), (2, 1, 3, 1, 1, 60, 2, 5, 130, 64) + (1,) * 31):
        eng = make(cfg, w)
        got = _in_portions(eng, h, cut, [0], lambda model, x, c: model.ssm_mixer(0, x, c))
        _close(got, want, tol, f"recurrence, portions {cut[:3]}...")


def convolved_queries_and_keys_in_portions(make, tol):
    """The attention mixer with convolutions of 5 taps and every dimension rotated, in portions of one to three rows: the history of
    the projected rows is carried in the slot, values are the keys before rotation."""
    cfg = LC.config(layers=[dict(LC.attention(heads=4, kv_heads=2, dim=6, taps=5, rot_dims=6, base=50.0, scale=0.8), mlp=None)], loop=None)
    w = LC.random_tensors(cfg, seed=33)
    m = cfg["layers"][0]["mixer"]
    n = 75
    h = torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).float()
    want = L.attention_mixer(h.double(), _mix64(w, 0), m, cfg["norm"]["eps"], list(range(n)), L.new_attention_state(m))
    for cut in ((75,), (2, 1, 3, 1, 1, 2, 50, 2, 1, 1, 3, 8)):
        eng = make(cfg, w)
        got = _in_portions(eng, h, cut, [1, 0], lambda model, x, c: model.conv_attention_mixer(0, x, c))
        _close(got, want, tol, f"convolved attention, portions {cut[:3]}...")


def routed_experts_alone(make, tol):
    """Sigmoid scores, the `top` largest, each expert fed score * h: few rows (expert-major kernels) and many (grouped GEMMs)
    against the oracle; scores well apart from one so that scaling the input (squared by the activation) differs from
    scaling the output."""
    # the last two: rows so long that eight of them (as float) would crowd an SM's shared memory, first in the up stage, then in the down stage
    for top, experts, ff, n, width in ((2, 5, 24, 6, 48), (1, 3, 10, 5, 48), (3, 3, 16, 200, 48), (2, 4, 9, 260, 48), (2, 3, 24, 11, 2400),
                                       (2, 2, 2400, 11, 48)):
        cfg = LC.config(layers=[dict(LC.ssm(), mlp=LC.moe(experts=experts, top=top, ff=ff))], loop=None, width=width)
        w = LC.random_tensors(cfg, seed=34 + top)
        w["l0.mlp.router"] = (0.15 * w["l0.mlp.router"]).to(torch.bfloat16).float()       # logits of order one: scores between 0 and 1
        eng = make(cfg, w)
        model = eng.model
        h = torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).float()
        p64 = {k[len("l0.mlp."):]: v.double() for k, v in w.items() if k.startswith("l0.mlp.")}
        want = L.routed_ff(h.double(), p64, cfg["layers"][0]["mlp"])
        out = model.routed_experts(0, None, h.to(model.device, model.T).contiguous(), n)
        ids, wts = model.last_routing
        assert float(wts.min()) > 0 and float(wts.max()) < 1 and float((wts - 0.5).abs().max()) > 0.2
        _close(out.sum(1).cpu(), want, tol, f"experts top {top} of {experts}, {n} rows, width {width}, ff {ff}")


def residual_and_two_norms(make, tol):
    """The stream takes in mult * (mixer output + the experts' partial outputs), the embedding output and a pass's vector, then
    both norms (one plus the stored weight) read the same stream."""
    cfg = LC.config(loop=None)
    w = LC.random_tensors(cfg, seed=35)
    eng = make(cfg, w)
    model, lib = eng.model, eng.model.lib
    W, n, eps, mult = cfg["width"], 37, cfg["norm"]["eps"], cfg["residual_mult"]
    g = torch.Generator().manual_seed(9)
    r = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).float()
    x0, mix, ff, add, vec = r(n, W), r(n, W), r(n, 3, W), r(n, W), r(W)
    xs = (x0 + mult * (mix + ff.sum(1)) + add + vec).double()
    dev, T = model.device, model.T
    x = x0.to(dev).contiguous()
    d = [t.to(dev, T).contiguous() for t in (mix, vec)] + [t.to(dev).contiguous() for t in (ff, add)]
    h1, h2 = torch.empty(n, W, dtype=T, device=dev), torch.empty(n, W, dtype=T, device=dev)
    h2f = torch.empty(n, W, dtype=torch.float32, device=dev)
    from lmdeploy_b200 import _hybrid_lib as H
    H.check(lib.b200h_parallel_residual_norm(x.data_ptr(), d[0].data_ptr(), d[2].data_ptr(), 3, mult, d[3].data_ptr(), d[1].data_ptr(),
                                             model.w["l0.norm1"].data_ptr(), model.w["l0.norm2"].data_ptr(), n, W, eps, h1.data_ptr(),
                                             h2.data_ptr(), h2f.data_ptr(), model.dt, model._stream()))
    _close(x.cpu(), xs, 1e-6, "stream after the add")
    _close(h1.float().cpu(), L.offset_norm(xs, w["l0.norm1"].double(), eps), tol, "first norm")
    _close(h2.float().cpu(), L.offset_norm(xs, w["l0.norm2"].double(), eps), tol, "second norm")
    _close(h2f.cpu(), L.offset_norm(xs, w["l0.norm2"].double(), eps), 2e-6, "second norm as float")


def score_scratch_in_row_chunks(make, tol):
    """The rows of a step pass through the attention in chunks when the scratch between its two passes is bounded: chunks of 4
    rows here, cut inside sequences and between them."""
    cfg = _config(make)
    w = LC.random_tensors(cfg, seed=36)
    P = LC.prompts_for(cfg, {"a": 93, "b": 21, "c": 3})
    eng = make(cfg, w)
    eng.model.window_scratch_bytes = 1
    got = LC.replay(eng, P, [[("a", 50), ("b", 21), ("c", 2)], [("a", 43), ("c", 1)]])
    for k in P:
        _check(got[k], LC.oracle_logits(cfg, w, P[k]), tol, f"row chunks {k}")


MECHANISMS = [routed_experts_alone, residual_and_two_norms, recurrence_in_portions, convolved_queries_and_keys_in_portions,
              far_keys_first_tokens_and_the_sink]
ENGINE = [score_scratch_in_row_chunks, whole_prompt, layer_by_layer, prefill_then_decode, token_by_token, portions, unequal_batch,
          reuse_of_pages_and_slots, other_sizes, wider_sizes, greedy_generation]
ALL = MECHANISMS + ENGINE
