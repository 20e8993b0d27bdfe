"""Scenarios every engine serving a Fogizen decoder must pass, whatever runs its operators: `make(cfg, tensors, **kw)` builds
the engine (fogizen_cases.build_engine with a device, dtype and library chosen by the caller), `tol` bounds
hybrid_cases.rel_error against the float64 oracle.  Run on the CPU through the numpy stand-in (tests/test_fogizen_cpu.py: host
logic -- pages, slots, row addressing, scheduling, state offsets) and on a GPU through the CUDA kernels (tests/test_fogizen_gpu.py)."""
import numpy as np
import torch

import fogizen_cases as FC
from oracle import fogizen as F


def _check(got, want, tol, what):
    err = FC.rel_error(got, want)
    assert err.max() <= tol, f"{what}: relative error {err.max():.3g} at position {int(err.argmax())} (bound {tol})"


def _config(make, **kw):
    """FC.config for an engine built by `make`.  A bfloat16 engine's stream differs from the float64 oracle's by rounding, and
    rounding flips a router's choice wherever two choice scores are close: among hundreds of (position, layer) pairs with random
    weights some always are, and a flip moves the logits by their whole size without being a fault.  So engines that say so
    (make.all_experts) get configurations in which every router keeps every group and takes ALL its experts -- the weights are
    still renormalised and scaled --, and the choice itself is tested at that precision on exact inputs (grouped_router_alone)
    and in float32 everywhere."""
    cfg = FC.config(**kw)
    if getattr(make, "all_experts", False):
        for entry in cfg["layers"]:
            if entry["mlp"] is not None and entry["mlp"]["kind"] == "moe":
                r = entry["mlp"]["router"]
                r["top"] = r["experts"]
                if "groups" in r:
                    r["groups"]["keep"] = r["groups"]["count"]
    return cfg


def whole_prompt(make, tol):
    """Whole prompts: longer than two pages and several chunks, a single token, a few tokens."""
    cfg = _config(make)
    w = FC.random_tensors(cfg)
    P = FC.prompts_for(cfg, {"a": 150, "b": 1, "c": 5})
    got = FC.replay(make(cfg, w), P, [[("a", 150)], [("b", 1)], [("c", 5)]])
    for k in P:
        _check(got[k], FC.oracle_logits(cfg, w, P[k]), tol, f"whole prompt {k}")


def layer_by_layer(make, tol):
    """The residual stream after every layer against the oracle's."""
    cfg = _config(make)
    w = FC.random_tensors(cfg, seed=2)
    P = FC.prompts_for(cfg, {"a": 80})
    eng = make(cfg, w)
    eng.layer_trace = []
    FC.replay(eng, P, [[("a", 80)]])
    want = []
    FC.oracle_logits(cfg, w, P["a"], trace=want)
    assert len(eng.layer_trace) == len(want) == 4
    for r, (g, x) in enumerate(zip(eng.layer_trace, want)):
        err = float((g.double().cpu() - x).abs().max() / x.abs().max())
        assert err <= tol, f"stream after layer {r}: {err:.3g} of its largest value (bound {tol})"


def prefill_then_decode(make, tol, n=200, tail=120):
    """Most of a prompt in one step, the rest token by token: decoded tokens cross page borders (127 -> 128, 191 -> 192) and chunk
    edges (99 -> 100, 110 -> 111, 147 -> 148, 149 -> 150, 184 -> 185), the recurrent state and the shifted rows are carried over
    more than a hundred single-token steps."""
    cfg = _config(make)
    w = FC.random_tensors(cfg, seed=3)
    P = FC.prompts_for(cfg, {"a": n})
    got = FC.replay(make(cfg, w), P, [[("a", n - tail)]] + [[("a", 1)]] * tail)
    _check(got["a"], FC.oracle_logits(cfg, w, P["a"]), tol, "prefill then decode")


def token_by_token(make, tol, n=70):
    """Every token alone from the first: the first token blends with zeros, reads the last row of the second table, meets a
    zero state and a lone key beside the sink."""
    cfg = _config(make)
    w = FC.random_tensors(cfg, seed=4)
    P = FC.prompts_for(cfg, {"a": n})
    got = FC.replay(make(cfg, w), P, [[("a", 1)]] * n)
    _check(got["a"], FC.oracle_logits(cfg, w, P["a"]), tol, "token by token")


def portions(make, tol):
    """Portions of several sizes down to one and two tokens (the blends reach two rows back: into the slot), cut inside pages
    and chunks and at their borders."""
    cfg = _config(make)
    w = FC.random_tensors(cfg, seed=5)
    cuts = [2, 3, 1, 2, 29, 13, 14, 2, 1, 33, 28, 2, 64, 5, 9, 2, 33]          # cuts at 37, 50, 64, 100, 128, 192 among others
    P = FC.prompts_for(cfg, {"a": sum(cuts)})
    got = FC.replay(make(cfg, w), P, [[("a", c)] for c in cuts])
    _check(got["a"], FC.oracle_logits(cfg, w, P["a"]), tol, "portions")


def unequal_batch(make, tol):
    """Requests of unequal length in one batch -- portions beside single tokens -- against each alone."""
    cfg = _config(make)
    w = FC.random_tensors(cfg, seed=6)
    P = FC.prompts_for(cfg, {"a": 90, "b": 7, "c": 66, "d": 2})
    sched = [[("a", 30), ("b", 3)], [("b", 1), ("c", 64), ("a", 2)], [("a", 50), ("d", 2), ("c", 1), ("b", 1)],
             [("c", 1), ("a", 1), ("b", 2)], [("a", 7)]]
    got = FC.replay(make(cfg, w), P, sched)
    for k in P:
        _check(got[k], FC.oracle_logits(cfg, w, P[k]), tol, f"batched {k}")


def reuse_of_pages_and_slots(make, tol):
    """A pool of 3 pages and 2 state slots serves requests one after another and side by side: every page and slot is handed
    out again, and a request repeated in a used slot (whose state, shifted rows and last token another request left) gives what
    it gave in a fresh one."""
    cfg = _config(make)
    w = FC.random_tensors(cfg, seed=7)
    P = FC.prompts_for(cfg, {"a": 100, "b": 20, "c": 64})
    eng = make(cfg, w, blocks=3, max_batch=2)
    sched = [[("a", 64), ("b", 20)], [("a", 36), ("c", 10)], [("c", 54), ("b#2", 5)], [("b#2", 15), ("a#2", 30)], [("a#2", 70)],
             [("c#2", 64), ("b#3", 20)]]
    got = FC.replay(eng, P, sched)
    assert eng.scheduler.alloc.num_free == 3 and sorted(eng.scheduler.slots) == [0, 1]
    for k, v in got.items():
        _check(v, FC.oracle_logits(cfg, w, P[k.split("#")[0]]), tol, f"reuse {k}")


def other_sizes(make, tol):
    """Sizes that a given model may make equal or 1: one layer; one head on each side; as many key/value heads as heads; value
    heads wider and narrower than key heads; every dimension rotated, none rotated; no scaling factor; no chunks, chunks of one
    position, chunks of a page, chunks longer than the prompt; a recurrence wider than a warp and narrower, wider than 128 channels,
    with states that are not 16-byte aligned; an inner decay size of 1; one expert, all experts chosen, one group, as many groups as experts, every group kept; no feed-forward; no second
    embedding table; multipliers larger than the table."""
    L, Lf, R, E, D = FC.layer, FC.left, FC.right, FC.moe, FC.dense
    stacks = [
        dict(layers=[L(Lf(heads=1, kv_heads=1, dim=4, vdim=4, chunk=1, rot_dims=0, factor=None), R(heads=1, dim=4, rank=1))], width=16, vocab=9,
             bigram=None),
        dict(layers=[L(Lf(heads=5, kv_heads=5, dim=6, vdim=3, chunk=64, rot_dims=6, factor=1.0), R(heads=1, dim=40, rank=2),
                       mlp=E(experts=1, top=1, ff=8, groups=1, keep=1))], width=16, vocab=9, bigram=(3, 1000003, 999983)),
        dict(layers=[L(Lf(heads=8, kv_heads=2, dim=4, vdim=9, chunk=1000, rot_dims=2), R(heads=6, dim=3, rank=4), mlp=E(experts=4, top=4, ff=12, groups=4, keep=4)),
                     L(mlp=D(ff=7)), L(Lf(chunk=0), mlp=E(experts=8, top=2, ff=10, groups=0))], width=40, vocab=33, bigram=(1, 1, 1)),
        dict(layers=[L(mlp=D()), L(Lf(heads=2, kv_heads=1, dim=10, vdim=10, chunk=3, rot_dims=4, factor=8.0), R(heads=2, dim=64, rank=6),
                       mlp=E(experts=6, top=1, ff=16, groups=6, keep=1))], width=24, vocab=20),
        # a width that leaves the recurrent states unaligned for 16-byte reads; heads wider than 128 channels (a warp per pair of columns)
        dict(layers=[L(r=R(heads=1, dim=130, rank=3)), L(r=R(heads=2, dim=36, rank=2), mlp=D(ff=9))], width=33, vocab=20),
    ]
    for k, kw in enumerate(stacks):
        cfg = _config(make, **kw)
        w = FC.random_tensors(cfg, seed=10 + k)
        P = FC.prompts_for(cfg, {"a": 131, "b": 4})
        got = FC.replay(make(cfg, w), P, [[("a", 3)], [("a", 62), ("b", 2)], [("a", 1), ("b", 1)], [("a", 1)], [("a", 62), ("b", 1)], [("a", 1)],
                                          [("a", 1)]])
        for name in P:
            _check(got[name], FC.oracle_logits(cfg, w, P[name]), tol, f"sizes {k} {name}")


def wider_sizes(make, tol):
    """Sizes of the order of a real layer's heads: 16 query heads on 2 key/value heads, head dimensions of 64 and 128 (16-byte
    key reads) and an odd one (scalar reads), recurrences of 64 and 128 channels per head, expert widths that are and are not
    multiples of eight, prompts long enough for the grouped expert GEMMs and for key ranges, chunks of 256 and of 100."""
    L, Lf, R, E, D = FC.layer, FC.left, FC.right, FC.moe, FC.dense
    stacks = [
        dict(layers=[L(Lf(heads=16, kv_heads=2, dim=64, vdim=64, chunk=256, rot_dims=32, scale=0.125), R(heads=4, dim=64, rank=16),
                       mlp=E(experts=4, top=2, ff=64, groups=2, keep=1)),
                     L(Lf(heads=4, kv_heads=4, dim=128, vdim=32, chunk=0, rot_dims=128, scale=0.09), R(heads=2, dim=128, rank=8), mlp=D(ff=96))],
             width=128, vocab=77),
        dict(layers=[L(Lf(heads=3, kv_heads=1, dim=33, vdim=5, chunk=100, rot_dims=10, scale=0.2), R(heads=5, dim=9, rank=3),
                       mlp=E(experts=6, top=2, ff=21, groups=3, keep=2))], width=66, vocab=50),
    ]
    for k, kw in enumerate(stacks):
        cfg = _config(make, **kw)
        w = FC.random_tensors(cfg, seed=20 + k)
        P = FC.prompts_for(cfg, {"a": 380, "b": 5})
        got = FC.replay(make(cfg, w, blocks=8), P, [[("a", 310), ("b", 2)], [("a", 60), ("b", 1)], [("a", 1), ("b", 2)]] + [[("a", 1)]] * 9)
        for name in P:
            _check(got[name], FC.oracle_logits(cfg, w, P[name]), tol, f"wider sizes {k} {name}")


def greedy_generation(make, tol, new=10):
    """batched_generate (the scheduler's own admission, chunking and retirement, greedy sampling on the device) against the
    oracle generating greedily; a position whose two best oracle logits are closer than the tolerance may differ."""
    from lmdeploy_b200.messages import GenerationConfig
    from lmdeploy_b200.turbomind.engine import batched_generate
    cfg = _config(make)
    w = FC.random_tensors(cfg, seed=8)
    P = FC.prompts_for(cfg, {"a": 9, "b": 70, "c": 1})
    eng = make(cfg, w, blocks=4, max_batch=2, prefill_tokens=32)       # prompts longer than a step's token budget are chunked
    seqs = batched_generate(eng, [P[k] for k in "abc"], GenerationConfig(max_new_tokens=new, ignore_eos=True))
    assert eng.scheduler.alloc.num_free == 4 and sorted(eng.scheduler.slots) == [0, 1]
    for k, s in zip("abc", seqs):
        assert len(s.generated) == new and s.finish_reason == "length"
        toks = list(P[k])
        for i, t in enumerate(s.generated):
            lg = FC.oracle_logits(cfg, w, toks)[-1]
            if int(lg.argmax()) != t:
                assert lg.max() - lg[t] <= 4 * tol * np.abs(lg).max(), f"{k}: token {i} is {t}, oracle {int(lg.argmax())}"
            toks.append(t)


def score_scratch_in_row_chunks(make, tol):
    """The rows of a step pass through the attention in chunks when the scratch between its passes is bounded: chunks of 4
    rows here, cut inside sequences and between them; the scores are mixed across heads chunk by chunk."""
    cfg = _config(make)
    w = FC.random_tensors(cfg, seed=36)
    P = FC.prompts_for(cfg, {"a": 93, "b": 21, "c": 3})
    eng = make(cfg, w)
    eng.model.window_scratch_bytes = 1
    got = FC.replay(eng, P, [[("a", 50), ("b", 21), ("c", 2)], [("a", 43), ("c", 1)]])
    for k in P:
        _check(got[k], FC.oracle_logits(cfg, w, P[k]), tol, f"row chunks {k}")


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


def _sub64(w, prefix):
    return {k[len(prefix):]: v.double() for k, v in w.items() if k.startswith(prefix)}


def _in_portions(eng, n, cuts, pages, run):
    """Call run(model, lo, hi, step arrays) over rows [0, n) in portions; -> the concatenated results (on the CPU)."""
    at, got = 0, []
    eng.state.reset(1)
    for c in cuts:
        c = min(c, n - at)
        if c <= 0:
            break
        got.append(run(eng.model, at, at + c, _step_arrays(eng, at, c, pages)).float().cpu())
        at += c
    assert at == n
    return torch.cat(got)


def marked_keys_chunk_edges_and_sinks(make, tol, cuts=((230,), (61, 3, 35, 1, 1, 26, 1, 22, 45) + (1,) * 35)):
    """The attention side alone, with weights and inputs made so that single scores stand out.  Heads of 12 dimensions of which the
    first 4 turn; chunks of 100 positions.  Input channels 0..3 are markers: a row marked on channel c gets a KEY along dimension
    4 + c and a QUERY along dimension 4 + (c + 1) % 4 of every head, so after the per-head norm it gives every visible key marked on
    channel c + 1 some nineteen units of score and every other marked key about zero.  All other rows carry channel 4, which makes
    their keys and queries opposite along dimension 8: they give each other nineteen units BELOW zero, so their weights are shared
    between the few marked keys of their chunk and the sink.  Marked keys sit at a sequence's first token, at page borders
    (63, 64, 127, 128) and on both sides of the chunk edges (99 | 100, 199 | 200); the queries that must find them -- or must NOT,
    by one position -- come up to 99 keys later, in a prompt and decoded alone.  The oracle itself is checked for showing the
    fault: without chunks, with chunks one position longer or shorter, or without the sink its answer at those rows moves by a large part."""
    cfg = FC.config(layers=[FC.layer(FC.left(heads=4, kv_heads=2, dim=12, vdim=8, chunk=100, rot_dims=4, scale=1.6, factor=2.0))])
    w = FC.random_tensors(cfg, seed=31)
    m = cfg["layers"][0]["mixer"]["left"]
    W = cfg["width"]
    pre = "l0.mix.left."
    wq, wk = w[pre + "q"].view(4, 12, W), w[pre + "k"].view(2, 12, W)
    wq *= 0.05
    wk *= 0.05
    wq[:, :, :5] = 0.0
    wk[:, :, :5] = 0.0
    for c in range(4):
        wk[:, 4 + c, c] = 0.5
        wq[:, 4 + (c + 1) % 4, c] = 0.5
    wk[:, 8, 4], wq[:, 8, 4] = 0.5, -0.5
    for k in ("q", "k"):
        w[pre + k] = w[pre + k].to(torch.bfloat16).float()
        w[pre + k + ".b"] *= 0.05
        w[pre + k + ".norm"] = (1.0 + 0.05 * (w[pre + k + ".norm"] - 1.0)).to(torch.bfloat16).float()
    w[pre + "talk"] = (torch.eye(4) + 0.1 * (w[pre + "talk"] - torch.eye(4))).to(torch.bfloat16).float()
    w[pre + "sink"] = torch.tensor([0.0, 1.0, -1.0, 2.0])
    # (position, channel, size): a query marked c finds the visible keys marked c + 1
    marks = [(0, 1, 40.0), (63, 2, 44.0), (64, 3, 36.0), (99, 1, -48.0),                       # chunk 0: keys
             (90, 0, 40.0), (91, 1, 40.0), (92, 2, 40.0),                                      #   90 -> 0;  91 -> 63;  92 -> 64
             (100, 1, 52.0), (127, 2, -48.0), (128, 3, -52.0),                                 # chunk 1: keys
             (150, 0, 40.0), (151, 1, 40.0), (152, 2, -40.0), (199, 0, 40.0),                  #   150 -> 100, NOT 99 or 0;  151 -> 127;  152 -> 128;  199 -> 100
             (200, 0, 40.0), (201, 3, 40.0), (229, 3, 40.0)]                                  # chunk 2: 200 -> nothing (not 100);  201, 229 -> 200, NOT 199
    n = 230
    h = 0.2 * torch.randn(n, W, generator=torch.Generator().manual_seed(5))
    h[:, :5] = 0.0
    h[:, 4] = 30.0
    for pos, ch, size in marks:
        h[pos, 4] = 0.0
        h[pos, ch] = size
    # channel 5 reaches the values only (queries and keys read it a hundred times weaker than a marker): neighbouring marked keys
    # carry it with opposite signs, so that a weight that goes to the wrong one of them shows in the output
    for pos, tag in ((0, 30.0), (63, -30.0), (64, 30.0), (99, 30.0), (100, -30.0), (127, 30.0), (128, -30.0), (199, 30.0), (200, -30.0)):
        h[pos, 5] = tag
    h = h.to(torch.bfloat16).to(torch.float32)
    eps = cfg["norm"]["eps"]

    def oracle(mm, p=None):
        return F.chunk_attention(h.double(), p or _sub64(w, pre), mm, eps, list(range(n)), F.new_attention_state(mm))

    want = oracle(m)
    size = lambda t: float(t.abs().max())
    for other, rows in ((dict(m, mask={"size": 0}), [150, 200, 201]), (dict(m, mask={"size": 101}), [199, 201]), (dict(m, mask={"size": 99}), [199, 229])):
        moved = oracle(other)
        for r in rows:
            assert size(moved[r] - want[r]) > 0.2 * size(want[r]), f"the oracle does not show chunks of {other['mask']['size']} at row {r}"
    no_sink = oracle(m, dict(_sub64(w, pre), sink=torch.full((4,), -30.0, dtype=torch.float64)))
    assert size(no_sink[200] - want[200]) > 0.2 * size(want[200]) and size(no_sink[1] - want[1]) > 0.1 * size(want[1])
    for cut in cuts:
        eng = make(cfg, w)

        def run(model, lo, hi, c):
            y = model.window_mixer(0, h[lo:hi].to(model.device, model.T).contiguous(), c, m=model.spec.layers[0].mixer.left, p="l0.left.")
            return torch.mm(y.float(), model.w["l0.left.o"].float().t())

        got = _in_portions(eng, n, cut, [2, 0, 1, 3], run)
        _close(got, want, tol, f"marked keys, portions {cut[:3]}...")


def recurrence_in_portions(make, tol):
    """The recurrent side alone over 300 rows: channels whose decay is slow (the state remembers hundreds of rows) and fast, as one
    prompt, in portions of one to three rows and token by token at the end; the five blends come from the token-shift operator,
    whose previous rows live in the slot."""
    cfg = FC.config(layers=[FC.layer(r=FC.right(heads=3, dim=40, rank=4))])
    w = FC.random_tensors(cfg, seed=32)
    pre = "l0.mix.right."
    w[pre + "w0"] = torch.linspace(-7.0, 1.0, 120).to(torch.bfloat16).float()             # decays from 0.999 to 0.066 per row
    m = cfg["layers"][0]["mixer"]["right"]
    n, W, eps = 300, cfg["width"], cfg["norm"]["eps"]
    a = torch.randn(n, W, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).float()
    want = F.decayed_recurrence(a.double(), torch.zeros(W, dtype=torch.float64), _sub64(w, pre), m, eps, F.new_recurrence_state(m))
    from lmdeploy_b200 import _hybrid_lib as H
    for cut in ((300,), (2, 1, 3, 1, 1, 60, 2, 5, 130, 64) + (1,) * 31):
        eng = make(cfg, w)

        def run(model, lo, hi, c):
            # the blends of rows a (no shift: a is the mixer's input itself) through the operator that owns the previous rows
            k = hi - lo
            blends = torch.empty(5, k, W, dtype=model.T, device=model.device)
            hf = a[lo:hi].to(model.device).contiguous()
            H.check(model.lib.b200h_token_shift(hf.data_ptr(), None, model.w["l0.right.mu"].data_ptr(), 5, c.state.ptr(model.shift_off[0]),
                                                c.state.storage.stride(0), c.tok_seq.data_ptr(), c.cu_q.data_ptr(), c.seq_slot.data_ptr(),
                                                k, 1, W, None, blends.data_ptr(), model.dt, model._stream()))
            y = model.channel_decay_mixer(0, blends, c, m=model.spec.layers[0].mixer.right, p="l0.right.")
            return torch.mm(y.float(), model.w["l0.right.o"].float().t())

        got = _in_portions(eng, n, cut, [0], run)
        _close(got, want, tol, f"recurrence, portions {cut[:3]}...")


def token_shift_in_portions(make, tol):
    """The token shift alone: the shifted row and the five blends against the oracle's, in portions of one, two and three rows
    (a blend reaches two normed rows back: one or both of them in the slot) and restarted in a slot another sequence used."""
    cfg = FC.config(layers=[FC.layer()])
    w = FC.random_tensors(cfg, seed=33)
    n, W = 41, cfg["width"]
    hn = torch.randn(n, W, generator=torch.Generator().manual_seed(7))
    shift, mu = w["l0.shift"].double(), torch.stack([w["l0.mix.right.mu." + k] for k in "rkvgw"]).double()
    a = F.shifted(hn.double(), torch.zeros(W, dtype=torch.float64), shift)
    want = torch.stack([F.shifted(a, torch.zeros(W, dtype=torch.float64), mu[k]) for k in range(5)], 1)         # [n, 5, W]
    from lmdeploy_b200 import _hybrid_lib as H
    eng = make(cfg, w)
    for cut in ((41,), (1, 1, 2, 1, 3, 2, 1, 1, 20, 2, 7), (2, 39)):

        def run(model, lo, hi, c):
            k = hi - lo
            out_a = torch.empty(k, W, dtype=model.T, device=model.device)
            blends = torch.empty(5, k, W, dtype=model.T, device=model.device)
            hf = hn[lo:hi].to(model.device).contiguous()
            H.check(model.lib.b200h_token_shift(hf.data_ptr(), model.w["l0.shift"].data_ptr(), model.w["l0.right.mu"].data_ptr(), 5,
                                                c.state.ptr(model.shift_off[0]), c.state.storage.stride(0), c.tok_seq.data_ptr(),
                                                c.cu_q.data_ptr(), c.seq_slot.data_ptr(), k, 1, W, out_a.data_ptr(), blends.data_ptr(),
                                                model.dt, model._stream()))
            return torch.cat([out_a[:, None], blends.transpose(0, 1)], 1)

        got = _in_portions(eng, n, cut, [0], run)
        _close(got[:, 0], a, tol, f"shifted rows, portions {cut[:3]}...")
        _close(got[:, 1:], want, tol, f"blends, portions {cut[:3]}...")


def grouped_router_alone(make, tol):
    """The router on inputs made so that its rules show: the input is one-hot times a size, so a row's logits are a column of
    the router matrix.  Row 0: the correction changes the choice but not the weights.  Row 1: the best single expert sits in a
    group that loses on the sum of its two best.  Row 2: every choice score is negative (sigmoid near 0 plus a negative
    correction), and an excluded group's experts must not come back as zeros.  Row 3: a tie between two experts goes to the
    lower index.  Then random rows against the oracle, few (expert-major kernels) and many (grouped GEMMs)."""
    cfg = FC.config(layers=[FC.layer(mlp=FC.moe(experts=6, top=2, ff=24, groups=3, keep=2, scale=1.5))], width=48)
    w = FC.random_tensors(cfg, seed=34)
    W = cfg["width"]
    logit = lambda s: float(np.log(s / (1.0 - s)))
    cols = torch.zeros(6, W)
    # scores s per expert for rows 0..3 (groups: {0,1}, {2,3}, {4,5})
    rows = [[0.70, 0.10, 0.60, 0.10, 0.50, 0.55],          # expert 4 gains 0.5 for the choice: groups .8 | .7 | 1.55 -> experts 4, 0 with weights from .5, .7
            [0.95, 0.05, 0.60, 0.55, 0.50, 0.52],          # group sums 1.0 | 1.15 | 1.52 -> {2,3} and {4,5} stay, expert 0 (.95) is out: 4, 2
            [0.02, 0.01, 0.03, 0.01, 0.02, 0.04],          # -> 4, 5
            [0.30, 0.30, 0.20, 0.10, 0.05, 0.05]]          # groups .6 | .3 | .6: both stay; after expert 4, experts 0 and 1 tie: 0
    for r, scores in enumerate(rows):
        cols[:, r] = torch.tensor([logit(s) for s in scores])
    w["l0.mlp.router"] = cols.to(torch.bfloat16).float()
    w["l0.mlp.correction"] = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.5, 0.0])
    special = torch.zeros(4, W)
    for r in range(4):
        special[r, r] = 1.0
    eng = make(cfg, w)
    model = eng.model
    f = cfg["layers"][0]["mlp"]
    p64 = _sub64(w, "l0.mlp.")

    def routed(h, corr=None):
        if corr is not None:
            model.w["l0.correction"].copy_(corr)
        out = model.routed_experts(0, h.to(model.device).contiguous(), h.to(model.device, model.T).contiguous(), h.shape[0])
        ids, wts = model.last_routing
        return out.sum(1).cpu(), ids.cpu().tolist(), wts.cpu()

    _, ids, wts = routed(special)
    assert [sorted(r) for r in ids] == [[0, 4], [2, 4], [4, 5], [0, 4]], ids
    s64 = torch.sigmoid(w["l0.mlp.router"].double()[:, :4]).T                                    # [row, expert]
    for r in range(4):
        pair = torch.tensor([float(s64[r, e]) for e in ids[r]])
        _close(wts[r], 1.5 * pair / pair.sum(), 1e-5, f"weights of row {r}")
    # row 2 with a correction that makes every choice score negative: same choice within the kept groups, same weights
    _, ids_neg, wts_neg = routed(special, torch.tensor([-1.0, -1.0, -1.0, -1.0, -0.5, -1.0]))
    assert sorted(ids_neg[2]) == [4, 5] and sorted(ids_neg[1]) == [2, 4], ids_neg
    routed(special, w["l0.mlp.correction"])
    for n in (7, 200):
        h = torch.randn(n, W, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).float()
        got, _, _ = routed(h)
        _close(got, F.routed_ff(h.double(), p64, f), tol, f"experts on {n} rows")


def dense_activation_alone(make, tol):
    """The dense feed-forward alone: both branches of the activation, its two learned numbers of either sign."""
    for act in ([0.4, -0.8], [-2.0, 3.0]):
        cfg = FC.config(layers=[FC.layer(mlp=FC.dense(ff=37))])
        w = FC.random_tensors(cfg, seed=35)
        w["l0.mlp.act"] = torch.tensor(act).to(torch.bfloat16).float()
        h = 2.0 * torch.randn(50, cfg["width"], generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).float()
        model = make(cfg, w).model
        got = model.dense_mlp(0, h.to(model.device, model.T).contiguous())
        z = h.double() @ w["l0.mlp.up"].double().T
        assert float((z > 1).double().mean()) > 0.1 and float((z < -1).double().mean()) > 0.1
        _close(got.float().cpu(), F.dense_ff(h.double(), _sub64(w, "l0.mlp.")), tol, f"dense feed-forward, act {act}")


def side_norms_and_residual(make, tol):
    """The stream takes in half the sum of the two sides, each normed over the width with its own weight, and the feed-forward's
    parts (as T or as float); then the next norm reads it."""
    cfg = FC.config()
    w = FC.random_tensors(cfg, seed=37)
    model = make(cfg, w).model
    W, n, eps = cfg["width"], 37, cfg["norm"]["eps"]
    g = torch.Generator().manual_seed(9)
    r = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).float()
    x0, lf, rt, ff = r(n, W), 4.0 * r(n, W), 0.25 * r(n, W), r(n, 3, W)          # powers of two keep the values in bfloat16
    wl, wr, wn = w["l0.mix.left.out"].double(), w["l0.mix.right.out"].double(), w["l1.norm1"].double()
    xs = x0.double() + 0.5 * (F.unit_rms(lf.double(), eps) * wl + F.unit_rms(rt.double(), eps) * wr) + ff.double().sum(1)
    dev, T = model.device, model.T
    from lmdeploy_b200 import _hybrid_lib as H
    for as_float in (1, 0):
        x = x0.clone().to(dev).contiguous()
        d = [t.to(dev, T).contiguous() for t in (lf, rt)] + [ff.to(dev, torch.float32 if as_float else T).contiguous()]
        h, hf = torch.empty(n, W, dtype=T, device=dev), torch.empty(n, W, dtype=torch.float32, device=dev)
        H.check(model.lib.b200h_branch_residual_norm(x.data_ptr(), d[0].data_ptr(), d[1].data_ptr(), model.w["l0.left.out"].data_ptr(),
                                                     model.w["l0.right.out"].data_ptr(), 0.5, d[2].data_ptr(), as_float, 3,
                                                     model.w["l1.norm1"].data_ptr(), n, W, eps, h.data_ptr(), hf.data_ptr(), model.dt,
                                                     model._stream()))
        _close(x.cpu(), xs, 2e-6, "stream after the add")
        _close(hf.cpu(), F.unit_rms(xs, eps) * wn, 2e-6, "norm as float")
        _close(h.float().cpu(), F.unit_rms(xs, eps) * wn, tol, "norm")


def hashed_embedding_in_portions(make, tol):
    """The two-table embedding alone: the first token reads the last row, every other the row its predecessor and itself hash
    to -- also when the predecessor came in an earlier step (the slot keeps it), with multipliers whose products pass 2^31."""
    cfg = FC.config(layers=[FC.layer()], vocab=50000, bigram=(101, 1000003, 70001), width=16)
    w = FC.random_tensors(cfg, seed=38)
    toks = [49999, 3, 49998, 49999, 0, 7, 7, 31000, 12, 49999, 49997]
    want = F.embed(toks, None, {k: v.double() for k, v in w.items()}, cfg)
    eng = make(cfg, w)
    from lmdeploy_b200 import _hybrid_lib as H
    for cut in ((11,), (1, 1, 2, 1, 3, 2, 1)):

        def run(model, lo, hi, c):
            k = hi - lo
            x = torch.empty(k, 16, dtype=torch.float32, device=model.device)
            t = torch.tensor(toks[lo:hi], dtype=torch.int32, device=model.device)
            H.check(model.lib.b200h_embed_hashed(t.data_ptr(), model.w["embed"].data_ptr(), model.w["bigram"].data_ptr(), 101, 1000003, 70001,
                                                 c.state.ptr(model.token_off), c.state.storage.stride(0), c.tok_seq.data_ptr(),
                                                 c.tok_pos.data_ptr(), c.cu_q.data_ptr(), c.seq_slot.data_ptr(), x.data_ptr(), k, 1, 16,
                                                 model.dt, model._stream()))
            return x

        _close(_in_portions(eng, 11, cut, [0], run), want, 1e-6, f"embedding, portions {cut[:3]}...")


MECHANISMS = [hashed_embedding_in_portions, side_norms_and_residual, token_shift_in_portions, dense_activation_alone, grouped_router_alone,
              recurrence_in_portions, marked_keys_chunk_edges_and_sinks]
ENGINE = [score_scratch_in_row_chunks, whole_prompt, layer_by_layer, prefill_then_decode, token_by_token, portions, unequal_batch,
          reuse_of_pages_and_slots, other_sizes, wider_sizes, greedy_generation]
ALL = MECHANISMS + ENGINE
