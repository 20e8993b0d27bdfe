"""Fogizen decoders without a GPU: the host side (spec parsing, state and cache offsets, page / slot / row addressing of
turbomind/hybrid.py and the engine) runs the scenarios of tests/fogizen_scenarios.py with the numpy stand-in for the CUDA
library, in float32, against the float64 oracle; and the oracle's own mechanisms are checked on cases worked by hand."""
import math

import pytest
import torch

import fogizen_cases as FC
import fogizen_scenarios as S
from oracle import fogizen as F


def _make(cfg, tensors, **kw):
    return FC.build_engine(cfg, tensors, device="cpu", dtype="f32", emulate=True, **kw)


@pytest.mark.parametrize("scenario", S.ALL, ids=lambda f: f.__name__)
def test_engine_scenario_on_the_emulated_library(scenario):
    scenario(_make, 2e-5)


def test_spec_reads_every_size_from_the_config():
    cfg = FC.config()
    spec = FC.spec_of(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["paired"] * 4 and spec.block == "shared_norm" and spec.plain_norms
    assert spec.layers[1].mlp is None and (spec.layers[2].mlp.kind, spec.layers[2].mlp.ff, spec.layers[2].mlp.act) == ("dense", 40, "xielu")
    f = spec.layers[3].mlp
    assert (f.experts, f.top, f.ff, f.score, f.act, f.grouped, f.correction, f.groups, f.keep, f.group_top, f.renorm, f.scale) == \
        (4, 3, 16, "sigmoid", "silu_gate", True, True, 2, 2, 2, True, 0.5)
    assert (spec.width, spec.vocab, spec.norm_eps) == (48, 61, 1e-5) and (spec.bigram.buckets, spec.bigram.mul_prev, spec.bigram.mul_cur) == (23, 7, 5)
    a = spec.layers[1].mixer.left
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.chunk, a.window, a.span, a.rot.dims, a.rot.base, a.rot.linear) == \
        (4, 1, 12, 6, 0.3, 37, 0, 37, 12, 1000.0, 1.0)
    assert a.head_norm and a.talk_scores and a.sink and a.gate_per_head and a.bias and not a.distance_bias
    assert spec.layers[0].mixer.left.rot.linear == 4.0 and spec.layers[2].mixer.left.chunk == 0
    r = spec.layers[2].mixer.right
    assert (r.heads, r.dim, r.vdim, r.rank) == (4, 33, 33, 8)
    assert FC.spec_of(FC.config(bigram=None)).bigram is None
    # the decay's inner size from a tensor's shape when the config does not carry it
    bare = FC.config()
    for e in bare["layers"]:
        del e["mixer"]["right"]["rank"]
    from lmdeploy_b200.turbomind.specs import fogizen_spec
    assert fogizen_spec(bare, tensor_shapes={f"l{i}.mix.right.w1": (9 + i, 48) for i in range(4)}).layers[3].mixer.right.rank == 12
    with pytest.raises(ValueError):
        fogizen_spec(bare)
    with pytest.raises(NotImplementedError):
        FC.spec_of(FC.config(layers=[{"type": "attention", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError):
        FC.spec_of(FC.config(layers=[FC.layer(FC.left(heads=5, kv_heads=2))]))
    with pytest.raises(ValueError):
        FC.spec_of(FC.config(layers=[FC.layer(FC.left(rot_dims=10))]))
    with pytest.raises(ValueError):
        FC.spec_of(FC.config(layers=[FC.layer(mlp=FC.moe(experts=6, top=5, groups=3, keep=2))]))
    with pytest.raises(ValueError):
        FC.spec_of(FC.config(layers=[FC.layer(mlp=FC.moe(experts=7, groups=3))]))


def test_state_and_cache_geometry():
    cfg = FC.config()
    eng = _make(cfg, FC.random_tensors(cfg))
    model = eng.model
    W = cfg["width"]
    at, want_shift, want_mix = 4, {}, {}                  # the first float of a slot holds the last token's id; three pad it
    for r, e in enumerate(cfg["layers"]):
        want_shift[r] = at
        at += 2 * W
        at = (at + 3) // 4 * 4
        want_mix[r] = at
        at += e["mixer"]["right"]["heads"] * e["mixer"]["right"]["dim"] ** 2
    assert model.token_off == 0 and model.shift_off == want_shift and model.mix_off == want_mix and model.slot_floats == at
    per_run = [64 * e["mixer"]["left"]["kv_heads"] * (e["mixer"]["left"]["dim"] + e["mixer"]["left"]["vdim"]) * 4 for e in cfg["layers"]]
    assert model.block_bytes == sum(per_run)              # float32 keys and values of every layer's attention side
    assert model.w["l0.left.in"].shape == (6 * 8 + 3 * 8 + 3 * 10 + 6, W) and model.w["l0.right.in"].shape == (4, 36, W)
    assert "l0.norm2" not in model.w and "l1.up" not in model.w and model.w["l2.act"].shape == (2,)
    assert torch.equal(model.w["l0.norm1"].cpu(), FC.random_tensors(cfg)["l0.norm1"])        # plain weights: nothing is added


# ------------------------------------------------------------------------------------------------ the oracle on hand-worked cases
def test_oracle_embedding_and_shift():
    cfg = {"embedding": {"bigram": {"buckets": 5, "mul_prev": 3, "mul_cur": 2}}}
    w = {"embed": torch.arange(4.0, dtype=torch.float64)[:, None] * 10, "bigram": torch.arange(6.0, dtype=torch.float64)[:, None]}
    # first token 2: row 5 (the last); then (2 * 3 + 3 * 2) % 5 = 2; then (3 * 3 + 1 * 2) % 5 = 1
    assert F.embed([2, 3, 1], None, w, cfg).reshape(-1).tolist() == [25.0, 32.0, 11.0]
    assert F.embed([3, 1], 2, w, cfg).reshape(-1).tolist() == [32.0, 11.0]
    h = torch.tensor([[1.0, 10.0], [3.0, 30.0]], dtype=torch.float64)
    out = F.shifted(h, torch.tensor([5.0, 50.0], dtype=torch.float64), torch.tensor([0.5, 0.0], dtype=torch.float64))
    assert out.tolist() == [[3.0, 10.0], [2.0, 30.0]]


def test_oracle_rotation_sink_and_chunks():
    v = torch.tensor([[1.0, 0.0, 0.0, 2.0, 5.0, 6.0]], dtype=torch.float64)
    r = F.rotate_pairs(v, 3, 4, 100.0, 2.0)              # pair 0 turns by 3 / 2, pair 1 by 3 / 10 / 2, the last two dimensions stay
    want = [math.cos(1.5), math.sin(1.5), -2 * math.sin(0.15), 2 * math.cos(0.15), 5.0, 6.0]
    assert torch.allclose(r, torch.tensor([want], dtype=torch.float64))
    s = torch.tensor([0.0, math.log(2.0)], dtype=torch.float64)
    assert torch.allclose(F.sink_softmax(s, math.log(5.0)), torch.tensor([0.125, 0.25], dtype=torch.float64))       # 1 / (5 + 1 + 2), 2 / 8
    assert torch.allclose(F.sink_softmax(torch.tensor([800.0, 800.0], dtype=torch.float64), -800.0), torch.tensor([0.5, 0.5], dtype=torch.float64))
    # one head of one dimension, no rotation, identity maps: with chunks of 2 the third token sees only itself
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "scale": 1.0, "rot": {"dims": 0, "base": 10.0}, "mask": {"size": 2}}
    one = lambda x: torch.tensor(x, dtype=torch.float64)
    p = {"q": one([[1.0]]), "k": one([[1.0]]), "v": one([[1.0]]), "q.b": one([0.0]), "k.b": one([0.0]), "v.b": one([0.0]), "q.norm": one([1.0]),
         "k.norm": one([1.0]), "talk": one([[1.0]]), "sink": one([-1e9]), "g": one([[0.0]]), "o": one([[2.0]])}
    out = F.chunk_attention(one([[1.0], [3.0], [5.0]]), p, m, 0.0, [0, 1, 2], F.new_attention_state(m))
    # q = k = 1 after the norm, equal scores: the second token averages values 1 and 3; gate sigmoid(0) = 1/2; output map 2
    assert torch.allclose(out.reshape(-1), one([1.0, 2.0, 5.0]))
    both = F.chunk_attention(one([[1.0], [3.0], [5.0]]), dict(p, talk=one([[0.0]])), dict(m, mask={"size": 0}), 0.0, [0, 1, 2], F.new_attention_state(m))
    assert torch.allclose(both.reshape(-1), one([1.0, 2.0, 3.0]))


def test_oracle_recurrence_of_one_head():
    m = {"heads": 1, "dim": 1}
    one = lambda x: torch.tensor(x, dtype=torch.float64)
    zero = one([0.0])
    # width 1; r = k = v = a (no blending: mu = 0), gate silu(50 a) ~ 50 a, decay exp(-exp(w0)) = 1/2, bonus 3
    p = {"mu.r": zero, "mu.k": zero, "mu.v": zero, "mu.g": zero, "mu.w": zero, "r": one([[1.0]]), "k": one([[1.0]]), "v": one([[1.0]]),
         "g": one([[50.0]]), "w1": one([[0.0]]), "w2": one([[0.0]]), "w0": one([math.log(math.log(2.0))]), "u": one([[3.0]]), "norm": one([1.0]),
         "o": one([[1.0]])}
    st = F.new_recurrence_state(m)
    out = F.decayed_recurrence(one([[1.0], [2.0]]), zero, p, m, 0.0, st)
    # o_1 = 1 * (0 + 3 * 1) = 3, S = 1;  o_2 = 2 * (1 + 3 * 4) = 26, S = 1/2 + 4
    assert abs(float(st["S"][0, 0, 0]) - 4.5) < 1e-12
    assert torch.allclose(out.reshape(-1), one([50.0, 100.0]))             # the unit norm leaves the sign, the gate scales it
    # a blend of one takes the previous row instead: k reads a_(t-1)
    st = F.new_recurrence_state(m)
    F.decayed_recurrence(one([[1.0], [2.0]]), one([7.0]), dict(p, **{"mu.k": one([1.0])}), m, 0.0, st)
    assert abs(float(st["S"][0, 0, 0]) - (0.5 * 7.0 * 1.0 + 1.0 * 2.0)) < 1e-12


def test_oracle_activation_and_router():
    sp = lambda z: math.log1p(math.exp(z))
    got = F.xielu(torch.tensor([2.0, -1.0, 0.0], dtype=torch.float64), torch.tensor([0.3, -0.2], dtype=torch.float64))
    want = [sp(0.3) * 4 + 1.0, (0.5 + sp(-0.2)) * (math.exp(-1.0) - 1 + 1) - 0.5, 0.0]
    assert torch.allclose(got, torch.tensor(want, dtype=torch.float64))
    f = {"router": {"experts": 4, "top": 1, "scale": 2.0, "groups": {"count": 2, "keep": 1}}}
    logit = lambda s: math.log(s / (1 - s))
    p = {"router": torch.tensor([[logit(0.9)], [logit(0.1)], [logit(0.6)], [logit(0.5)]], dtype=torch.float64),
         "correction": torch.zeros(4, dtype=torch.float64)}
    # groups {0, 1}: 1.0 and {2, 3}: 1.1 -> the best single expert is out; one chosen expert's weight is scale * s / s
    (e, wt), = F.route(torch.tensor([1.0], dtype=torch.float64), p, f)
    assert e == 2 and abs(float(wt) - 2.0) < 1e-12
    p["correction"] = torch.tensor([0.0, 0.0, -0.2, 0.0], dtype=torch.float64)
    (e, wt), = F.route(torch.tensor([1.0], dtype=torch.float64), p, f)          # 0.9 + 0.1 = 1.0 against 0.4 + 0.5: group 0 wins on a tie? no: 1.0 > 0.9
    assert e == 0


def test_bench_configuration_builds_a_spec():
    """The sizes bench.py --hybrid-design fogizen runs parse into a spec whose tensors have the expected shapes."""
    import bench
    from lmdeploy_b200.turbomind.hybrid import HybridModel
    from lmdeploy_b200.turbomind.specs import fogizen_spec
    for size, z in bench.HYBRID_SIZES.items():
        spec = fogizen_spec(bench.fogizen_bench_config(z), name=size)
        assert len(spec.layers) == 4 and spec.layers[0].mlp.kind == "dense" and all(l.mlp.kind == "moe" for l in spec.layers[1:])
        shapes = HybridModel.tensor_shapes(FC._Shapes(spec))
        W = z["width"]
        assert shapes["l0.mix.right.w1"] == (64, W) and shapes["l3.mix.left.g"] == (z["dense"]["heads"], W)
        assert shapes["bigram"] == (65522, W) and shapes["l1.mlp.correction"] == (z["experts"],)
