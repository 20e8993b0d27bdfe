"""Lifuzen decoders without a GPU: the host side (spec parsing, runs of looped layers, state slots, page / slot / row
addressing of turbomind/hybrid.py and the engine) runs the scenarios of tests/lifuzen_scenarios.py with the numpy stand-in for
the CUDA library, in float32, against the float64 oracle; and the oracle's own mechanisms are checked on cases worked by hand."""
import math

import pytest
import torch

import lifuzen_cases as LC
import lifuzen_scenarios as S
from oracle import lifuzen as L


def _make(cfg, tensors, **kw):
    return LC.build_engine(cfg, tensors, device="cpu", dtype="f32", emulate=True, **kw)


@pytest.mark.parametrize("scenario", S.ALL, ids=lambda f: f.__name__)
def test_engine_scenario_on_the_emulated_library(scenario):
    scenario(_make, 2e-5)


def test_spec_reads_every_size_from_the_config():
    cfg = LC.config()
    spec = LC.spec_of(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["mamba2", "conv_attention", "mamba2", "conv_attention"] and spec.block == "parallel"
    assert spec.layers[1].mlp is None and spec.layers[2].mlp.ff == 16 and spec.layers[0].mlp.kind == "moe"
    f = spec.layers[3].mlp
    assert (f.experts, f.top, f.ff, f.score, f.act, f.scale_input) == (3, 3, 8, "sigmoid", "relu2", True)
    assert (spec.width, spec.vocab, spec.residual_mult, spec.logit_softcap, spec.loop, spec.tied_head) == (48, 61, 0.4, 8.0, (1, 3, 3), True)
    a = spec.layers[3].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.conv_taps, a.scale, a.rot.dims, a.rot.base, a.sink) == (4, 1, 12, 12, 5, 0.3, 12, 1000.0, 0.0)
    m = spec.layers[2].mixer
    assert (m.heads, m.vdim, m.state, m.groups, m.norm_groups, m.conv_taps, m.inner, m.conv_channels, m.proj_cols) == (3, 12, 40, 1, 1, 2, 36, 116, 155)
    assert spec.runs() == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2), (3, None)]
    assert LC.spec_of(LC.config(loop=None)).runs() == [(i, None) for i in range(4)]
    assert LC.spec_of(LC.config(loop=(2, 2, 5))).loop is None
    with pytest.raises(NotImplementedError):
        LC.spec_of(LC.config(layers=[{"type": "lightning", "mixer": {}, "mlp": None}]))
    with pytest.raises(NotImplementedError):
        LC.spec_of(LC.config(layers=[dict(LC.attention(), mlp={"kind": "dense"})]))
    with pytest.raises(ValueError):
        LC.spec_of(LC.config(layers=[dict(LC.attention(heads=5, kv_heads=2), mlp=None)]))
    with pytest.raises(ValueError):
        LC.spec_of(LC.config(layers=[dict(LC.attention(rot_dims=10), mlp=None)]))
    with pytest.raises(ValueError):
        LC.spec_of(LC.config(layers=[dict(LC.ssm(heads=4, groups=3), mlp=None)]))
    with pytest.raises(ValueError):
        LC.spec_of(LC.config(loop=(2, 5, 2)))


def test_runs_own_caches_and_states_layers_own_weights():
    cfg = LC.config()
    eng = _make(cfg, LC.random_tensors(cfg))
    model = eng.model
    assert sorted(model.cache_off) == [1, 3, 5, 7] and len(set(model.cache_off.values())) == 4
    want, at = {}, 0
    for r, (i, _) in enumerate(model.runs):
        e = cfg["layers"][i]
        m = e["mixer"]
        if e["type"] == "attention":
            want[r] = (at, None)
            at += (m["conv"] - 1) * (m["heads"] + m["kv_heads"]) * m["dim"]
        else:
            ch = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
            want[r] = (at, at + (m["conv"] - 1) * ch)
            at += (m["conv"] - 1) * ch + m["heads"] * m["vdim"] * m["state"]
    assert {r: (model.conv_off[r], model.mix_off.get(r)) for r in want} == want and model.slot_floats == at
    per_run = [64 * 2 * m["kv_heads"] * m["dim"] * 4 for m in (cfg["layers"][i]["mixer"] for i, _ in model.runs) if "kv_heads" in m]
    assert model.block_bytes == sum(per_run)          # float32 keys and values of every attention run
    assert model.w["head"] is model.w["embed"] and "l1.gate" not in model.w and "l0.canon1" not in model.w


# ------------------------------------------------------------------------------------------------ the oracle on hand-worked cases
def test_oracle_short_conv_and_rotation():
    u = torch.tensor([[1.0], [10.0], [100.0]], dtype=torch.float64)
    y, keep = L.short_conv(u, torch.tensor([[2.0, 3.0, 5.0]], dtype=torch.float64), torch.tensor([[7.0], [0.5]], dtype=torch.float64),
                           torch.tensor([0.25], dtype=torch.float64))
    # taps [2, 3, 5] weigh the inputs two back, one back and the present one
    assert y.reshape(-1).tolist() == [0.25 + 2 * 7 + 3 * 0.5 + 5 * 1, 0.25 + 2 * 0.5 + 3 * 1 + 5 * 10, 0.25 + 2 * 1 + 3 * 10 + 5 * 100]
    assert keep.reshape(-1).tolist() == [10.0, 100.0]
    v = torch.tensor([[1.0, 0.0, 0.0, 2.0, 5.0, 6.0]], dtype=torch.float64)
    r = L.rotate_pairs(v, 3, 4, 100.0)                   # pair 0 turns by 3, pair 1 by 3 / 10, the last two dimensions stay
    want = [math.cos(3), math.sin(3), -2 * math.sin(0.3), 2 * math.cos(0.3), 5.0, 6.0]
    assert torch.allclose(r, torch.tensor([want], dtype=torch.float64))


def test_oracle_sink_softmax_and_router():
    s = torch.tensor([0.0, math.log(2.0)], dtype=torch.float64)
    assert torch.allclose(L.sink_softmax(s), torch.tensor([0.25, 0.5], dtype=torch.float64))          # 1 / (1 + 1 + 2), 2 / 4
    assert torch.allclose(L.sink_softmax(torch.tensor([-800.0], dtype=torch.float64)), torch.zeros(1, dtype=torch.float64))
    big = L.sink_softmax(torch.tensor([800.0, 800.0], dtype=torch.float64))
    assert torch.allclose(big, torch.tensor([0.5, 0.5], dtype=torch.float64))
    # two experts of one hidden unit each: the chosen one sees score * h, so its output carries the score squared
    p = {"router": torch.tensor([[1.0], [-1.0]], dtype=torch.float64), "e0.up": torch.tensor([[3.0]], dtype=torch.float64),
         "e0.down": torch.tensor([[1.0]], dtype=torch.float64), "e1.up": torch.tensor([[-1.0]], dtype=torch.float64),
         "e1.down": torch.tensor([[10.0]], dtype=torch.float64)}
    f = {"router": {"experts": 2, "top": 1}}
    sc = 1.0 / (1.0 + math.exp(-2.0))
    out = L.routed_ff(torch.tensor([[2.0], [-2.0]], dtype=torch.float64), p, f)
    assert torch.allclose(out, torch.tensor([[(3 * sc * 2) ** 2], [10 * (sc * 2) ** 2]], dtype=torch.float64))


def test_oracle_recurrence_of_one_head():
    m = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "norm_groups": 1, "conv": 1}
    one = lambda v: torch.tensor(v, dtype=torch.float64)
    # projection rows: z | x | B | C | dt picked from a 5-wide input by an identity; conv of one tap with weight 1, no bias
    p = {"in": torch.eye(5, dtype=torch.float64), "conv": torch.ones(3, 1, dtype=torch.float64), "conv.b": torch.zeros(3, dtype=torch.float64),
         "dt_bias": one([0.0]), "A_log": one([0.0]), "D": one([0.5]), "norm": one([1.0]), "o": one([[1.0]])}
    h = one([[50.0, 1.0, 2.0, 3.0, 0.0], [50.0, 1.0, 2.0, 3.0, 0.0]])
    silu = lambda v: v / (1 + math.exp(-v))
    x, B, Cm, dt = silu(1.0), silu(2.0), silu(3.0), math.log(2.0)
    s1 = dt * B * x
    s2 = math.exp(-dt) * s1 + dt * B * x
    y = [s1 * Cm + 0.5 * x, s2 * Cm + 0.5 * x]
    got = L.ssm_mixer(h, p, m, 0.0, L.new_ssm_state(m))
    # silu(50) = 50 scales y, the norm over one channel leaves its sign: +1
    assert torch.allclose(got.reshape(-1), one([1.0, 1.0])) and y[1] > y[0] > 0
    st = L.new_ssm_state(m)
    L.ssm_mixer(h, p, m, 0.0, st)
    assert abs(float(st["S"][0, 0, 0]) - s2) < 1e-12


def test_oracle_layer_runs():
    cfg = {"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}
    assert L.layer_runs(cfg) == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2), (3, None), (4, None)]
    assert L.layer_runs({"layers": [0] * 2}) == [(0, None), (1, None)]
