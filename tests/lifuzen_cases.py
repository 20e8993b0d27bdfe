"""Scaffolding of the Lifuzen tests: small configurations with random weights, the engine built on them (on a GPU with the
CUDA library, or on the CPU with tests/hybrid_emulator.py standing in for it) and the same tokens through the plain oracle
(oracle/lifuzen.py, float64).  Schedules are replayed with hybrid_cases.replay."""
import dataclasses

import torch

from hybrid_cases import BLOCK, _Shapes, prompts_for, rel_error, replay  # noqa: F401  (re-exported for the scenarios)
from oracle import lifuzen as L


def attention(heads=6, kv_heads=3, dim=8, taps=3, rot_dims=6, base=100.0, scale=0.7):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": taps, "scale": scale,
                      "rot": {"dims": rot_dims, "base": base}}}


def ssm(heads=4, vdim=6, state=10, groups=2, norm_groups=3, taps=4):
    return {"type": "mamba2",
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": taps}}


def moe(experts=5, top=2, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers=None, width=48, vocab=61, eps=1e-5, loop=(1, 3, 3), mult=0.4, softcap=8.0):
    """A Lifuzen config.json as a dict.  The default stack has a recurrent layer before the loop, a looped pair (attention
    and recurrence, the first without a feed-forward) that runs three times, an attention layer after it; sizes that are
    neither equal to each other nor powers of two, different taps per layer, a router that takes one expert and one that
    takes all."""
    if layers is None:
        layers = [dict(ssm(), mlp=moe()),
                  dict(attention(), mlp=None),
                  dict(ssm(heads=3, vdim=12, state=40, groups=1, norm_groups=1, taps=2), mlp=moe(experts=4, top=1, ff=16)),
                  dict(attention(heads=4, kv_heads=1, dim=12, taps=5, rot_dims=12, base=1000.0, scale=0.3), mlp=moe(experts=3, top=3, ff=8))]
    cfg = {"architecture": "Lifuzen", "layers": layers, "logit_softcap": softcap, "norm": {"eps": eps}, "residual_mult": mult,
           "vocab": vocab, "width": width}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def spec_of(cfg):
    from lmdeploy_b200.turbomind.specs import lifuzen_spec
    return lifuzen_spec(cfg)


def random_tensors(cfg, seed=0):
    """name -> float32 tensor with bf16-representable values (so bf16 and float32 engines and the float64 oracle share them)."""
    from lmdeploy_b200.turbomind.hybrid import HybridModel
    shapes = HybridModel.tensor_shapes(_Shapes(spec_of(cfg)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes.items():
        if name.endswith(("norm1", "norm2", "final.norm")):
            t = 0.3 * torch.randn(shape, generator=g)                       # deviation from one
        elif name.endswith("mix.norm"):
            t = 1.0 + 0.4 * torch.randn(shape, generator=g)
        elif name.endswith(".conv"):
            t = 0.6 * torch.randn(shape, generator=g)
        elif name.endswith(".conv.b"):
            t = 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("A_log"):
            t = torch.log(0.2 + 3.0 * torch.rand(shape, generator=g))
        elif name.endswith("dt_bias"):
            t = torch.randn(shape, generator=g) - 1.0
        elif name.endswith(".D"):
            t = 1.0 + 0.5 * torch.randn(shape, generator=g)
        elif name.endswith("router"):
            t = torch.randn(shape, generator=g)
        elif name == "loop.step":
            t = 0.4 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = 0.5 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / shape[-1] ** 0.5)
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def build_engine(cfg, tensors, *, device, dtype="f32", blocks=8, max_batch=4, emulate=False, prefill_tokens=None):
    """TurboMind over a HybridModel holding `tensors`.  emulate: the numpy stand-in replaces the CUDA library (CPU only)."""
    from lmdeploy_b200 import _hybrid_lib as H
    from lmdeploy_b200.messages import TurbomindEngineConfig
    from lmdeploy_b200.turbomind.engine import TurboMind
    from lmdeploy_b200.turbomind.hybrid import HybridModel
    spec = dataclasses.replace(spec_of(cfg), dtype=dtype)
    real = H.load
    if emulate:
        from hybrid_emulator import EmulatedHybridLib
        H.load = lambda: EmulatedHybridLib()
    try:
        model = HybridModel(spec, block_len=BLOCK, max_batch=max_batch, device=device)
    finally:
        H.load = real
    model.load_weights(lambda k: tensors[k])
    ecfg = TurbomindEngineConfig(cache_max_entry_count=blocks, max_batch_size=max_batch,
                                 session_len=blocks * BLOCK + 1, max_prefill_token_num=prefill_tokens or blocks * BLOCK)
    return TurboMind(spec, ecfg, model=model)


def oracle_logits(cfg, tensors, tokens, trace=None):
    """The whole prompt through the plain implementation in float64 -> [n, vocab]."""
    return L.Decoder(cfg, tensors, torch.float64).forward(list(tokens), trace).numpy()
