"""Scaffolding of the Fogizen tests: small configurations with random weights, the engine built on them (on a GPU with the
CUDA library, or on the CPU with tests/hybrid_emulator.py standing in for it) and the same tokens through the plain oracle
(oracle/fogizen.py, float64).  Schedules are replayed with hybrid_cases.replay."""
import dataclasses

import torch

from hybrid_cases import BLOCK, _Shapes, prompts_for, rel_error, replay  # noqa: F401  (re-exported for the scenarios)
from oracle import fogizen as F


def left(heads=6, kv_heads=3, dim=8, vdim=10, chunk=50, rot_dims=6, base=100.0, factor=4.0, scale=0.7):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot_dims, "base": base}}
    if chunk:
        m["mask"] = {"size": chunk}
    if factor is not None:
        m["rot"]["scaling"] = {"factor": factor}
    return m


def right(heads=3, dim=12, rank=5):
    return {"heads": heads, "dim": dim, "rank": rank}


def layer(l=None, r=None, mlp=None):
    return {"type": "parallel", "mixer": {"left": l or left(), "right": r or right()}, "mlp": mlp}


def moe(experts=6, top=2, ff=24, groups=3, keep=2, scale=1.5):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def config(layers=None, width=48, vocab=61, eps=1e-5, bigram=(23, 7, 5)):
    """A Fogizen config.json as a dict.  The default stack: a routed layer first, a layer without a feed-forward, a dense one and a
    routed one whose router keeps every group; sizes that are neither equal to each other nor powers of two, chunks of different
    lengths that are not multiples of a page, heads with and without unrotated dimensions."""
    if layers is None:
        layers = [layer(mlp=moe()),
                  layer(left(heads=4, kv_heads=1, dim=12, vdim=6, chunk=37, rot_dims=12, base=1000.0, factor=None, scale=0.3), right(heads=2, dim=7, rank=3)),
                  layer(left(heads=2, kv_heads=2, dim=6, vdim=6, chunk=0, rot_dims=2, factor=1.5), right(heads=4, dim=33, rank=8), mlp=dense()),
                  layer(mlp=moe(experts=4, top=3, ff=16, groups=2, keep=2, scale=0.5))]
    cfg = {"architecture": "Fogizen", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if bigram is not None:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return cfg




def spec_of(cfg):
    from lmdeploy_b200.turbomind.specs import fogizen_spec
    return fogizen_spec(cfg)


def random_tensors(cfg, seed=0):
    """name -> float32 tensor with bf16-representable values (so bf16 and float32 engines and the float64 oracle share them)."""
    from lmdeploy_b200.turbomind.hybrid import HybridModel
    shapes = HybridModel.tensor_shapes(_Shapes(spec_of(cfg)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes.items():
        if name.endswith(("norm1", "final.norm", ".norm", ".out")):
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("shift") or ".mu." in name:
            t = torch.rand(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("talk"):
            t = torch.eye(shape[0]) + 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("sink"):
            t = 2.0 * torch.randn(shape, generator=g)
        elif name.endswith(".w0"):
            t = -5.0 + 5.5 * torch.rand(shape, generator=g)                  # decays from exp(-exp(0.5)) = 0.19 to 0.993
        elif name.endswith(".u"):
            t = 0.7 * torch.randn(shape, generator=g)
        elif name.endswith("mlp.act"):
            t = torch.tensor([0.4, -0.8]) + 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("correction"):
            t = 0.4 * torch.randn(shape, generator=g)
        elif name.endswith("router"):
            t = torch.randn(shape, generator=g) * (3.0 / shape[-1] ** 0.5)
        elif name in ("embed", "bigram"):
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
    return F.Decoder(cfg, tensors, torch.float64).forward(list(tokens), trace).numpy()
