"""Device runtime of hybrid decoders (specs.HybridSpec): weights, cache / state geometry and the step function.

A hybrid decoder mixes layer kinds, so a sequence owns two things between steps:
  * pages of the engine's block pool (runtime.KvCachePool, handed out by scheduler.BlockAllocator) -- every latent-attention
    layer keeps, per position, its normed key/value latent (as T) and the rotated key part all heads share (as float); every
    windowed-, chunked- or convolved-rotary-attention layer its normed (and rotated) keys and its values (as T);
  * one slot of the StatePool (handed out by scheduler.Scheduler's slot list) -- per layer the last taps-1 inputs of the
    short convolution (of both sublayers in pre-norm blocks; of the stacked q | k projection of a convolved attention; of the
    x | B | C channels of a state-space mixer), per decayed-linear-attention or channel-decay layer the [heads, vdim, dim] float
    state and per state-space layer the [heads, vdim, state] float state; in shared-norm blocks per run the last normed row and the
    last shifted row (the token shift), and once the id of the last token (hashed bigram embedding).
A layer that a spec loops (HybridSpec.loop) is executed several times per step with the same weights: caches and states
belong to RUNS (HybridSpec.runs()), weights to layers.
The step is a mixed step like b200_model_chunk_step: any number of rows per sequence, prompt portions beside single decoded
tokens; kernels address rows through (sequence, position) arrays, pages through the block table, state through the slot.

Compute: every operator except the plain matrix products is a kernel of libb200hybrid.so (csrc/hybrid/hybrid_ops.cu); the
plain projections are cuBLAS GEMMs through torch (bf16 with float accumulation, or true float32 with TF32 off).  What the
design wants in 32 bits (residual stream and its history, norms, rotary angles, scores, softmax, recurrent state, router)
is float in every kernel whatever the projection type is."""
import contextlib
import ctypes as C

import torch

from .. import _hybrid_lib as H
from .runtime import KvCachePool
from .specs import HybridSpec

_TORCH_T = {"bf16": torch.bfloat16, "f32": torch.float32}
_DT = {"bf16": H.BF16, "f32": H.F32}


def _align(n, a=16):
    return (n + a - 1) // a * a


class StatePool:
    """Recurrent-state slots: one float row per live sequence.  A slot is zeroed when a sequence starts (or restarts after a
    preemption) in it; the scheduler owns the free list."""

    def __init__(self, slots, floats_per_slot, device):
        self.slots, self.floats_per_slot = slots, floats_per_slot
        self.storage = torch.zeros(slots, max(floats_per_slot, 1), dtype=torch.float32, device=device)

    def reset(self, slot):
        self.storage[slot].zero_()

    def ptr(self, float_offset):
        return self.storage.data_ptr() + 4 * float_offset


class StepArrays:
    """The device arrays every operator of a step addresses rows, pages and state through (see HybridModel.step)."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


class HybridModel:
    """Weights of one hybrid decoder on one GPU and its step function."""
    kind = "hybrid"
    tp_size = 1

    def __init__(self, spec: HybridSpec, *, block_len=64, max_batch=64, device=None):
        if spec.dtype not in _DT:
            raise ValueError(f"dtype {spec.dtype!r}: hybrid decoders run in 'bf16' or 'f32'")
        if not 1 <= spec.conv_taps <= H.MAX_TAPS:
            raise NotImplementedError(f"conv taps {spec.conv_taps} (1..{H.MAX_TAPS})")
        if spec.width % spec.norm_groups:
            raise ValueError(f"width {spec.width} is not divisible into {spec.norm_groups} norm groups")
        self.lib = H.load()
        self.spec = spec
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.T, self.dt = _TORCH_T[spec.dtype], _DT[spec.dtype]
        self.block_len, self.max_batch = block_len, max_batch
        esize = 2 if spec.dtype == "bf16" else 4
        # cache page: the attention runs' regions one after another; a latent region is [block_len, kv_rank] T then [block_len, rot_dim] float
        # state slot: per run [taps-1, width] conv inputs (twice where the feed-forward has a conv too), then per decay layer [heads, vdim, dim]
        self.cache_off, self.rot_off, self.conv_off, self.mix_off, self.conv2_off, self.v_off = {}, {}, {}, {}, {}, {}
        self.shift_off = {}
        self.runs = spec.runs()
        if spec.block not in ("post_norm", "pre_norm", "parallel", "shared_norm"):
            raise NotImplementedError(f"block {spec.block!r}")
        pre = spec.block == "pre_norm"
        page = slot = 0
        taps = spec.conv_taps
        self.token_off = None
        if spec.bigram is not None:             # the sequence's last token id, an int in a float's place (four floats: what follows stays 16-byte aligned)
            self.token_off = slot
            slot += 4
        for r, (i, _) in enumerate(self.runs):
            layer = spec.layers[i]
            m = layer.mixer
            self.conv_off[r] = slot             # parallel blocks have no convolution on the stream: the mixers bring their own
            if spec.block == "shared_norm":     # token shift: the last normed row and the last shifted row
                self.shift_off[r] = slot
                slot += 2 * spec.width
            elif spec.block != "parallel":
                slot += (taps - 1) * spec.width
            if pre and layer.mlp is not None:
                self.conv2_off[r] = slot
                slot += (taps - 1) * spec.width
            if m.kind == "conv_attention":
                if not 1 <= m.conv_taps <= H.MAX_TAPS:
                    raise NotImplementedError(f"conv taps {m.conv_taps} (1..{H.MAX_TAPS})")
                if not m.values_from_keys:
                    raise NotImplementedError("convolved attention with a value projection of its own")
                # state: the last taps-1 rows of the stacked q | k projection; cache region as for windowed attention
                self.conv_off[r] = slot
                slot += (m.conv_taps - 1) * (m.heads + m.kv_heads) * m.dim
                self.cache_off[r] = page
                self.v_off[r] = _align(block_len * m.kv_heads * m.dim * esize)
                page += self.v_off[r] + _align(block_len * m.kv_heads * m.vdim * esize)
            elif m.kind == "mamba2":
                if not 1 <= m.conv_taps <= H.MAX_TAPS:
                    raise NotImplementedError(f"conv taps {m.conv_taps} (1..{H.MAX_TAPS})")
                if m.state > 256:
                    raise NotImplementedError("state-space mixer: state <= 256")
                self.conv_off[r] = slot
                slot += (m.conv_taps - 1) * m.conv_channels
                self.mix_off[r] = slot
                slot += m.heads * m.vdim * m.state
            elif m.kind == "latent_attention":
                if m.kv_rank > 512 or m.rot_dim > 128:
                    raise NotImplementedError("latent attention: kv_rank <= 512 and rot_dim <= 128")
                self.cache_off[r] = page
                self.rot_off[r] = _align(block_len * m.kv_rank * esize)
                page += self.rot_off[r] + _align(block_len * m.rot_dim * 4)
            elif m.kind == "lightning":
                if m.dim > 256:
                    raise NotImplementedError("decayed linear attention: dim <= 256")
                self.mix_off[r] = slot
                slot += m.heads * m.vdim * m.dim
            elif m.kind in ("window_attention", "paired"):
                if m.kind == "paired":
                    if spec.block != "shared_norm" or m.left.kind != "window_attention" or m.right.kind != "channel_decay":
                        raise NotImplementedError("paired mixers: windowed attention beside a channel-decay recurrence in shared-norm blocks")
                    if m.right.dim > 256:
                        raise NotImplementedError("channel-decay recurrence: dim <= 256")
                    slot = _align(slot, 4)                  # 16-byte reads of the state's columns
                    self.mix_off[r] = slot
                    slot += m.right.heads * m.right.vdim * m.right.dim
                    m = m.left
                if m.window and m.chunk:
                    raise NotImplementedError("windowed attention: a sliding window or chunks, not both")
                # in a region [block_len, kv_heads * dim] keys as T then [block_len, kv_heads * vdim] values as T
                self.cache_off[r] = page
                self.v_off[r] = _align(block_len * m.kv_heads * m.dim * esize)
                page += self.v_off[r] + _align(block_len * m.kv_heads * m.vdim * esize)
            else:
                raise NotImplementedError(m.kind)
        self.block_bytes = max(page, 16)
        self.layer_bytes = self.block_bytes         # bytes of one block per "layer unit" as the engine sizes pools: whole block
        self.slot_floats = slot
        self.w = {}
        self.weight_bytes = 0
        self.grouped_experts_rows = 24    # steps that give an expert this many rows on average run the experts as grouped GEMMs
        self.attention_warps = 148 * 16   # warps a latent-attention launch aims for (one per row, head and key range)
        self.window_scratch_bytes = 256 << 20    # most bytes of scores a windowed-attention launch leaves between its two passes
        self.events = None          # a list while profiling: (operator, start event, end event) of every timed region
        if spec.dtype == "f32":
            # float32 serving means true 32-bit products: no TF32, no reduced-precision accumulation
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
            torch.set_float32_matmul_precision("highest")
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    # ------------------------------------------------------------------ pools
    def make_cache(self, num_blocks):
        return KvCachePool(num_blocks, 1, 1, block_len=self.block_len, device=self.device, block_bytes=self.block_bytes)

    def make_state(self, slots):
        return StatePool(slots, self.slot_floats, self.device)

    # ------------------------------------------------------------------ weights
    def load_weights(self, get):
        """get(name) -> host tensor by checkpoint name ('embed', 'l<i>.mix.dq', 'l<i>.mlp.e<k>.gate', ...).  Linear weights stay
        [out, in] as T; projections that read the same input are stacked into one matrix; experts are stacked per layer;
        everything the kernels read as float (norm, conv, router weights, sinks, decays, depth coefficients) is float."""
        s, dev, T = self.spec, self.device, self.T
        w = self.w

        def lin(*names, shape=None):
            t = torch.cat([get(n).to(torch.float32) for n in names], 0)
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"{'+'.join(names)}: shape {tuple(t.shape)}, expected {tuple(shape)}")
            t = t.to(dev, T).contiguous()
            self.weight_bytes += t.numel() * t.element_size()
            return t

        def f32(name, shape):
            t = get(name).to(torch.float32)
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(t.shape)}, expected {tuple(shape)}")
            return t.to(dev).contiguous()

        W = s.width
        pre = s.block == "pre_norm"
        par = s.block == "parallel"

        def norm_w(name):
            # pre-norm and parallel blocks store a norm weight as its deviation from one: the kernels get the full factor
            t = f32(name, (W,))
            return t + 1.0 if (pre or par) and not s.plain_norms else t

        def window_weights(p, ck, m):
            """Windowed attention: checkpoint tensors ck + 'q' ... -> w[p + 'in'] ..."""
            HD, GD, GV, HV = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim, m.heads * m.vdim
            gate_cols = (m.heads if m.gate_per_head else HV) if m.gate else 0
            parts = [ck + "q", ck + "k", ck + "v"] + ([ck + "g"] if m.gate else [])
            w[p + "in"] = lin(*parts, shape=(HD + GD + GV + gate_cols, W))
            if m.bias:          # added in float by the kernel that norms q and k and stores the cache (no bias pass over the GEMM's output)
                w[p + "in.b"] = torch.cat([f32(ck + f"{k}.b", (cols,)) for k, cols in (("q", HD), ("k", GD), ("v", GV))]).contiguous()
            w[p + "o"] = lin(ck + "o", shape=(W, HV))
            if m.qk_norm:
                w[p + "q.norm"] = f32(ck + "q.norm", (m.dim,) if m.head_norm else (HD,))
                w[p + "k.norm"] = f32(ck + "k.norm", (m.dim,) if m.head_norm else (GD,))
            if m.distance_bias:
                w[p + "r1"] = f32(ck + "r1", (m.heads,))
                w[p + "r2"] = f32(ck + "r2", (m.heads,))
            if m.talking_heads:
                w[p + "talk"] = f32(ck + "talk", (m.heads, m.heads))
            if m.sink:
                w[p + "sink"] = f32(ck + "sink", (m.heads,))
            if m.rot is not None:
                freqs, mag = m.rot.frequencies()
                w[p + "freqs"] = torch.tensor(freqs, dtype=torch.float64, device=dev)
                w[p + "mag"] = float(mag)

        w["embed"] = lin("embed", shape=(s.vocab, W))
        w["head"] = w["embed"] if s.tied_head else lin("head", shape=(s.vocab, W))
        w["final.norm"] = norm_w("final.norm")
        if s.bigram is not None:
            w["bigram"] = lin("bigram", shape=(s.bigram.buckets + 1, W))
        if s.max_positions:
            w["pos"] = lin("pos", shape=(s.max_positions, W))
        if s.loop is not None:
            w["loop.step"] = lin("loop.step", shape=(s.loop[2], W))
        for i, layer in enumerate(s.layers):
            p, m = f"l{i}.", layer.mixer
            w[p + "norm1"] = norm_w(p + "norm1")
            shared = s.block == "shared_norm"
            if shared:
                w[p + "shift"] = f32(p + "shift", (W,))
            elif not par:
                w[p + "canon1"] = f32(p + "canon1", (W, s.conv_taps))
            if s.block == "post_norm":
                w[p + "dwa"] = f32(p + "dwa", (i + 2,))
            if m.kind == "conv_attention":
                HD, GD = m.heads * m.dim, m.kv_heads * m.dim
                w[p + "in"] = lin(p + "mix.q", p + "mix.k", shape=(HD + GD, W))
                w[p + "conv"] = torch.cat([f32(p + "mix.q.conv", (HD, m.conv_taps)), f32(p + "mix.k.conv", (GD, m.conv_taps))]).contiguous()
                w[p + "o"] = lin(p + "mix.o", shape=(W, m.heads * m.vdim))
                freqs, mag = m.rot.frequencies()
                w[p + "freqs"] = torch.tensor(freqs, dtype=torch.float64, device=dev)
                w[p + "mag"] = float(mag)
                if m.sink is not None:
                    w[p + "sink"] = torch.full((m.heads,), float(m.sink), dtype=torch.float32, device=dev)
            elif m.kind == "mamba2":
                w[p + "in"] = lin(p + "mix.in", shape=(m.proj_cols, W))
                w[p + "conv"] = f32(p + "mix.conv", (m.conv_channels, m.conv_taps))
                w[p + "conv.b"] = f32(p + "mix.conv.b", (m.conv_channels,))
                for k in ("dt_bias", "A_log", "D"):
                    w[p + k] = f32(p + "mix." + k, (m.heads,))
                w[p + "mixnorm"] = f32(p + "mix.norm", (m.inner,))
                w[p + "o"] = lin(p + "mix.o", shape=(W, m.inner))
            elif m.kind == "latent_attention":
                HV = m.heads * m.vdim
                w[p + "in"] = lin(p + "mix.dq", p + "mix.dkv", p + "mix.g", shape=(m.q_rank + m.kv_rank + m.rot_dim + HV, W))
                w[p + "uq"] = lin(p + "mix.uq", shape=(m.heads * (m.dim + m.rot_dim), m.q_rank))
                w[p + "uk"] = lin(p + "mix.uk", shape=(m.heads * m.dim, m.kv_rank))
                w[p + "uv"] = lin(p + "mix.uv", shape=(HV, m.kv_rank))
                w[p + "o"] = lin(p + "mix.o", shape=(W, HV))
                w[p + "dq.norm"] = f32(p + "mix.dq.norm", (m.q_rank,))
                w[p + "dkv.norm"] = f32(p + "mix.dkv.norm", (m.kv_rank,))
                w[p + "sink"] = f32(p + "mix.sink", (m.heads,))
                freqs, mag = m.rot.frequencies()
                w[p + "freqs"] = torch.tensor(freqs, dtype=torch.float64, device=dev)
                w[p + "mag"] = float(mag)
            elif m.kind == "window_attention":
                window_weights(p, p + "mix.", m)
            elif m.kind == "paired":
                window_weights(p + "left.", p + "mix.left.", m.left)
                R, ck = m.right, p + "mix.right."
                HD = R.heads * R.dim
                # r | k | v | g stacked for ONE batched product over the four blends; the decay's two matrices apart
                w[p + "right.in"] = torch.stack([lin(ck + k, shape=(HD, W)) for k in "rkvg"]).contiguous()
                w[p + "right.mu"] = torch.stack([f32(ck + "mu." + k, (W,)) for k in "rkvgw"]).contiguous()
                w[p + "right.w1"] = lin(ck + "w1", shape=(R.rank, W))
                w[p + "right.w2"] = lin(ck + "w2", shape=(HD, R.rank))
                w[p + "right.w0"] = f32(ck + "w0", (HD,))
                w[p + "right.u"] = f32(ck + "u", (R.heads, R.dim))
                w[p + "right.norm"] = f32(ck + "norm", (HD,))
                w[p + "right.o"] = lin(ck + "o", shape=(W, HD))
                w[p + "left.out"] = f32(p + "mix.left.out", (W,))
                w[p + "right.out"] = f32(p + "mix.right.out", (W,))
            else:
                HD, HV = m.heads * m.dim, m.heads * m.vdim
                w[p + "in"] = lin(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g", shape=(2 * HD + 2 * HV, W))
                w[p + "o"] = lin(p + "mix.o", shape=(W, HV))
                w[p + "mixnorm"] = f32(p + "mix.norm", (HV,))
                w[p + "decay"] = torch.tensor(m.decay, dtype=torch.float32, device=dev)
            f = layer.mlp
            if f is not None:
                if not shared:
                    w[p + "norm2"] = norm_w(p + "norm2")
                if pre:
                    w[p + "canon2"] = f32(p + "canon2", (W, s.conv_taps))
                if f.kind == "dense":
                    w[p + "up"] = lin(p + "mlp.up", shape=(f.ff, W))
                    w[p + "down"] = lin(p + "mlp.down", shape=(W, f.ff))
                    if f.act == "xielu":
                        w[p + "act"] = f32(p + "mlp.act", (2,))
                    continue
                w[p + "router"] = f32(p + "mlp.router", (f.experts, W))
                if f.correction:
                    w[p + "correction"] = f32(p + "mlp.correction", (f.experts,))
                for part, shape in (("gate", (f.ff, W)), ("up", (f.ff, W)), ("down", (W, f.ff))):
                    if part == "gate" and f.act != "silu_gate":
                        continue
                    w[p + part] = torch.stack([lin(f"{p}mlp.e{e}.{part}", shape=shape) for e in range(f.experts)]).contiguous()
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)

    def load_synthetic(self, seed=0):
        """Random weights of the spec's shapes (benchmarks and tests)."""
        g = torch.Generator().manual_seed(seed)
        taps = self.spec.conv_taps

        def get(name):
            shape = self.tensor_shapes()[name]
            if name.endswith(("norm1", "norm2", "final.norm")) and self.spec.block in ("pre_norm", "parallel") and not self.spec.plain_norms:
                return 0.1 * torch.randn(shape, generator=g)            # stored as the deviation from one
            if name.endswith((".conv", ".conv.b")):
                return torch.randn(shape, generator=g) / (shape[-1] if name.endswith(".conv") else 10.0)
            if name.endswith(".A_log"):
                return torch.log(1.0 + 15.0 * torch.rand(shape, generator=g))
            if name.endswith(".dt_bias"):
                return torch.log(torch.expm1(0.001 + 0.099 * torch.rand(shape, generator=g)))
            if name.endswith(".D"):
                return torch.ones(shape)
            if name.endswith(("norm1", "norm2", ".norm", ".out")):
                return 1.0 + 0.1 * torch.randn(shape, generator=g)
            if name.endswith("shift") or ".mu." in name:
                return torch.rand(shape, generator=g)
            if name.endswith(".w0"):                                     # decays exp(-exp(w0 + ...)) between about 0.37 and 0.998
                return -6.0 + 6.0 * torch.rand(shape, generator=g)
            if name.endswith(".u"):
                return 0.5 * torch.randn(shape, generator=g)
            if name.endswith("mlp.act"):
                return torch.tensor([0.5, -0.5])
            if name.endswith("correction"):
                return 0.1 * torch.randn(shape, generator=g)
            if name.endswith(("canon1", "canon2")):
                return torch.randn(shape, generator=g) / taps
            if name.endswith((".r1", ".r2")):
                return torch.rand(shape, generator=g)
            if name.endswith(".talk"):
                return torch.eye(shape[0]) + 0.1 * torch.randn(shape, generator=g)
            if name.endswith(".b") or name in ("pos", "loop.step"):
                return (0.1 * torch.randn(shape, generator=g)).to(torch.bfloat16)
            if name.endswith("dwa"):
                return torch.softmax(torch.randn(shape, generator=g), 0)
            if name.endswith("sink"):
                return torch.randn(shape, generator=g)
            scale = 0.02 if name == "embed" else 1.0 / (shape[-1] ** 0.5)
            return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16)

        self.load_weights(get)

    def tensor_shapes(self):
        """Checkpoint tensor names -> shapes for this spec."""
        s, W = self.spec, self.spec.width
        pre = s.block == "pre_norm"
        par = s.block == "parallel"
        out = {"embed": (s.vocab, W)}
        if not s.tied_head:
            out["head"] = (s.vocab, W)
        out["final.norm"] = (W,)
        if s.bigram is not None:
            out["bigram"] = (s.bigram.buckets + 1, W)
        if s.max_positions:
            out["pos"] = (s.max_positions, W)
        if s.loop is not None:
            out["loop.step"] = (s.loop[2], W)
        shared = s.block == "shared_norm"

        def window_shapes(ck, m):
            HD, GD, GV, HV = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim, m.heads * m.vdim
            out.update({ck + "q": (HD, W), ck + "k": (GD, W), ck + "v": (GV, W), ck + "o": (W, HV)})
            if m.bias:
                out.update({ck + "q.b": (HD,), ck + "k.b": (GD,), ck + "v.b": (GV,)})
            if m.qk_norm:
                out.update({ck + "q.norm": (m.dim,) if m.head_norm else (HD,), ck + "k.norm": (m.dim,) if m.head_norm else (GD,)})
            if m.distance_bias:
                out.update({ck + "r1": (m.heads,), ck + "r2": (m.heads,)})
            if m.talking_heads:
                out[ck + "talk"] = (m.heads, m.heads)
            if m.sink:
                out[ck + "sink"] = (m.heads,)
            if m.gate:
                out[ck + "g"] = (m.heads if m.gate_per_head else HV, W)

        for i, layer in enumerate(s.layers):
            p, m = f"l{i}.", layer.mixer
            out[p + "norm1"] = (W,)
            if shared:
                out[p + "shift"] = (W,)
            elif not par:
                out[p + "canon1"] = (W, s.conv_taps)
            if s.block == "post_norm":
                out[p + "dwa"] = (i + 2,)
            if m.kind == "conv_attention":
                HD, GD = m.heads * m.dim, m.kv_heads * m.dim
                out.update({p + "mix.q": (HD, W), p + "mix.k": (GD, W), p + "mix.q.conv": (HD, m.conv_taps), p + "mix.k.conv": (GD, m.conv_taps),
                            p + "mix.o": (W, m.heads * m.vdim)})
            elif m.kind == "mamba2":
                out.update({p + "mix.in": (m.proj_cols, W), p + "mix.conv": (m.conv_channels, m.conv_taps), p + "mix.conv.b": (m.conv_channels,),
                            p + "mix.dt_bias": (m.heads,), p + "mix.A_log": (m.heads,), p + "mix.D": (m.heads,), p + "mix.norm": (m.inner,),
                            p + "mix.o": (W, m.inner)})
            elif m.kind == "latent_attention":
                HV = m.heads * m.vdim
                out.update({p + "mix.dq": (m.q_rank, W), p + "mix.dq.norm": (m.q_rank,), p + "mix.uq": (m.heads * (m.dim + m.rot_dim), m.q_rank),
                            p + "mix.dkv": (m.kv_rank + m.rot_dim, W), p + "mix.dkv.norm": (m.kv_rank,),
                            p + "mix.uk": (m.heads * m.dim, m.kv_rank), p + "mix.uv": (HV, m.kv_rank), p + "mix.sink": (m.heads,),
                            p + "mix.g": (HV, W), p + "mix.o": (W, HV)})
            elif m.kind == "window_attention":
                window_shapes(p + "mix.", m)
            elif m.kind == "paired":
                window_shapes(p + "mix.left.", m.left)
                R, ck = m.right, p + "mix.right."
                HD = R.heads * R.dim
                out.update({ck + k: (HD, W) for k in "rkvg"})
                out.update({ck + "mu." + k: (W,) for k in "rkvgw"})
                out.update({ck + "w1": (R.rank, W), ck + "w2": (HD, R.rank), ck + "w0": (HD,), ck + "u": (R.heads, R.dim), ck + "norm": (HD,),
                            ck + "o": (W, HD), p + "mix.left.out": (W,), p + "mix.right.out": (W,)})
            else:
                HD, HV = m.heads * m.dim, m.heads * m.vdim
                out.update({p + "mix.q": (HD, W), p + "mix.k": (HD, W), p + "mix.v": (HV, W), p + "mix.g": (HV, W),
                            p + "mix.o": (W, HV), p + "mix.norm": (HV,)})
            f = layer.mlp
            if f is not None:
                if not shared:
                    out[p + "norm2"] = (W,)
                if pre:
                    out[p + "canon2"] = (W, s.conv_taps)
                if f.kind == "dense":
                    out.update({p + "mlp.up": (f.ff, W), p + "mlp.down": (W, f.ff)})
                    if f.act == "xielu":
                        out[p + "mlp.act"] = (2,)
                    continue
                out[p + "mlp.router"] = (f.experts, W)
                if f.correction:
                    out[p + "mlp.correction"] = (f.experts,)
                for e in range(f.experts):
                    if f.act == "silu_gate":
                        out[f"{p}mlp.e{e}.gate"] = (f.ff, W)
                    out.update({f"{p}mlp.e{e}.up": (f.ff, W), f"{p}mlp.e{e}.down": (W, f.ff)})
        return out

    # ------------------------------------------------------------------ step
    @contextlib.contextmanager
    def timed(self, name):
        """Bracket an operator with CUDA events while profiling (bench.py); free otherwise."""
        if self.events is None:
            yield
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        yield
        b.record()
        self.events.append((name, a, b))

    def operator_ms(self):
        """Profiling: total milliseconds per operator since `events` was last cleared."""
        torch.cuda.synchronize(self.device)
        out = {}
        for name, a, b in self.events:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        self.events = []
        return out

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream if self.device.type == "cuda" else None

    def _linear(self, x, w):
        return torch.mm(x, w.t())

    def step(self, *, n, batch, tokens, tok_seq, tok_pos, cu_q, seq_slot, block_ptrs, cu_blocks, state: StatePool, rows, n_rows,
             max_pos, trace=None):
        """One mixed step.  Device tensors: tokens / tok_seq / tok_pos int32 [n]; cu_q, cu_blocks int32 [batch + 1]; seq_slot
        int32 [batch]; block_ptrs int64 (page addresses); rows int32 [n_rows] = the rows whose logits are wanted; max_pos (host
        int) = the largest position of the step.
        Returns float logits [n_rows, vocab].  trace: a list that receives a copy of the stream after every layer."""
        s, lib, w, dev, T, dt = self.spec, self.lib, self.w, self.device, self.T, self.dt
        W, eps, groups = s.width, s.norm_eps, s.norm_groups
        st = self._stream()
        if s.max_positions and max_pos >= s.max_positions:
            raise ValueError(f"position {max_pos}: the model has {s.max_positions} learned positions")
        if s.block == "shared_norm":
            return self._step_shared_norm(n=n, batch=batch, tokens=tokens, tok_seq=tok_seq, tok_pos=tok_pos, cu_q=cu_q, seq_slot=seq_slot,
                                          block_ptrs=block_ptrs, cu_blocks=cu_blocks, state=state, rows=rows, n_rows=n_rows,
                                          max_pos=max_pos, trace=trace)
        if s.block == "parallel":
            return self._step_parallel(n=n, batch=batch, tokens=tokens, tok_seq=tok_seq, tok_pos=tok_pos, cu_q=cu_q, seq_slot=seq_slot,
                                       block_ptrs=block_ptrs, cu_blocks=cu_blocks, state=state, rows=rows, n_rows=n_rows, max_pos=max_pos,
                                       trace=trace)
        if s.block == "pre_norm":
            return self._step_pre_norm(n=n, batch=batch, tokens=tokens, tok_seq=tok_seq, tok_pos=tok_pos, cu_q=cu_q, seq_slot=seq_slot,
                                       block_ptrs=block_ptrs, cu_blocks=cu_blocks, state=state, rows=rows, n_rows=n_rows, max_pos=max_pos,
                                       trace=trace)
        c = StepArrays(n=n, batch=batch, tok_seq=tok_seq, tok_pos=tok_pos, cu_q=cu_q, seq_slot=seq_slot, block_ptrs=block_ptrs,
                       cu_blocks=cu_blocks, state=state, max_pos=max_pos)
        f32 = dict(dtype=torch.float32, device=dev)
        hist = torch.empty(len(s.layers) + 1, n, W, **f32)
        x = torch.empty(n, W, **f32)
        with self.timed("embed"):
            H.check(lib.b200h_embed(tokens.data_ptr(), w["embed"].data_ptr(), s.embedding_scale, hist.data_ptr(), n, W, dt, st), "embed")
            x.copy_(hist[0])
        xt = torch.empty(n, W, dtype=T, device=dev)
        for i, layer in enumerate(s.layers):
            p = f"l{i}."
            h = self.conv_input(i, x, c)
            y = self.mixer(i, i, h, c)
            with self.timed("gemm out"):
                mixed = self._linear(y, w[p + "o"])
            f = layer.mlp
            with self.timed("residual + grouped norm"):
                H.check(lib.b200h_residual_group_norm(x.data_ptr(), mixed.data_ptr(), 0, 1, w[p + "norm1"].data_ptr(), n, W, groups, eps,
                                                      xt.data_ptr() if f is not None else None, dt, st), "residual_group_norm")
            if f is not None:
                if f.kind != "moe":
                    raise NotImplementedError(f"post-norm blocks with a {f.kind!r} feed-forward")
                out = self.routed_experts(i, x, xt, n)
                with self.timed("residual + grouped norm"):
                    H.check(lib.b200h_residual_group_norm(x.data_ptr(), out.data_ptr(), 1, f.top, w[p + "norm2"].data_ptr(), n, W, groups,
                                                          eps, None, dt, st), "residual_group_norm")
            with self.timed("depth mix"):
                H.check(lib.b200h_depth_mix(x.data_ptr(), hist.data_ptr(), n * W, w[p + "dwa"].data_ptr(), i + 2, n * W, st), "depth_mix")
            if trace is not None:
                trace.append(x.clone())
        xn = torch.empty(n_rows, W, dtype=T, device=dev)
        with self.timed("final norm + head"):
            H.check(lib.b200h_group_norm_rows(x.data_ptr(), rows.data_ptr(), w["final.norm"].data_ptr(), n_rows, W, groups, eps,
                                              xn.data_ptr(), dt, st), "group_norm_rows")
            return self._logits(xn)

    def _step_pre_norm(self, *, n, batch, tokens, tok_seq, tok_pos, cu_q, seq_slot, block_ptrs, cu_blocks, state, rows, n_rows, max_pos,
                       trace=None):
        """The step of pre-norm blocks: x <- x + mixer(conv(norm1(x))), x <- x + ff(conv(norm2(x))) per run.  A sublayer's output
        joins the float stream inside the kernel that norms the stream for the next reader (residual add + norm in one pass)."""
        s, lib, w, dev, T, dt = self.spec, self.lib, self.w, self.device, self.T, self.dt
        W, eps, st = s.width, s.norm_eps, self._stream()
        c = StepArrays(n=n, batch=batch, tok_seq=tok_seq, tok_pos=tok_pos, cu_q=cu_q, seq_slot=seq_slot, block_ptrs=block_ptrs,
                       cu_blocks=cu_blocks, state=state, max_pos=max_pos)
        x = torch.empty(n, W, dtype=torch.float32, device=dev)
        with self.timed("embed"):
            H.check(lib.b200h_embed(tokens.data_ptr(), w["embed"].data_ptr(), s.embedding_scale, x.data_ptr(), n, W, dt, st), "embed")
            if s.max_positions:
                H.check(lib.b200h_add_rows(x.data_ptr(), w["pos"].data_ptr(), tok_pos.data_ptr(), 0, n, W, dt, st), "add_rows")
        pending = None                   # a sublayer's output (T) that the stream has not taken in yet
        for r, (i, t) in enumerate(self.runs):
            p, layer = f"l{i}.", s.layers[i]
            extra = None
            if t is not None and i == s.loop[0]:
                extra = w["loop.step"].data_ptr() + t * W * w["loop.step"].element_size()
            h = self.norm_conv_input(r, i, 1, x, pending, extra, c)
            y = self.mixer(r, i, h, c)
            with self.timed("gemm out"):
                pending = self._linear(y, w[p + "o"])
            f = layer.mlp
            if f is not None:
                h = self.norm_conv_input(r, i, 2, x, pending, None, c)
                pending = self.dense_mlp(i, h)
            if trace is not None:
                H.check(lib.b200h_residual_norm(x.data_ptr(), pending.data_ptr(), None, None, n, W, eps, None, dt, st), "residual_norm")
                pending = None
                trace.append(x.clone())
        xn = torch.empty(n_rows, W, dtype=T, device=dev)
        with self.timed("final norm + head"):
            if pending is not None:
                H.check(lib.b200h_residual_norm(x.data_ptr(), pending.data_ptr(), None, None, n, W, eps, None, dt, st), "residual_norm")
            H.check(lib.b200h_group_norm_rows(x.data_ptr(), rows.data_ptr(), w["final.norm"].data_ptr(), n_rows, W, 1, eps, xn.data_ptr(),
                                              dt, st), "group_norm_rows")
            return self._logits(xn)

    def _step_parallel(self, *, n, batch, tokens, tok_seq, tok_pos, cu_q, seq_slot, block_ptrs, cu_blocks, state, rows, n_rows, max_pos,
                       trace=None):
        """The step of parallel blocks: x <- x + mult * (mixer(n1(x)) + ff(n2(x))) per run, both sublayers reading the same stream.
        One kernel per run takes the previous run's two outputs into the float stream (and, before a pass of looped layers, the
        embedding output and the pass's vector) and emits both normed inputs of this run."""
        s, lib, w, dev, T, dt = self.spec, self.lib, self.w, self.device, self.T, self.dt
        W, eps, st = s.width, s.norm_eps, self._stream()
        c = StepArrays(n=n, batch=batch, tok_seq=tok_seq, tok_pos=tok_pos, cu_q=cu_q, seq_slot=seq_slot, block_ptrs=block_ptrs,
                       cu_blocks=cu_blocks, state=state, max_pos=max_pos)
        x = torch.empty(n, W, dtype=torch.float32, device=dev)
        with self.timed("embed"):
            H.check(lib.b200h_embed(tokens.data_ptr(), w["embed"].data_ptr(), s.embedding_scale, x.data_ptr(), n, W, dt, st), "embed")
            e0 = x.clone() if s.loop is not None and s.loop_readds_embedding and s.loop[2] > 1 else None
        h1 = torch.empty(n, W, dtype=T, device=dev)
        h2 = torch.empty(n, W, dtype=T, device=dev)
        h2f = torch.empty(n, W, dtype=torch.float32, device=dev)         # the router reads the second norm unrounded
        mix = ff = None                  # the previous run's outputs that the stream has not taken in yet
        parts = 0

        def join(add, extra, w1, w2):
            with self.timed("residual + two norms"):
                H.check(lib.b200h_parallel_residual_norm(
                    x.data_ptr(), None if mix is None else mix.data_ptr(), None if ff is None else ff.data_ptr(), parts, s.residual_mult,
                    add, extra, None if w1 is None else w1.data_ptr(), None if w2 is None else w2.data_ptr(), n, W, eps,
                    None if w1 is None else h1.data_ptr(), None if w2 is None else h2.data_ptr(), None if w2 is None else h2f.data_ptr(),
                    dt, st), "parallel_residual_norm")

        for r, (i, t) in enumerate(self.runs):
            p, layer = f"l{i}.", s.layers[i]
            add = extra = None
            if t is not None and i == s.loop[0]:
                if t > 0 and e0 is not None:
                    add = e0.data_ptr()
                extra = w["loop.step"].data_ptr() + t * W * w["loop.step"].element_size()
            f = layer.mlp
            join(add, extra, w[p + "norm1"], w[p + "norm2"] if f is not None else None)
            y = self.mixer(r, i, h1, c)
            with self.timed("gemm out"):
                mix = self._linear(y, w[p + "o"])
            ff, parts = None, 0
            if f is not None:
                if f.kind != "moe":
                    raise NotImplementedError(f"parallel blocks with a {f.kind!r} feed-forward")
                ff, parts = self.routed_experts(i, h2f, h2, n), f.top
            if trace is not None:
                join(None, None, None, None)
                mix = ff = None
                trace.append(x.clone())
        xn = torch.empty(n_rows, W, dtype=T, device=dev)
        with self.timed("final norm + head"):
            if mix is not None or ff is not None:
                join(None, None, None, None)
            H.check(lib.b200h_group_norm_rows(x.data_ptr(), rows.data_ptr(), w["final.norm"].data_ptr(), n_rows, W, 1, eps, xn.data_ptr(),
                                              dt, st), "group_norm_rows")
            return self._logits(xn)

    def _step_shared_norm(self, *, n, batch, tokens, tok_seq, tok_pos, cu_q, seq_slot, block_ptrs, cu_blocks, state, rows, n_rows, max_pos,
                          trace=None):
        """The step of shared-norm blocks: h = n(x), x <- x + mixer(shift(h)) + ff(h) per run.  One kernel per run takes the previous
        run's outputs (the two sides of a paired mixer, each normed over the width, and the feed-forward's) into the float stream and
        emits this run's normed rows; one kernel shifts them (and forms the recurrence's blends) against the previous token's."""
        s, lib, w, dev, T, dt = self.spec, self.lib, self.w, self.device, self.T, self.dt
        W, eps, st = s.width, s.norm_eps, self._stream()
        c = StepArrays(n=n, batch=batch, tok_seq=tok_seq, tok_pos=tok_pos, cu_q=cu_q, seq_slot=seq_slot, block_ptrs=block_ptrs,
                       cu_blocks=cu_blocks, state=state, max_pos=max_pos)
        stride = state.storage.stride(0)
        x = torch.empty(n, W, dtype=torch.float32, device=dev)
        with self.timed("embed"):
            if s.bigram is not None:
                b = s.bigram
                H.check(lib.b200h_embed_hashed(tokens.data_ptr(), w["embed"].data_ptr(), w["bigram"].data_ptr(), b.buckets, b.mul_prev,
                                               b.mul_cur, state.ptr(self.token_off), stride, tok_seq.data_ptr(), tok_pos.data_ptr(),
                                               cu_q.data_ptr(), seq_slot.data_ptr(), x.data_ptr(), n, batch, W, dt, st), "embed_hashed")
            else:
                H.check(lib.b200h_embed(tokens.data_ptr(), w["embed"].data_ptr(), s.embedding_scale, x.data_ptr(), n, W, dt, st), "embed")
        h = torch.empty(n, W, dtype=T, device=dev)
        hf = torch.empty(n, W, dtype=torch.float32, device=dev)
        sides = ff = None                # the previous run's outputs that the stream has not taken in yet
        ff_f32, parts = 0, 0

        def join(norm):
            left, right, wl, wr = sides if sides is not None else (None, None, None, None)
            with self.timed("residual + side norms + norm"):
                H.check(lib.b200h_branch_residual_norm(
                    x.data_ptr(), None if left is None else left.data_ptr(), None if right is None else right.data_ptr(),
                    None if wl is None else wl.data_ptr(), None if wr is None else wr.data_ptr(), 0.5,
                    None if ff is None else ff.data_ptr(), ff_f32, parts, None if norm is None else norm.data_ptr(), n, W, eps,
                    None if norm is None else h.data_ptr(), None if norm is None else hf.data_ptr(), dt, st), "branch_residual_norm")

        for r, (i, _) in enumerate(self.runs):
            p, layer = f"l{i}.", s.layers[i]
            join(w[p + "norm1"])
            m = layer.mixer
            if m.kind != "paired":
                raise NotImplementedError(f"shared-norm blocks with a {m.kind!r} mixer")
            nmu = 5
            a = torch.empty(n, W, dtype=T, device=dev)
            blends = torch.empty(nmu, n, W, dtype=T, device=dev)
            with self.timed("token shift + blends"):
                H.check(lib.b200h_token_shift(hf.data_ptr(), w[p + "shift"].data_ptr(), w[p + "right.mu"].data_ptr(), nmu,
                                              state.ptr(self.shift_off[r]), stride, tok_seq.data_ptr(), cu_q.data_ptr(), seq_slot.data_ptr(),
                                              n, batch, W, a.data_ptr(), blends.data_ptr(), dt, st), "token_shift")
            y = self.window_mixer(i, a, c, run=r, m=m.left, p=p + "left.")
            with self.timed("gemm out"):
                left = self._linear(y, w[p + "left.o"])
            y = self.channel_decay_mixer(i, blends, c, run=r, m=m.right, p=p + "right.")
            with self.timed("gemm out"):
                right = self._linear(y, w[p + "right.o"])
            sides = (left, right, w[p + "left.out"], w[p + "right.out"])
            f = layer.mlp
            ff, ff_f32, parts = None, 0, 0
            if f is not None:
                if f.kind == "dense":
                    ff, parts = self.dense_mlp(i, h), 1
                else:
                    ff, ff_f32, parts = self.routed_experts(i, hf, h, n), 1, f.top
            if trace is not None:
                join(None)
                sides = ff = None
                parts = 0
                trace.append(x.clone())
        xn = torch.empty(n_rows, W, dtype=T, device=dev)
        with self.timed("final norm + head"):
            if sides is not None or ff is not None:
                join(None)
            H.check(lib.b200h_group_norm_rows(x.data_ptr(), rows.data_ptr(), w["final.norm"].data_ptr(), n_rows, W, 1, eps, xn.data_ptr(),
                                              dt, st), "group_norm_rows")
            return self._logits(xn)

    def channel_decay_mixer(self, i, blends, c, run=None, m=None, p=None):
        """Channel-decay recurrence of layer i over the five blends [5, n, width] (T; for r, k, v, the gate and the decay): one batched
        product for r | k | v | g, the decay's two small products around a tanh, the per-channel decays and the per-head recurrence on
        the sequence's float state, then the per-head unit norm, its weight and silu(g).  Returns [n, heads * dim] (T)."""
        r = i if run is None else run
        m = self.spec.layers[i].mixer if m is None else m
        p = f"l{i}." if p is None else p
        w, lib, dev, n, st = self.w, self.lib, self.device, c.n, self._stream()
        HD = m.heads * m.dim
        with self.timed("gemm in"):
            proj = torch.bmm(blends[:4], w[p + "in"].transpose(1, 2))              # [4, n, HD]: r, k, v, g
            low = self._linear(blends[4], w[p + "w1"])
        with self.timed("tanh"):
            H.check(lib.b200h_tanh(low.data_ptr(), low.numel(), self.dt, st), "tanh")
        with self.timed("gemm decay"):
            d = self._linear_f32(low, w[p + "w2"])
        es = proj.element_size()
        base, plane = proj.data_ptr(), n * HD * es
        o = torch.empty(n, HD, dtype=torch.float32, device=dev)
        decay = torch.empty(n, HD, dtype=torch.float32, device=dev)
        with self.timed("channel-decay recurrence"):
            H.check(lib.b200h_channel_decay_scan(base, base + plane, base + 2 * plane, HD, d.data_ptr(), w[p + "w0"].data_ptr(),
                                                 w[p + "u"].data_ptr(), c.state.ptr(self.mix_off[r]), c.state.storage.stride(0),
                                                 c.cu_q.data_ptr(), c.seq_slot.data_ptr(), n, c.batch, m.heads, m.dim, m.vdim,
                                                 decay.data_ptr(), o.data_ptr(), self.dt, st), "channel_decay_scan")
        y = torch.empty(n, HD, dtype=self.T, device=dev)
        with self.timed("head norm + gate"):
            H.check(lib.b200h_group_norm_gate(o.data_ptr(), w[p + "norm"].data_ptr(), base + 3 * plane, HD, n, HD, m.heads, H.GATE_ACT["silu"],
                                              self.spec.norm_eps, y.data_ptr(), self.dt, st), "group_norm_gate")
        return y

    def norm_conv_input(self, r, i, sub, x, pending, extra, c):
        """What sublayer `sub` (1: mixer, 2: feed-forward) of run r reads: first the stream takes in `pending` (the previous
        sublayer's output) and `extra` (a vector for all rows), then h = norm(x), then h + causal convolution of h over the
        sequence (as T); advances the sublayer's conv state."""
        s, w, n = self.spec, self.w, c.n
        hn = torch.empty(n, s.width, dtype=torch.float32, device=self.device)
        with self.timed("residual + norm"):
            H.check(self.lib.b200h_residual_norm(x.data_ptr(), None if pending is None else pending.data_ptr(), extra,
                                                 w[f"l{i}.norm{sub}"].data_ptr(), n, s.width, s.norm_eps, hn.data_ptr(), self.dt,
                                                 self._stream()), "residual_norm")
        return self.conv_input(i, hn, c, run=r, sub=sub)

    def mixer(self, r, i, h, c):
        """The sequence mixer of layer i in run r over its input h [n, width] (T) -> the output projection's input."""
        kind = self.spec.layers[i].mixer.kind
        if kind == "latent_attention":
            return self.latent_mixer(i, h, c, run=r)
        if kind == "window_attention":
            return self.window_mixer(i, h, c, run=r)
        if kind == "conv_attention":
            return self.conv_attention_mixer(i, h, c, run=r)
        if kind == "mamba2":
            return self.ssm_mixer(i, h, c, run=r)
        return self.decay_mixer(i, h, c, run=r)

    def window_splits(self, n, window, max_pos):
        """Key ranges per row of a windowed-attention launch: one for prompt portions; a step of few rows cuts its window into
        ranges of at least 32 keys until the launch has about eight blocks per SM.  A power of two (the engine keys its decode
        graphs on it)."""
        keys = min(window, max_pos + 1) if window else max_pos + 1
        want = min(1184 // max(n, 1), keys // 32, 64)
        splits = 1
        while splits * 2 <= want:
            splits *= 2
        return splits

    @staticmethod
    def window_score_ld(window, max_pos):
        """Row length of the score scratch: the keys a row of the step can see, in steps of 256 (a captured decode step is valid
        until the context outgrows it: the engine keys its graphs on this) and never more than the window."""
        keys = min(window, max_pos + 1) if window else max_pos + 1
        ld = (keys + 255) // 256 * 256
        return min(ld, (window + 3) // 4 * 4) if window else ld

    def window_mixer(self, i, h, c, run=None, m=None, p=None):
        """Windowed attention of layer i (m, p: the spec and weight prefix of one side of a paired mixer): one stacked projection
        (q | k | v | gate); biases + RMS norm of q and k (over their whole projections, or per head followed by a rotation) + cache
        store in one kernel; then attention over the window or chunk of cached keys with capped scores, distance penalty, the heads'
        scores or softmax weights recombined, a sink, and the output gate.  Returns [n, heads * vdim] (T)."""
        r = i if run is None else run
        m = self.spec.layers[i].mixer if m is None else m
        p = f"l{i}." if p is None else p
        w, lib, dev, T, n = self.w, self.lib, self.device, self.T, c.n
        HD, GD, GV, HV = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim, m.heads * m.vdim
        with self.timed("gemm in"):
            proj = self._linear(h, w[p + "in"])
        ld, es, base = proj.stride(0), proj.element_size(), proj.data_ptr()
        f32 = dict(dtype=torch.float32, device=dev)
        a = H.WindowArgs()
        a.n, a.heads, a.kv_heads, a.dim, a.vdim, a.block_len, a.window = n, m.heads, m.kv_heads, m.dim, m.vdim, self.block_len, m.window
        a.chunk, a.talk_scores, a.gate_heads = m.chunk, int(m.talk_scores), int(m.gate_per_head)
        a.splits = self.window_splits(n, m.span, c.max_pos)
        a.scale, a.softcap, a.eps = m.scale, m.softcap, self.spec.norm_eps
        a.q, a.k, a.v, a.ld = base, base + es * HD, base + es * (HD + GD), ld
        if m.bias:
            a.bias = w[p + "in.b"].data_ptr()
        if m.qk_norm:
            a.q_norm, a.k_norm = w[p + "q.norm"].data_ptr(), w[p + "k.norm"].data_ptr()
        qn = torch.empty(n, HD, **f32)
        a.qn = qn.data_ptr()
        if m.distance_bias:
            a.r1, a.r2 = w[p + "r1"].data_ptr(), w[p + "r2"].data_ptr()
        if m.talking_heads:
            a.talk = w[p + "talk"].data_ptr()
        if m.sink:
            a.sink = w[p + "sink"].data_ptr()
        if m.gate:
            a.gate, a.ld_gate = base + es * (HD + GD + GV), ld
        y = torch.empty(n, HV, dtype=T, device=dev)
        a.tok_seq, a.tok_pos = c.tok_seq.data_ptr(), c.tok_pos.data_ptr()
        a.block_ptrs, a.cu_blocks = c.block_ptrs.data_ptr(), c.cu_blocks.data_ptr()
        a.layer_off, a.v_off, a.dtype, a.stream = self.cache_off[r], self.v_off[r], self.dt, self._stream()
        if m.head_norm or m.rot is not None:
            if m.qk_norm and not m.head_norm:
                raise NotImplementedError("rotation after a norm over the whole projection")
            rot = H.Rotary(w[p + "freqs"].data_ptr(), m.rot.dims // 2, w[p + "mag"]) if m.rot is not None else H.Rotary(None, 0, 1.0)
            with self.timed("head norm + rotate + cache store"):
                H.check(lib.b200h_head_rope_prep(C.byref(a), C.byref(rot)), "head_rope_prep")
        else:
            with self.timed("qk norm + cache store"):
                H.check(lib.b200h_window_prep(C.byref(a)), "window_prep")
        self._window_attend(a, m, c, qn, y, "chunked attention" if m.chunk else "windowed attention")
        return y

    def _window_attend(self, a, m, c, qn, y, name):
        """The two attention passes over the cache for a prepared step (a: WindowArgs with sizes, switches, cache offsets and, if any,
        gate filled in; qn float [n, heads * dim]; y T [n, heads * vdim]).  Pass 1 leaves every row's scores in a scratch [rows,
        heads, keys a row can see] for pass 2; the step's rows go through the two passes in chunks that keep the scratch within
        `window_scratch_bytes`."""
        n, HD, HV, es = c.n, m.heads * m.dim, m.heads * m.vdim, y.element_size()
        f32 = dict(dtype=torch.float32, device=self.device)
        a.score_ld = self.window_score_ld(getattr(m, "span", m.window), c.max_pos)
        chunk = max(4, self.window_scratch_bytes // (4 * m.heads * a.score_ld) // 4 * 4)
        rows = min(n, chunk)
        scores = torch.empty(rows, m.heads, a.score_ld, **f32)
        ml = torch.empty(rows, m.heads, a.splits, 2, **f32)
        o_part = torch.empty(rows, a.splits, HV, **f32)
        a.scores, a.ml, a.o_part = scores.data_ptr(), ml.data_ptr(), o_part.data_ptr()
        gate, ld_gate = a.gate, a.ld_gate
        with self.timed(name):
            for at in range(0, n, chunk):
                a.n = min(chunk, n - at)
                a.qn, a.y = qn.data_ptr() + 4 * at * HD, y.data_ptr() + es * at * HV
                a.tok_seq, a.tok_pos = c.tok_seq.data_ptr() + 4 * at, c.tok_pos.data_ptr() + 4 * at
                if gate:
                    a.gate = gate + es * at * ld_gate
                H.check(self.lib.b200h_window_attention(C.byref(a)), "window_attention")

    def conv_attention_mixer(self, i, h, c, run=None):
        """Convolved rotary attention of layer i: one stacked projection (q | k); one kernel convolves every channel over the
        sequence (state: the last taps-1 projected rows), stores the convolved key as the VALUE, rotates, norms per head and stores
        the key; then attention over all cached keys with the sink in the denominator.  Returns [n, heads * vdim] (T)."""
        r = i if run is None else run
        m, w, lib, dev, T, n = self.spec.layers[i].mixer, self.w, self.lib, self.device, self.T, c.n
        p = f"l{i}."
        HD, HV = m.heads * m.dim, m.heads * m.vdim
        with self.timed("gemm in"):
            proj = self._linear(h, w[p + "in"])
        qn = torch.empty(n, HD, dtype=torch.float32, device=dev)
        pa = H.ConvPrepArgs()
        pa.n, pa.batch, pa.heads, pa.kv_heads, pa.dim, pa.taps, pa.block_len = n, c.batch, m.heads, m.kv_heads, m.dim, m.conv_taps, self.block_len
        pa.eps = self.spec.norm_eps
        pa.rot = H.Rotary(w[p + "freqs"].data_ptr(), m.rot.dims // 2, w[p + "mag"])
        pa.qk, pa.ld, pa.conv = proj.data_ptr(), proj.stride(0), w[p + "conv"].data_ptr()
        pa.state, pa.slot_stride, pa.qn = c.state.ptr(self.conv_off[r]), c.state.storage.stride(0), qn.data_ptr()
        pa.tok_seq, pa.tok_pos, pa.cu_q, pa.seq_slot = c.tok_seq.data_ptr(), c.tok_pos.data_ptr(), c.cu_q.data_ptr(), c.seq_slot.data_ptr()
        pa.block_ptrs, pa.cu_blocks = c.block_ptrs.data_ptr(), c.cu_blocks.data_ptr()
        pa.layer_off, pa.v_off, pa.dtype, pa.stream = self.cache_off[r], self.v_off[r], self.dt, self._stream()
        with self.timed("conv + rotate + head norm + cache store"):
            H.check(lib.b200h_conv_rope_prep(C.byref(pa)), "conv_rope_prep")
        a = H.WindowArgs()
        a.n, a.heads, a.kv_heads, a.dim, a.vdim, a.block_len, a.window = n, m.heads, m.kv_heads, m.dim, m.vdim, self.block_len, m.window
        a.splits = self.window_splits(n, m.window, c.max_pos)
        a.scale, a.softcap, a.eps = m.scale, 0.0, self.spec.norm_eps
        if m.sink is not None:
            a.sink = w[p + "sink"].data_ptr()
        a.qn = qn.data_ptr()
        a.tok_seq, a.tok_pos = c.tok_seq.data_ptr(), c.tok_pos.data_ptr()
        a.block_ptrs, a.cu_blocks = c.block_ptrs.data_ptr(), c.cu_blocks.data_ptr()
        a.layer_off, a.v_off, a.dtype, a.stream = self.cache_off[r], self.v_off[r], self.dt, self._stream()
        y = torch.empty(n, HV, dtype=T, device=dev)
        self._window_attend(a, m, c, qn, y, "attention with sink")
        return y

    def ssm_mixer(self, i, h, c, run=None):
        """State-space mixer of layer i: one projection (z | x | B | C | dt), the short convolution with bias and silu over
        x | B | C (float out), the per-head recurrence on the sequence's float state, then the gate silu(z) and the RMS norm in
        groups.  Returns [n, heads * vdim] (T)."""
        r = i if run is None else run
        m, w, lib, dev, n = self.spec.layers[i].mixer, self.w, self.lib, self.device, c.n
        p = f"l{i}."
        with self.timed("gemm in"):
            proj = self._linear(h, w[p + "in"])
        ld, es, base = proj.stride(0), proj.element_size(), proj.data_ptr()
        stride, st = c.state.storage.stride(0), self._stream()
        xbc = torch.empty(n, m.conv_channels, dtype=torch.float32, device=dev)
        with self.timed("short conv + silu"):
            H.check(lib.b200h_short_conv(base + es * m.inner, ld, w[p + "conv"].data_ptr(), w[p + "conv.b"].data_ptr(), 1,
                                         c.state.ptr(self.conv_off[r]), stride, c.tok_seq.data_ptr(), c.cu_q.data_ptr(),
                                         c.seq_slot.data_ptr(), xbc.data_ptr(), n, c.batch, m.conv_channels, m.conv_taps, self.dt, st),
                    "short_conv")
        o = torch.empty(n, m.inner, dtype=torch.float32, device=dev)
        steps = torch.empty(n, m.heads, 2, dtype=torch.float32, device=dev)
        with self.timed("state-space scan"):
            H.check(lib.b200h_ssm_scan(xbc.data_ptr(), base + es * (m.inner + m.conv_channels), ld, w[p + "dt_bias"].data_ptr(),
                                       w[p + "A_log"].data_ptr(), w[p + "D"].data_ptr(), c.state.ptr(self.mix_off[r]), stride,
                                       c.cu_q.data_ptr(), c.seq_slot.data_ptr(), n, c.batch, m.heads, m.vdim, m.state, m.groups,
                                       steps.data_ptr(), o.data_ptr(), self.dt, st), "ssm_scan")
        y = torch.empty(n, m.inner, dtype=self.T, device=dev)
        with self.timed("gate + grouped norm"):
            H.check(lib.b200h_gate_group_norm(o.data_ptr(), base, ld, w[p + "mixnorm"].data_ptr(), n, m.inner, m.norm_groups,
                                              self.spec.norm_eps, y.data_ptr(), self.dt, st), "gate_group_norm")
        return y

    def dense_mlp(self, i, h):
        """Dense feed-forward of layer i over its input h [n, width] (T): down(act(up h)) -> [n, width] (T)."""
        f, w = self.spec.layers[i].mlp, self.w
        if f.act not in ("relu2", "xielu"):
            raise NotImplementedError(f"activation {f.act!r}")
        with self.timed("gemm up"):
            a = self._linear(h, w[f"l{i}.up"])
        with self.timed("activation"):
            if f.act == "xielu":
                H.check(self.lib.b200h_xielu(a.data_ptr(), a.numel(), w[f"l{i}.act"].data_ptr(), self.dt, self._stream()), "xielu")
            else:
                H.check(self.lib.b200h_relu2(a.data_ptr(), a.numel(), self.dt, self._stream()), "relu2")
        with self.timed("gemm down"):
            return self._linear(a, w[f"l{i}.down"])

    def _logits(self, xn):
        """Float logits of normed rows: bf16 operands keep a float result (no rounding of the logits to bf16)."""
        out = self._head_product(xn)
        cap = self.spec.logit_softcap
        if cap > 0 and out.numel():
            H.check(self.lib.b200h_softcap(out.data_ptr(), out.numel(), cap, self._stream()), "softcap")
        return out

    def _head_product(self, xn):
        return self._linear_f32(xn, self.w["head"])

    def _linear_f32(self, x, wt):
        """x wt^T with a float result (bf16 operands accumulate and stay in float)."""
        if self.T is torch.float32 or x.device.type != "cuda":
            return torch.mm(x.float(), wt.float().t())
        try:
            return torch.mm(x, wt.t(), out_dtype=torch.float32)
        except RuntimeError:            # a shape the float-output GEMM refuses: float operands (same values, wider reads)
            return torch.mm(x.float(), wt.float().t())

    # ---- the mechanisms, one method each (the step above strings them together; tests call them alone)
    def attention_splits(self, n, heads, max_pos):
        """Key ranges per row of a latent-attention launch: enough to reach `attention_warps` warps, at least two pages each,
        a power of two (so that a growing context changes it rarely: the engine keys its decode graphs on it)."""
        want = min(self.attention_warps // max(n * heads, 1), (max_pos // self.block_len + 2) // 2, 64)
        splits = 1
        while splits * 2 <= want:
            splits *= 2
        return splits

    def decode_key(self, n, max_pos):
        """What a captured decode step depends on besides its row count."""
        key = []
        for l in self.spec.layers:
            if l.mixer.kind == "latent_attention":
                key.append(self.attention_splits(n, l.mixer.heads, max_pos))
            elif l.mixer.kind in ("window_attention", "conv_attention", "paired"):
                m = l.mixer.left if l.mixer.kind == "paired" else l.mixer
                span = getattr(m, "span", m.window)
                key.append((self.window_splits(n, span, max_pos), self.window_score_ld(span, max_pos)))
        return tuple(key)

    def conv_input(self, i, x, c, run=None, sub=1):
        """What a sublayer of layer i reads (sub 1: the mixer, 2: the feed-forward): x + causal convolution of x over the sequence
        (as T); advances that sublayer's conv state of the run."""
        s, w = self.spec, self.w
        r = i if run is None else run
        off = self.conv_off[r] if sub == 1 else self.conv2_off[r]
        h = torch.empty(c.n, s.width, dtype=self.T, device=self.device)
        with self.timed("causal conv"):
            H.check(self.lib.b200h_causal_conv(x.data_ptr(), w[f"l{i}.canon{sub}"].data_ptr(), c.state.ptr(off),
                                               c.state.storage.stride(0), c.tok_seq.data_ptr(), c.cu_q.data_ptr(), c.seq_slot.data_ptr(),
                                               h.data_ptr(), c.n, c.batch, s.width, s.conv_taps, self.dt, self._stream()), "causal_conv")
        return h

    def latent_mixer(self, i, h, c, run=None):
        """Latent attention of layer i over rows h [n, width] (T): one stacked projection (query latent | key/value latent +
        shared rotated key | gate), norms + rotation + cache store, query expansion, attention over the paged latents with the
        sink, value expansion and gate.  Returns the gated heads [n, heads * vdim] (T), the output projection's input."""
        m, w, lib, dev, T, n = self.spec.layers[i].mixer, self.w, self.lib, self.device, self.T, c.n
        p = f"l{i}."
        f32 = dict(dtype=torch.float32, device=dev)
        with self.timed("gemm in"):
            proj = self._linear(h, w[p + "in"])
        ld, es = proj.stride(0), proj.element_size()
        a = H.LatentArgs()
        a.n, a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.q_rank = n, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank
        a.block_len, a.scale, a.eps = self.block_len, m.scale, self.spec.norm_eps
        a.rot = H.Rotary(w[p + "freqs"].data_ptr(), m.rot.dims // 2, w[p + "mag"])
        a.dq, a.ld_dq = proj.data_ptr(), ld
        a.dkv, a.ld_dkv = proj.data_ptr() + es * m.q_rank, ld
        gate = proj.data_ptr() + es * (m.q_rank + m.kv_rank + m.rot_dim)
        a.q_norm, a.kv_norm, a.sink = w[p + "dq.norm"].data_ptr(), w[p + "dkv.norm"].data_ptr(), w[p + "sink"].data_ptr()
        cq = torch.empty(n, m.q_rank, dtype=T, device=dev)
        a.cq = cq.data_ptr()
        a.tok_seq, a.tok_pos = c.tok_seq.data_ptr(), c.tok_pos.data_ptr()
        a.block_ptrs, a.cu_blocks = c.block_ptrs.data_ptr(), c.cu_blocks.data_ptr()
        r = i if run is None else run
        a.layer_off, a.rot_off, a.dtype, a.stream = self.cache_off[r], self.rot_off[r], self.dt, self._stream()
        with self.timed("latent norm + rotate + cache store"):
            H.check(lib.b200h_latent_prep(C.byref(a)), "latent_prep")
        with self.timed("gemm query up"):
            q = self._linear(cq, w[p + "uq"])
        a.q, a.ld_q = q.data_ptr(), q.stride(0)
        q_rot = torch.empty(n, m.heads, m.rot_dim, **f32)
        a.q_rot = q_rot.data_ptr()
        with self.timed("rotate query"):
            H.check(lib.b200h_rotate_query(C.byref(a)), "rotate_query")
        with self.timed("gemm query into latent"):
            # q_lat[t, h] = uk_h^T q_plain[t, h]: one batched GEMM over the heads, float result
            q_plain = q.view(n, m.heads, m.dim + m.rot_dim)[:, :, :m.dim].transpose(0, 1)
            q_lat = self._bmm(q_plain, w[p + "uk"].view(m.heads, m.dim, m.kv_rank)).transpose(0, 1).contiguous()
        # key ranges per row: one for prompt portions (rows x heads already fill the SMs), several whole-page ranges when a step
        # of few rows would leave most SMs idle
        splits = self.attention_splits(n, m.heads, c.max_pos)
        o_lat = torch.empty(n, m.heads, splits, m.kv_rank, **f32)
        ml = torch.empty(n, m.heads, splits, 2, **f32)
        o_heads = torch.empty(m.heads, n, m.kv_rank, dtype=T, device=dev)
        a.q_lat, a.o_lat, a.ml, a.splits, a.o_heads = q_lat.data_ptr(), o_lat.data_ptr(), ml.data_ptr(), splits, o_heads.data_ptr()
        with self.timed("latent attention"):
            H.check(lib.b200h_latent_attention(C.byref(a)), "latent_attention")
        with self.timed("gemm latent into values"):
            o = self._bmm(o_heads, w[p + "uv"].view(m.heads, m.vdim, m.kv_rank).transpose(1, 2))       # float [heads, n, vdim]
        y = torch.empty(n, m.heads * m.vdim, dtype=T, device=dev)
        with self.timed("output gate"):
            H.check(lib.b200h_head_gate(o.data_ptr(), gate, ld, n, m.heads, m.vdim, y.data_ptr(), self.dt, self._stream()), "head_gate")
        return y

    def _bmm(self, a, b):
        """Batched product with a float result (bf16 operands accumulate and stay in float)."""
        if self.T is torch.float32 or a.device.type != "cuda":
            return torch.bmm(a.float(), b.float())
        try:
            return torch.bmm(a, b, out_dtype=torch.float32)
        except RuntimeError:
            return torch.bmm(a.float(), b.float())

    def decay_mixer(self, i, h, c, run=None):
        """Decayed linear attention of layer i: one stacked projection (q | k | v | gate), the per-head recurrence on the
        sequence's float state, then unit-rms norm over the concatenated heads times sigmoid(gate).  Returns [n, heads * vdim] (T)."""
        m, w, lib, dev, n = self.spec.layers[i].mixer, self.w, self.lib, self.device, c.n
        p = f"l{i}."
        HD, HV = m.heads * m.dim, m.heads * m.vdim
        with self.timed("gemm in"):
            proj = self._linear(h, w[p + "in"])
        ld, es, base = proj.stride(0), proj.element_size(), proj.data_ptr()
        o = torch.empty(n, m.heads, m.vdim, dtype=torch.float32, device=dev)
        st = self._stream()
        with self.timed("decayed linear attention"):
            H.check(lib.b200h_decay_attention(base, base + es * HD, base + es * 2 * HD, ld, w[p + "decay"].data_ptr(),
                                              c.state.ptr(self.mix_off[i if run is None else run]), c.state.storage.stride(0), c.cu_q.data_ptr(),
                                              c.seq_slot.data_ptr(), c.batch, m.heads, m.dim, m.vdim, o.data_ptr(), self.dt, st),
                    "decay_attention")
        y = torch.empty(n, HV, dtype=self.T, device=dev)
        with self.timed("gated unit norm"):
            H.check(lib.b200h_gated_rms(o.data_ptr(), w[p + "mixnorm"].data_ptr(), base + es * (2 * HD + HV), ld, n, HV, self.spec.norm_eps,
                                        y.data_ptr(), self.dt, st), "gated_rms")
        return y

    def routed_experts(self, i, x, xt, n):
        """Routed experts of layer i: the router reads the float stream x (or, when x is None, the experts' own input xt), the
        experts the T rows xt.  The spec chooses the router's scores (softmax / sigmoid), the expert's activation and whether a
        score scales the expert's output or its input.  Returns float [n, top, width]: each chosen expert's (weighted) output,
        summed by the kernel that takes it into the stream."""
        f, w, lib, dev = self.spec.layers[i].mlp, self.w, self.lib, self.device
        p, W, st = f"l{i}.", self.spec.width, self._stream()
        ids = torch.empty(n, f.top, dtype=torch.int32, device=dev)
        wts = torch.empty(n, f.top, dtype=torch.float32, device=dev)
        with self.timed("router"):
            src, src_dt = (xt, self.dt) if x is None else (x, H.F32)
            if f.grouped:
                if f.score != "sigmoid":
                    raise NotImplementedError("a router that chooses among groups scores with sigmoids")
                H.check(lib.b200h_route_grouped(src.data_ptr(), src_dt, w[p + "router"].data_ptr(),
                                                w[p + "correction"].data_ptr() if f.correction else None, n, W, f.experts, f.top, f.groups,
                                                f.keep, f.group_top, int(f.renorm), f.scale, ids.data_ptr(), wts.data_ptr(), st), "route_grouped")
            else:
                H.check(lib.b200h_route_scored(src.data_ptr(), src_dt, w[p + "router"].data_ptr(), n, W, f.experts, f.top, H.SCORE_FN[f.score],
                                               ids.data_ptr(), wts.data_ptr(), st), "route")
        out = torch.empty(n, f.top, W, dtype=torch.float32, device=dev)
        self.last_routing = (ids, wts)
        capturing = dev.type == "cuda" and torch.cuda.is_current_stream_capturing()      # the grouped path reads counts on the host
        if n * f.top >= self.grouped_experts_rows * f.experts and not capturing:
            with self.timed("experts (grouped GEMMs)"):
                self._grouped_experts(i, xt, ids, wts, out, n)
            return out
        with self.timed("experts"):
            a = H.ExpertArgs()
            a.n, a.width, a.ff, a.experts, a.top, a.dtype = n, W, f.ff, f.experts, f.top, self.dt
            a.act, a.scale_input = H.EXPERT_ACT[f.act], int(f.scale_input)
            a.x, a.up, a.down = xt.data_ptr(), w[p + "up"].data_ptr(), w[p + "down"].data_ptr()
            if f.act == "silu_gate":
                a.gate = w[p + "gate"].data_ptr()
            a.ids, a.wts, a.out = ids.data_ptr(), wts.data_ptr(), out.data_ptr()
            mid = torch.empty(n * f.top, f.ff, dtype=self.T, device=dev)
            lists = torch.empty(f.experts * (n * f.top + 1), dtype=torch.int32, device=dev)
            a.mid, a.counts, a.lists, a.stream = mid.data_ptr(), lists.data_ptr(), lists.data_ptr() + 4 * f.experts, st
            H.check(lib.b200h_experts(C.byref(a)), "experts")
        return out

    def _grouped_experts(self, i, xt, ids, wts, out, n):
        """Prompt portions: rows are sorted by chosen expert (one host read of the per-expert counts), every expert runs its
        gate / up / down GEMMs over its rows, and the results return to their (row, choice) places times the router's score
        (a score that scales the expert's input goes to the first product's rows instead, inside the activation kernel).
        A step of few rows uses the expert-major kernels instead (b200h_experts: no host read, every expert's weights once)."""
        f, w, lib, st = self.spec.layers[i].mlp, self.w, self.lib, self._stream()
        p = f"l{i}."
        flat = ids.view(-1).long()
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=f.experts).cpu().tolist()
        xg = xt.index_select(0, torch.div(order, f.top, rounding_mode="floor"))
        m = n * f.top
        res = torch.empty(m, self.spec.width, dtype=self.T, device=self.device)
        if f.scale_input and f.act != "relu2":
            raise NotImplementedError("grouped experts: a score on the input of a gated expert")
        w_in = wts.view(-1).index_select(0, order).contiguous() if f.scale_input else None
        at = 0
        for e, cnt in enumerate(counts):
            if cnt == 0:
                continue
            seg = xg[at:at + cnt]
            if f.act == "relu2":
                g = torch.mm(seg, w[p + "up"][e].t())
                H.check(lib.b200h_scaled_relu2(g.data_ptr(), None if w_in is None else w_in.data_ptr() + 4 * at, cnt, f.ff, self.dt, st),
                        "scaled_relu2")
            else:
                g, u = torch.mm(seg, w[p + "gate"][e].t()), torch.mm(seg, w[p + "up"][e].t())
                H.check(lib.b200h_silu_mul(g.data_ptr(), u.data_ptr(), g.data_ptr(), g.numel(), self.dt, st), "silu_mul")
            torch.mm(g, w[p + "down"][e].t(), out=res[at:at + cnt])
            at += cnt
        slot = order.to(torch.int32)
        H.check(lib.b200h_weighted_scatter(res.data_ptr(), slot.data_ptr(), None if f.scale_input else wts.data_ptr(), out.data_ptr(), m,
                                           self.spec.width, self.dt, st), "weighted_scatter")

    def argmax(self, logits):
        """Greedy ids of float logits [r, vocab] (device int32 [r])."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        st = self._stream()
        H.check(self.lib.b200h_argmax(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], out.data_ptr(), st), "argmax")
        return out
