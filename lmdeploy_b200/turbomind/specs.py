"""Model geometries on the hot path (public HF configs of these models --
lmdeploy/turbomind/models/internlm2.py:70-84, models/llama.py:44-99 read the same fields)."""
from dataclasses import dataclass, replace


@dataclass(frozen=True)
class RopeSpec:
    """RoPE parameters as the reference parses them from an HF config (lmdeploy/turbomind/models/utils.py:76-166) and
    hands them to init_rope_kernel_param (src/turbomind/models/attention_weight.cc:37-93)."""
    type: str = "default"               # 'default' | 'linear' | 'llama3' | 'yarn' | 'dynamic' (prompts within the trained context)
    dim: int = 128                      # rotated dims = head_dim * partial_rotary_factor
    base: float = 10000.0
    factor: float = 0.0
    max_position_embeddings: int = 0    # the model's context length (yarn correction range; see loader.parse_rope)
    low_freq_factor: float = 1.0        # llama3
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192
    attention_factor: float = 1.0       # yarn
    beta_fast: float = 32.0
    beta_slow: float = 1.0

    TYPE_ID = {"default": 1, "linear": 2, "yarn": 4, "llama3": 5}

    def dynamic_ntk_base(self, prompt_len):
        """The rope base the reference gives a request of `prompt_len` prompt tokens under dynamic NTK scaling
        (init_dynamic_ntk, src/turbomind/models/llama/unified_attention_layer.cc:228-243)."""
        base = self.base
        if self.type == "dynamic" and self.factor > 1.0 and prompt_len > self.max_position_embeddings:
            f = self.factor * prompt_len / self.max_position_embeddings - (self.factor - 1.0)
            base *= f ** (self.dim / (self.dim - 2.0))
        return base

    def config_fields(self):
        """Field values of b200_rope_config (include/b200_turbomind.h) in declaration order, without exact_math --
        the counterpart of copy_rope_config (lmdeploy/turbomind/models/utils.py:170-187)."""
        if self.type == "dynamic":
            # the kernels see plain RoPE with the config's base and no position scaling -- exactly what the reference
            # computes for a prompt that fits the trained context (RopeType::kDynamic: inv_factor = 1, base unchanged)
            return dict(RopeSpec(type="default", dim=self.dim, base=self.base, factor=0.0,
                                 max_position_embeddings=self.max_position_embeddings).config_fields())
        if self.type not in self.TYPE_ID:
            raise NotImplementedError(f"rope type {self.type!r} (supported: {sorted(self.TYPE_ID)})")
        return dict(type=self.TYPE_ID[self.type], dim=self.dim, base=self.base, factor=self.factor,
                    max_position_embeddings=self.max_position_embeddings,
                    llama3_low_freq_factor=self.low_freq_factor, llama3_high_freq_factor=self.high_freq_factor,
                    llama3_original_max_position_embeddings=self.original_max_position_embeddings,
                    yarn_attention_factor=self.attention_factor, yarn_beta_fast=self.beta_fast, yarn_beta_slow=self.beta_slow)


@dataclass(frozen=True)
class ModelSpec:
    name: str
    arch: str                 # 'internlm2' | 'llama' | 'qwen2'
    hidden: int
    layers: int
    heads: int
    kv_heads: int
    inter: int
    vocab: int
    rope_theta: float
    head_dim: int = 128
    norm_eps: float = 1e-5
    rope_type: str = "default"      # 'default' | 'llama3'
    rope_factor: float = 0.0
    weight_format: str = "awq"      # on-GPU weight format: 'awq' (u4 g128, any int4 checkpoint family) | 'fp16' | 'fp8'
    dtype: str = "f16"
    checkpoint_format: str = None   # how the checkpoint packs it: 'awq' | 'gptq' | 'compressed-tensors' | None
    qkv_bias: bool = False          # q/k/v projections carry a bias (Qwen2 family), applied by the attention prologue
    qk_norm: bool = False           # per-head RMSNorm of q and k before RoPE (Qwen3 family)
    rope: RopeSpec = None           # full RoPE description (checkpoints); None = rope_type / rope_theta / rope_factor above
    max_position_embeddings: int = 0   # config.max_position_embeddings (0 = unknown); feeds the RoPE config
    session_len: int = 0               # default session length the reference derives from the config (0 = unknown)

    def tiny(self, layers=2):
        return replace(self, layers=layers)


SPECS = {
    "internlm2-1.8b": ModelSpec("internlm2-1.8b", "internlm2", 2048, 24, 16, 8, 8192, 92544, 1e6, weight_format="fp16"),
    "internlm2-7b": ModelSpec("internlm2-7b", "internlm2", 4096, 32, 32, 8, 14336, 92544, 1e6),
    "internlm2-20b": ModelSpec("internlm2-20b", "internlm2", 6144, 48, 48, 8, 16384, 92544, 1e6),
    "llama3-8b": ModelSpec("llama3-8b", "llama", 4096, 32, 32, 8, 14336, 128256, 5e5, weight_format="fp16"),
    # Qwen2-7B: q/k/v bias, GQA group 7 (public HF config; lmdeploy/turbomind/models/qwen2.py)
    "qwen2-7b": ModelSpec("qwen2-7b", "qwen2", 3584, 28, 28, 4, 18944, 152064, 1e6, qkv_bias=True),
    "llama3-70b": ModelSpec("llama3-70b", "llama", 8192, 80, 64, 8, 28672, 128256, 5e5, weight_format="fp8",
                            dtype="bf16"),
}


# ---------------------------------------------------------------------------------------------------- hybrid decoders
# Decoders whose layers differ from one another: each layer names its sequence mixer (attention over a cached latent,
# or a decayed linear-attention recurrence), its feed-forward (routed experts, or none) and their sizes; the per-layer
# record is the whole description, so another stack of the same mechanisms is another list.

@dataclass(frozen=True)
class RotarySpec:
    """Rotation of interleaved pairs (2i, 2i+1) of the first `dims` dimensions by position * f_i, f_i = base^(-2i/dims).
    scaling = (factor, original, fast, slow) or None: frequencies are blended with f_i / factor along a ramp over the
    pair index whose ends are the pairs that make `fast` and `slow` turns over `original` positions, and cos / sin grow
    by 0.1 ln(factor) + 1 (the YaRN recipe)."""
    dims: int
    base: float
    scaling: tuple = None
    linear: float = 1.0                 # every frequency is divided by this (positions stretched by a constant)

    def frequencies(self):
        """-> ([angle per position of pair i], factor on cos and sin), in double precision."""
        import math
        f = [self.base ** (-2.0 * i / self.dims) / self.linear for i in range(self.dims // 2)]
        if self.scaling is None:
            return f, 1.0
        factor, original, fast, slow = self.scaling

        def pair_of(turns):
            return self.dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

        lo = max(math.floor(pair_of(fast)), 0)
        hi = min(math.ceil(pair_of(slow)), self.dims - 1)
        span = max(hi - lo, 0.001)
        out = []
        for i, fi in enumerate(f):
            ramp = min(max((i - lo) / span, 0.0), 1.0)
            out.append(fi / factor * ramp + fi * (1.0 - ramp))
        return out, 0.1 * math.log(factor) + 1.0


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose keys and values are expanded from one cached latent per token, plus one rotated key part shared by
    all heads; queries pass through a latent of their own; a learned per-head sink joins the softmax denominator."""
    heads: int
    dim: int            # unrotated query / key dimensions per head
    rot_dim: int        # rotated ones
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: RotarySpec
    kind = "latent_attention"


@dataclass(frozen=True)
class DecayAttentionSpec:
    """Linear attention with a fixed decay per head: S <- decay_h S + k v^T, o = S^T q."""
    heads: int
    dim: int
    vdim: int
    decay: tuple
    kind = "lightning"


@dataclass(frozen=True)
class WindowAttentionSpec:
    """Softmax attention with grouped key/value heads over a sliding window of cached keys and values, without rotation.
    Score of query i and key j (max(0, i - window + 1) <= j <= i): scale * q.k, capped as softcap * tanh(. / softcap), minus
    r1_h * ln(1 + r2_h * (i - j)); after the softmax the heads' weight rows are recombined by a [heads, heads] matrix; the
    concatenated heads are gated by sigmoid of a projection of the mixer's input.  The optional parts are switches, so that
    another design can use the mechanism with some of them off."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0               # visible positions, the query's own included; 0: all earlier positions
    softcap: float = 0.0          # 0: scores are not capped
    qk_norm: bool = True          # RMS norm of q and of k over the whole projection (all heads at once), plain weights
    bias: bool = True             # q, k and v projections carry a bias
    distance_bias: bool = True    # per-head r1, r2
    talking_heads: bool = True    # [heads, heads] recombination of the softmax weights
    gate: bool = True
    # switches of a design that rotates: the norm of q and k is PER HEAD over dim with a weight of dim entries shared by the heads,
    # then interleaved pairs turn (rot); a row sees only the keys of its own chunk of `chunk` positions (counted from position 0);
    # the [heads, heads] matrix mixes the heads' SCORES before the softmax instead of their weights after it; a learned score per
    # head joins the softmax denominator (sink); the gate is ONE number per head.
    head_norm: bool = False
    rot: RotarySpec = None
    chunk: int = 0
    talk_scores: bool = False
    sink: bool = False
    gate_per_head: bool = False
    kind = "window_attention"

    @property
    def span(self):
        """The most keys a row sees (0: all earlier positions)."""
        return min(self.window, self.chunk) if self.window and self.chunk else (self.window or self.chunk)


@dataclass(frozen=True)
class ConvAttentionSpec:
    """Causal softmax attention with grouped key/value heads whose query and key projections each pass a short causal
    convolution per channel (taps weights, no bias, the last column is the current token's).  The convolved q and k are rotated
    (RotarySpec, interleaved pairs of the first rot.dims dimensions of every head) and THEN divided by their root mean square
    per head (no weight).  values_from_keys: there is no value projection, a key/value head's value is its convolved key before
    rotation and norm (so vdim == dim).  sink: a constant score that joins the softmax denominator and carries no value
    (p_j = exp(s_j) / (exp(sink) + sum exp(s_j))); None: a plain softmax."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv_taps: int
    rot: RotarySpec
    window: int = 0               # visible positions, the query's own included; 0: all earlier positions
    sink: float = 0.0
    values_from_keys: bool = True
    kind = "conv_attention"


@dataclass(frozen=True)
class SsmSpec:
    """Selective state-space mixer with a scalar decay per head and token.  One projection yields z | x | B | C | dt
    (inner = heads * vdim, groups * state each for B and C, one dt per head); x, B and C pass a short causal convolution with
    bias and silu; dt <- softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T ([state, vdim], float),
    y = S^T C + D x; y * silu(z) is RMS-normed in norm_groups equal parts, times a weight, then projected."""
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv_taps: int
    kind = "mamba2"

    @property
    def inner(self):
        return self.heads * self.vdim

    @property
    def conv_channels(self):
        return self.inner + 2 * self.groups * self.state

    @property
    def proj_cols(self):
        return 2 * self.inner + 2 * self.groups * self.state + self.heads


@dataclass(frozen=True)
class ChannelDecaySpec:
    """Linear recurrence whose decay depends on the token, per head and key channel:
        w_t = exp(-exp(W2 tanh(W1 b_w) + w0)),  o_t = (S + diag(u) k_t v_t^T)^T r_t,  S <- diag(w_t) S + k_t v_t^T
    with S a [dim, dim] float matrix per head.  Each of r, k, v, the gate g and the decay reads its own blend b_s = a_t + (a_(t-1) -
    a_t) * mu_s of the mixer's input with the previous token's; every head's o is divided by its root mean square, times a
    weight, times silu(W_g b_g), then projected.  `rank` is the inner size of the decay's two matrices."""
    heads: int
    dim: int
    rank: int
    kind = "channel_decay"

    @property
    def vdim(self):
        return self.dim


@dataclass(frozen=True)
class PairedMixerSpec:
    """Two mixers side by side on the same input, each with an output projection of its own; the result is
    (rms(left) * w_left + rms(right) * w_right) / 2 with RMS norms over the model width."""
    left: object                        # WindowAttentionSpec
    right: object                       # ChannelDecaySpec
    kind = "paired"


@dataclass(frozen=True)
class RoutedExpertsSpec:
    experts: int
    top: int
    ff: int
    score: str = "softmax"        # router scores: 'softmax' over all experts | 'sigmoid' of every logit on its own
    act: str = "silu_gate"        # expert: 'silu_gate' = down(silu(gate h) * up h) | 'relu2' = down(relu(up h)^2), no gate matrix
    scale_input: bool = False     # the router's score multiplies the expert's input instead of its output
    # a router that chooses among groups (score 'sigmoid' only): a learned correction joins the scores for the CHOICE; the experts form
    # `groups` equal groups of neighbours, a group's score is the sum of its `group_top` largest choice scores and only the `keep` best
    # groups stay eligible; the chosen experts' scores are divided by their sum (renorm) and multiplied by `scale`.
    grouped: bool = False
    correction: bool = False
    groups: int = 1
    keep: int = 1
    group_top: int = 2
    renorm: bool = False
    scale: float = 1.0
    kind = "moe"


@dataclass(frozen=True)
class DenseMlpSpec:
    """down(act(up h)); act 'relu2' = the square of relu; 'xielu' = softplus(p) z^2 + z / 2 for z > 0 and
    (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise, with the two learned numbers p, q of the layer's 'mlp.act'."""
    ff: int
    act: str = "relu2"
    kind = "dense"


@dataclass(frozen=True)
class HashedBigramSpec:
    """A second embedding table added to the first: row (previous token * mul_prev + token * mul_cur) mod buckets, and row `buckets`
    (the last of buckets + 1) for a sequence's first token."""
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class HybridLayerSpec:
    mixer: object                       # Latent / Decay / Window / Conv attention spec | SsmSpec | PairedMixerSpec
    mlp: object = None                  # RoutedExpertsSpec | DenseMlpSpec | None: the layer has no feed-forward


@dataclass(frozen=True)
class HybridSpec:
    name: str
    arch: str
    width: int
    vocab: int
    layers: tuple                       # of HybridLayerSpec
    norm_eps: float
    norm_groups: int
    conv_taps: int
    embedding_scale: float
    dtype: str = "bf16"                 # 'bf16' | 'f32': the type of projections and their weights
    session_len: int = 0
    # 'post_norm': conv -> mixer -> grouped RMS norm of the OUTPUT -> add, then the learned average over all earlier streams.
    # 'pre_norm':  each sublayer reads conv(norm(x)) with an RMS norm whose stored weight is the deviation from one, and its
    #              output is added to the stream as it is; the feed-forward has a conv of its own.
    block: str = "post_norm"
    max_positions: int = 0              # > 0: a learned vector per position is added to the embedding
    loop: tuple = None                  # (start, stop, times): layers start..stop-1 run `times` times in a row with the same weights,
    #                                     each pass with a cache and state of its own and a learned vector added before it
    # 'parallel' blocks: both sublayers read the SAME stream through offset norms of their own and their outputs join it together,
    #              x <- x + residual_mult * (mixer(n1(x)) + ff(n2(x))); the mixers carry their own convolutions (conv_taps is unused).
    residual_mult: float = 1.0
    logit_softcap: float = 0.0          # > 0: logits <- cap * tanh(logits / cap)
    tied_head: bool = False             # the head is the embedding table (no 'head' tensor)
    loop_readds_embedding: bool = False  # every pass of the loop but the first adds the embedding output to the stream before its vector
    # 'shared_norm' blocks: ONE norm per layer, x <- x + mixer(shift(n(x))) + ff(n(x)): the mixer reads the normed row blended with the
    #              previous token's normed row (h + (h' - h) * shift, a learned vector per layer), the feed-forward the row itself.
    plain_norms: bool = False           # norm weights are stored as the full factor also in pre-norm / parallel / shared-norm blocks
    bigram: HashedBigramSpec = None     # the embedding adds a hashed row of a second table chosen by the previous token
    hybrid = True

    @property
    def hidden(self):
        return self.width

    def runs(self):
        """[(layer index, pass index or None)] in execution order.  Caches and states belong to runs, weights to layers."""
        L = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(L)]
        a, b, times = self.loop
        return [(i, None) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)] + [(i, None) for i in range(b, L)]


def _gulozen_mixer(kind, m):
    if kind == "latent_attention":
        r = m["rot"]
        sc = r.get("scaling")
        rot = RotarySpec(int(r["dims"]), float(r["base"]),
                         None if not sc else (float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])))
        if rot.dims > m["rot_dim"] or rot.dims % 2:
            raise ValueError(f"rot.dims {rot.dims} does not fit rot_dim {m['rot_dim']}")
        return LatentAttentionSpec(int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]),
                                   int(m["q_rank"]), float(m["scale"]), rot)
    if kind == "lightning":
        decay = tuple(float(d) for d in m["decay"])
        if len(decay) != m["heads"]:
            raise ValueError(f"{len(decay)} decays for {m['heads']} heads")
        return DecayAttentionSpec(int(m["heads"]), int(m["dim"]), int(m["vdim"]), decay)
    raise NotImplementedError(f"mixer type {kind!r}")


def gulozen_spec(cfg, name="gulozen"):
    """config.json of a Gulozen checkpoint -> HybridSpec.  Every size and constant is read from the config."""
    layers = []
    for entry in cfg["layers"]:
        mlp = entry.get("mlp")
        if mlp is not None:
            if mlp.get("kind", "moe") != "moe":
                raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
            mlp = RoutedExpertsSpec(int(mlp["router"]["experts"]), int(mlp["router"]["top"]), int(mlp["expert"]["ff"]))
        layers.append(HybridLayerSpec(_gulozen_mixer(entry["type"], entry["mixer"]), mlp))
    return HybridSpec(name=name, arch="gulozen", width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=tuple(layers),
                      norm_eps=float(cfg["norm"]["eps"]), norm_groups=int(cfg["norm"]["groups"]),
                      conv_taps=int(cfg["canon"]["taps"]), embedding_scale=float(cfg["embedding"]["scale"]),
                      session_len=int(cfg.get("session_len", 0)))


def bodopel_spec(cfg, name="bodopel"):
    """config.json of a Bodopel checkpoint -> HybridSpec.  Every size and constant is read from the config."""
    layers = []
    for entry in cfg["layers"]:
        if entry["type"] != "attention":
            raise NotImplementedError(f"mixer type {entry['type']!r}")
        m = entry["mixer"]
        heads, kv_heads = int(m["heads"]), int(m["kv_heads"])
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads do not divide into {kv_heads} key/value heads")
        mixer = WindowAttentionSpec(heads, kv_heads, int(m["dim"]), int(m["vdim"]), float(m["scale"]),
                                    window=int((m.get("mask") or {}).get("size") or 0), softcap=float(m.get("softcap") or 0.0))
        mlp = entry.get("mlp")
        if mlp is not None:
            if mlp.get("kind", "dense") != "dense":
                raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
            mlp = DenseMlpSpec(int(mlp["ff"]))
        layers.append(HybridLayerSpec(mixer, mlp))
    loop = _loop_of(cfg, len(layers))
    return HybridSpec(name=name, arch="bodopel", width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=tuple(layers),
                      norm_eps=float(cfg["norm"]["eps"]), norm_groups=1, conv_taps=int(cfg["canon"]["taps"]),
                      embedding_scale=float(cfg["embedding"]["scale"]), session_len=int(cfg["max_positions"]), block="pre_norm",
                      max_positions=int(cfg["max_positions"]), loop=loop)


def _loop_of(cfg, layers):
    loop = cfg.get("loop")
    if loop is None:
        return None
    loop = (int(loop["start"]), int(loop["stop"]), int(loop["times"]))
    if not 0 <= loop[0] <= loop[1] <= layers or loop[2] < 1:
        raise ValueError(f"loop {loop} over {layers} layers")
    return None if loop[0] == loop[1] else loop


def _lifuzen_mixer(kind, m):
    if kind == "attention":
        heads, kv_heads, dim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
        vdim = int(m.get("vdim", dim))
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads do not divide into {kv_heads} key/value heads")
        if vdim != dim:
            raise ValueError(f"vdim {vdim} != dim {dim}: the values of this attention are its keys")
        rot = RotarySpec(int(m["rot"]["dims"]), float(m["rot"]["base"]))
        if rot.dims > dim or rot.dims % 2:
            raise ValueError(f"rot.dims {rot.dims} (even) does not fit dim {dim}")
        return ConvAttentionSpec(heads, kv_heads, dim, vdim, float(m["scale"]), int(m["conv"]), rot)
    if kind == "mamba2":
        s = SsmSpec(int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["norm_groups"]), int(m["conv"]))
        if s.heads % s.groups or s.inner % s.norm_groups:
            raise ValueError(f"{s.heads} heads in {s.groups} groups, {s.inner} channels in {s.norm_groups} norm groups")
        return s
    raise NotImplementedError(f"mixer type {kind!r}")


def lifuzen_spec(cfg, name="lifuzen"):
    """config.json of a Lifuzen checkpoint -> HybridSpec.  Every size and constant is read from the config."""
    layers = []
    for entry in cfg["layers"]:
        mlp = entry.get("mlp")
        if mlp is not None:
            if mlp.get("kind", "moe") != "moe":
                raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
            mlp = RoutedExpertsSpec(int(mlp["router"]["experts"]), int(mlp["router"]["top"]), int(mlp["expert"]["ff"]),
                                    score="sigmoid", act="relu2", scale_input=True)
            if not 1 <= mlp.top <= mlp.experts:
                raise ValueError(f"top {mlp.top} of {mlp.experts} experts")
        layers.append(HybridLayerSpec(_lifuzen_mixer(entry["type"], entry["mixer"]), mlp))
    return HybridSpec(name=name, arch="lifuzen", width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=tuple(layers),
                      norm_eps=float(cfg["norm"]["eps"]), norm_groups=1, conv_taps=1, embedding_scale=1.0,
                      session_len=int(cfg.get("session_len", 0)), block="parallel", loop=_loop_of(cfg, len(layers)),
                      residual_mult=float(cfg.get("residual_mult", 1.0)), logit_softcap=float(cfg.get("logit_softcap") or 0.0),
                      tied_head=True, loop_readds_embedding=True)


def _fogizen_left(m):
    heads, kv_heads, dim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    if heads % kv_heads:
        raise ValueError(f"{heads} query heads do not divide into {kv_heads} key/value heads")
    r = m["rot"]
    rot = RotarySpec(int(r["dims"]), float(r["base"]), linear=float((r.get("scaling") or {}).get("factor") or 1.0))
    if rot.dims > dim or rot.dims % 2:
        raise ValueError(f"rot.dims {rot.dims} (even) does not fit dim {dim}")
    return WindowAttentionSpec(heads, kv_heads, dim, int(m.get("vdim", dim)), float(m["scale"]), qk_norm=True, bias=True,
                               distance_bias=False, talking_heads=True, gate=True, head_norm=True, rot=rot,
                               chunk=int((m.get("mask") or {}).get("size") or 0), talk_scores=True, sink=True, gate_per_head=True)


def fogizen_spec(cfg, name="fogizen", tensor_shapes=None):
    """config.json of a Fogizen checkpoint -> HybridSpec.  Every size and constant is read from the config; the inner size of the
    decay's two matrices is a tensor's shape ('l<i>.mix.right.w1': [rank, width])."""
    layers = []
    for i, entry in enumerate(cfg["layers"]):
        if entry["type"] != "parallel":
            raise NotImplementedError(f"mixer type {entry['type']!r}")
        right = entry["mixer"]["right"]
        rank = int(right["rank"]) if "rank" in right else (int(tensor_shapes[f"l{i}.mix.right.w1"][0]) if tensor_shapes else 0)
        if rank < 1:
            raise ValueError(f"layer {i}: the decay's inner size is neither in the config nor a known tensor shape")
        mixer = PairedMixerSpec(_fogizen_left(entry["mixer"]["left"]), ChannelDecaySpec(int(right["heads"]), int(right["dim"]), rank))
        mlp = entry.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                mlp = DenseMlpSpec(int(mlp["ff"]), act="xielu")
            elif mlp["kind"] == "moe":
                r = mlp["router"]
                g = r.get("groups") or {}
                mlp = RoutedExpertsSpec(int(r["experts"]), int(r["top"]), int(mlp["expert"]["ff"]), score="sigmoid", grouped=True,
                                        correction=True, groups=int(g.get("count", 1)), keep=int(g.get("keep", g.get("count", 1))),
                                        renorm=True, scale=float(r.get("scale", 1.0)))
                if mlp.experts % mlp.groups or not 1 <= mlp.keep <= mlp.groups or not 1 <= mlp.top <= mlp.keep * (mlp.experts // mlp.groups):
                    raise ValueError(f"layer {i}: top {mlp.top} of {mlp.experts} experts in {mlp.groups} groups of which {mlp.keep} stay")
            else:
                raise NotImplementedError(f"feed-forward kind {mlp['kind']!r}")
        layers.append(HybridLayerSpec(mixer, mlp))
    b = (cfg.get("embedding") or {}).get("bigram")
    bigram = HashedBigramSpec(int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"])) if b else None
    return HybridSpec(name=name, arch="fogizen", width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=tuple(layers),
                      norm_eps=float(cfg["norm"]["eps"]), norm_groups=1, conv_taps=1, embedding_scale=1.0,
                      session_len=int(cfg.get("session_len", 0)), block="shared_norm", plain_norms=True, bigram=bigram)


# config.json "architecture" -> spec builder, for checkpoints that are not HF `architectures` configs
HYBRID_ARCHITECTURES = {"Gulozen": gulozen_spec, "Bodopel": bodopel_spec, "Lifuzen": lifuzen_spec, "Fogizen": fogizen_spec}
