"""Plain, slow restatement of the Lifuzen layer equations in torch on the CPU -- TEST INFRASTRUCTURE ONLY.

One function per mechanism, written token by token (explicit loops over positions, heads and experts; no paging, no
batching, no key ranges, no stacked projections): the opposite route from the product kernels in
lmdeploy_b200/csrc/hybrid, with which it shares no code.  `dt` is the dtype everything runs in (float64 by default).

Notation: n tokens of one sequence, W model width; weights are stored [out, in] and applied as x @ W.T; a "run" is one
execution of a layer (a looped layer has one run per pass, each with a cache / state of its own).

A Lifuzen layer is a PARALLEL block: both sublayers read the same stream through a norm of their own,
    x <- x + m * (mixer(n1(x)) + ff(n2(x))),      n(x) = x / sqrt(mean(x^2) + eps) * (1 + w).
Mixers: softmax attention whose values are its keys (before norm and rotation), with a short convolution on q and k, partial
interleaved rotation, a weightless per-head RMS norm AFTER the rotation and a sink of score 0 in the softmax denominator;
or a selective state-space recurrence with a scalar decay per head and token (S <- a_t S + dt_t B_t x_t^T).  Feed-forward:
routed experts with a sigmoid router whose score scales the expert's INPUT."""
import math

import torch


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the deviation from one."""
    return unit_rms(x, eps) * (1.0 + w)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0.0)


def short_conv(u, w, before, bias=None):
    """u [n, C]; w [C, taps]; `before` [taps-1, C] = the inputs that precede u (zeros at a sequence's start).
    y_t = bias + sum_j w[:, j] * u_(t - taps + 1 + j).  Returns (y, the last taps-1 inputs)."""
    taps = w.shape[1]
    full = torch.cat([before, u], 0)                       # index t + taps - 1 is u_t
    y = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            y[t] = y[t] + w[:, j] * full[t + j]
        if bias is not None:
            y[t] = y[t] + bias
    return y, full[full.shape[0] - (taps - 1):].clone()


def rotate_pairs(v, position, dims, base):
    """v [heads, dim]: pair (2i, 2i+1), i < dims/2, turns by position * base^(-2i/dims); the other dimensions stay."""
    out = v.clone()
    for i in range(dims // 2):
        a = position * base ** (-2.0 * i / dims)
        c, s = math.cos(a), math.sin(a)
        out[:, 2 * i] = v[:, 2 * i] * c - v[:, 2 * i + 1] * s
        out[:, 2 * i + 1] = v[:, 2 * i + 1] * c + v[:, 2 * i] * s
    return out


def sink_softmax(s):
    """exp(s_j) / (1 + sum_j exp(s_j)): a sink of score 0 that carries no value."""
    m = max(float(s.max()), 0.0)
    e = torch.exp(s - m)
    return e / (math.exp(-m) + e.sum())


def attention_mixer(h, p, m, eps, positions, state):
    """Causal softmax attention with grouped key/value heads.  h [n, W]; p = the layer's 'mix.*' tensors; m = its 'mixer'
    config; state = dict(k [P, G, dim] normed rotated keys, v [P, G, dim] values, q_in / k_in [taps-1, .] the conv inputs) of
    the earlier positions, extended in place."""
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    n = h.shape[0]
    q, state["q_in"] = short_conv(h @ p["q"].T, p["q.conv"], state["q_in"])
    k, state["k_in"] = short_conv(h @ p["k"].T, p["k.conv"], state["k_in"])
    q, k = q.reshape(n, H, D), k.reshape(n, G, D)
    v = k.clone()                                                   # the values: the keys as the convolution left them
    rot = m["rot"]
    qn = torch.stack([unit_rms(rotate_pairs(q[t], positions[t], rot["dims"], rot["base"]), eps) for t in range(n)])
    kn = torch.stack([unit_rms(rotate_pairs(k[t], positions[t], rot["dims"], rot["base"]), eps) for t in range(n)])
    first = state["k"].shape[0]
    state["k"] = torch.cat([state["k"], kn], 0)
    state["v"] = torch.cat([state["v"], v], 0)
    y = torch.zeros(n, H, D, dtype=h.dtype)
    for t in range(n):
        seen = first + t + 1
        for g in range(H):
            kv = g // (H // G)
            w = sink_softmax((state["k"][:seen, kv] @ qn[t, g]) * m["scale"])
            y[t, g] = w @ state["v"][:seen, kv]
    return y.reshape(n, H * D) @ p["o"].T


def new_attention_state(m, dt=torch.float64):
    H, G, D, taps = m["heads"], m["kv_heads"], m["dim"], m["conv"]
    return dict(k=torch.zeros(0, G, D, dtype=dt), v=torch.zeros(0, G, D, dtype=dt),
                q_in=torch.zeros(taps - 1, H * D, dtype=dt), k_in=torch.zeros(taps - 1, G * D, dtype=dt))


def ssm_mixer(h, p, m, eps, state):
    """Selective state-space mixer.  h [n, W]; state = dict(S [heads, N, P] , u_in [taps-1, channels])."""
    Hd, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hd * P
    n = h.shape[0]
    proj = h @ p["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc, state["u_in"] = short_conv(xbc, p["conv"], state["u_in"], p["conv.b"])
    xbc = silu(xbc)
    x = xbc[:, :inner].reshape(n, Hd, P)
    B = xbc[:, inner:inner + G * N].reshape(n, G, N)
    Cm = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + p["dt_bias"])
    y = torch.zeros(n, Hd, P, dtype=h.dtype)
    for t in range(n):
        for g in range(Hd):
            grp = g // (Hd // G)
            a = math.exp(-math.exp(float(p["A_log"][g])) * float(dt[t, g]))
            state["S"][g] = a * state["S"][g] + float(dt[t, g]) * torch.outer(B[t, grp], x[t, g])
            y[t, g] = state["S"][g].T @ Cm[t, grp] + p["D"][g] * x[t, g]
    y = y.reshape(n, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.reshape(n, parts, inner // parts), eps).reshape(n, inner) * p["norm"]
    return y @ p["o"].T


def new_ssm_state(m, dt=torch.float64):
    inner = m["heads"] * m["vdim"]
    return dict(S=torch.zeros(m["heads"], m["state"], m["vdim"], dtype=dt),
                u_in=torch.zeros(m["conv"] - 1, inner + 2 * m["groups"] * m["state"], dtype=dt))


def routed_ff(h, p, f):
    """Routed experts: scores = sigmoid(router h); the `top` largest are chosen and each chosen expert runs on
    score * h: out = sum_e down_e relu(up_e (s_e h))^2."""
    n = h.shape[0]
    top = f["router"]["top"]
    out = torch.zeros(n, p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(n):
        s = torch.sigmoid(p["router"] @ h[t])
        order = sorted(range(s.shape[0]), key=lambda e: (-float(s[e]), e))[:top]
        for e in order:
            a = torch.relu(p[f"e{e}.up"] @ (s[e] * h[t]))
            out[t] = out[t] + p[f"e{e}.down"] @ (a * a)
    return out


def layer_runs(cfg):
    """[(layer index, pass index or None)] in execution order."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["start"] == loop["stop"]:
        return [(i, None) for i in range(L)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return [(i, None) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)] + [(i, None) for i in range(b, L)]


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


class Decoder:
    """A Lifuzen decoder over one sequence: forward(tokens) continues from what earlier calls left."""

    def __init__(self, cfg, tensors, dt=torch.float64):
        self.cfg, self.dt = cfg, dt
        self.w = {k: v.to(dt) for k, v in tensors.items()}
        self.runs = layer_runs(cfg)
        self.state = []
        for i, _ in self.runs:
            e = cfg["layers"][i]
            self.state.append(new_attention_state(e["mixer"], dt) if e["type"] == "attention" else new_ssm_state(e["mixer"], dt))
        self.pos = 0

    def forward(self, tokens, trace=None):
        """-> logits [n, vocab]; trace (a list) receives the stream after every run."""
        cfg, w = self.cfg, self.w
        eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
        n = len(tokens)
        positions = list(range(self.pos, self.pos + n))
        self.pos += n
        e0 = w["embed"][torch.tensor(tokens, dtype=torch.long)]
        x = e0.clone()
        loop = cfg.get("loop")
        for r, (i, t) in enumerate(self.runs):
            if t is not None and i == loop["start"]:
                if t > 0:
                    x = x + e0
                x = x + w["loop.step"][t]
            entry = cfg["layers"][i]
            p = f"l{i}."
            h1 = offset_norm(x, w[p + "norm1"], eps)
            if entry["type"] == "attention":
                y = attention_mixer(h1, sub(w, p + "mix."), entry["mixer"], eps, positions, self.state[r])
            else:
                y = ssm_mixer(h1, sub(w, p + "mix."), entry["mixer"], eps, self.state[r])
            if entry.get("mlp") is not None:
                y = y + routed_ff(offset_norm(x, w[p + "norm2"], eps), sub(w, p + "mlp."), entry["mlp"])
            x = x + mult * y
            if trace is not None:
                trace.append(x.clone())
        logits = offset_norm(x, w["final.norm"], eps) @ w["embed"].T
        cap = cfg.get("logit_softcap")
        if cap:
            logits = cap * torch.tanh(logits / cap)
        return logits
