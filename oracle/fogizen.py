"""Plain, slow restatement of the Fogizen layer equations in torch on the CPU -- TEST INFRASTRUCTURE ONLY.

One function per mechanism, written token by token (explicit loops over positions, heads and experts; no paging, no
batching, no key ranges, no stacked projections): the opposite route from the product kernels in
lmdeploy_b200/csrc/hybrid, with which it shares no code.  `dt` is the dtype everything runs in (float64 by default).

Notation: n tokens of one sequence, W model width; weights are stored [out, in] and applied as x @ W.T.

A Fogizen layer is a PARALLEL block with ONE norm: h = rms(x) * w1, x <- x + mixer(shift(h)) + ff(h).
  shift:  what the mixer reads is h_t + (h_(t-1) - h_t) * s (element by element; h_(-1) = 0); the feed-forward reads h_t itself.
  mixer:  two mixers side by side on the same input a_t; the result is (rms(left(a)) * w_l + rms(right(a)) * w_r) / 2.
    left  -- softmax attention with grouped key/value heads: biased projections, an RMS norm per head over `dim` whose weight all
             heads share, interleaved rotation of the first rot.dims dimensions with every frequency divided by a factor, scores
             mixed ACROSS heads before the softmax (s'_h = sum_g T[h, g] s_g), keys of the query's own chunk of `mask.size`
             positions only, a learned per-head sink in the denominator, one sigmoid gate per head.
    right -- a linear recurrence with a decay per head, key channel and token computed from the input (low-rank, doubly
             exponential), a bonus for the current token, a unit norm per head and a silu gate; each of its five projections reads
             its own blend of a_t and a_(t-1).
  ff:     dense  down(act(up h)) with a two-parameter quadratic / exponential activation, or routed experts
          (sigmoid scores, a correction added for the CHOICE only, groups of neighbours of which the best few stay eligible,
          weights renormalised over the chosen and scaled).
The embedding adds a hashed row of a second table that depends on the previous token."""
import math

import torch


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0.0)


def embed(tokens, previous, w, cfg):
    """tokens: the ids of this call; previous: the id before the first of them (None at a sequence's start)."""
    b = (cfg.get("embedding") or {}).get("bigram")
    rows = []
    for tok in tokens:
        if b is None:                                   # a model without the second table
            rows.append(w["embed"][tok])
            continue
        row = b["buckets"] if previous is None else (previous * b["mul_prev"] + tok * b["mul_cur"]) % b["buckets"]
        rows.append(w["embed"][tok] + w["bigram"][row])
        previous = tok
    return torch.stack(rows)


def shifted(h, before, s):
    """h [n, W]; before [W] = the row that precedes h (zeros at a sequence's start): h_t + (h_(t-1) - h_t) * s."""
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        prev = before if t == 0 else h[t - 1]
        out[t] = h[t] + (prev - h[t]) * s
    return out


def rotate_pairs(v, position, dims, base, factor):
    """v [heads, dim]: pair (2i, 2i+1), i < dims/2, turns by position * base^(-2i/dims) / factor; the other dimensions stay."""
    out = v.clone()
    for i in range(dims // 2):
        a = position * (base ** (-2.0 * i / dims) / factor)
        c, s = math.cos(a), math.sin(a)
        out[:, 2 * i] = v[:, 2 * i] * c - v[:, 2 * i + 1] * s
        out[:, 2 * i + 1] = v[:, 2 * i + 1] * c + v[:, 2 * i] * s
    return out


def sink_softmax(s, sink):
    """exp(s_j) / (exp(sink) + sum_j exp(s_j)): the sink has no key and no value."""
    m = max(float(s.max()), float(sink))
    e = torch.exp(s - m)
    return e / (math.exp(float(sink) - m) + e.sum())


def new_attention_state(m, dt=torch.float64):
    G = m["kv_heads"]
    return dict(k=torch.zeros(0, G, m["dim"], dtype=dt), v=torch.zeros(0, G, m["vdim"], dtype=dt))


def chunk_attention(a, p, m, eps, positions, state):
    """The left mixer.  a [n, W]; p = the '...mix.left.*' tensors; state: the keys and values of earlier positions."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    size = int((m.get("mask") or {}).get("size") or 0)
    n = a.shape[0]
    out = torch.zeros(n, H * V, dtype=a.dtype)
    for t in range(n):
        pos = positions[t]
        q = (a[t] @ p["q"].T + p["q.b"]).reshape(H, D)
        k = (a[t] @ p["k"].T + p["k.b"]).reshape(G, D)
        v = (a[t] @ p["v"].T + p["v.b"]).reshape(G, V)
        q = rotate_pairs(unit_rms(q, eps) * p["q.norm"], pos, rot["dims"], rot["base"], factor)
        k = rotate_pairs(unit_rms(k, eps) * p["k.norm"], pos, rot["dims"], rot["base"], factor)
        state["k"] = torch.cat([state["k"], k[None]], 0)
        state["v"] = torch.cat([state["v"], v[None]], 0)
        first = pos // size * size if size else 0
        keys = list(range(first, pos + 1))
        raw = torch.zeros(H, len(keys), dtype=a.dtype)
        for h in range(H):
            g = h // (H // G)
            raw[h] = state["k"][first:pos + 1, g] @ q[h] * m["scale"]
        mixed = p["talk"] @ raw                                        # across heads, key by key
        gate = sigmoid(a[t] @ p["g"].T)                                # one number per head
        for h in range(H):
            g = h // (H // G)
            wts = sink_softmax(mixed[h], p["sink"][h])
            out[t, h * V:(h + 1) * V] = (wts @ state["v"][first:pos + 1, g]) * gate[h]
    return out @ p["o"].T


def new_recurrence_state(m, dt=torch.float64):
    return dict(S=torch.zeros(m["heads"], m["dim"], m["dim"], dtype=dt))


def decayed_recurrence(a, before, p, m, eps, state):
    """The right mixer.  a [n, W]; before [W] = the mixer input of the previous token (zeros at a sequence's start);
    state['S'] [heads, key channel, value channel]."""
    H, D = m["heads"], m["dim"]
    n = a.shape[0]
    out = torch.zeros(n, H * D, dtype=a.dtype)
    for t in range(n):
        prev = before if t == 0 else a[t - 1]
        blend = {s: a[t] + (prev - a[t]) * p["mu." + s] for s in "rkvgw"}
        r = (blend["r"] @ p["r"].T).reshape(H, D)
        k = (blend["k"] @ p["k"].T).reshape(H, D)
        v = (blend["v"] @ p["v"].T).reshape(H, D)
        gate = silu(blend["g"] @ p["g"].T)
        w = torch.exp(-torch.exp(torch.tanh(blend["w"] @ p["w1"].T) @ p["w2"].T + p["w0"])).reshape(H, D)
        o = torch.zeros(H, D, dtype=a.dtype)
        for h in range(H):
            S = state["S"][h]
            kv = k[h][:, None] * v[h][None, :]
            o[h] = (S + p["u"][h][:, None] * kv).T @ r[h]
            state["S"][h] = w[h][:, None] * S + kv
        o = unit_rms(o, eps)
        out[t] = o.reshape(-1) * p["norm"] * gate
    return out @ p["o"].T


def two_sided_mixer(a, before, p, m, eps, positions, state):
    """Half the sum of the two mixers' outputs, each RMS-normed over the width with its own weight."""
    left = chunk_attention(a, sub(p, "left."), m["left"], eps, positions, state["left"])
    right = decayed_recurrence(a, before, sub(p, "right."), m["right"], eps, state["right"])
    return 0.5 * (unit_rms(left, eps) * p["left.out"] + unit_rms(right, eps) * p["right.out"])


def xielu(z, params):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    ap, an = softplus(params[0]), 0.5 + softplus(params[1])
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)


def dense_ff(h, p):
    return xielu(h @ p["up"].T, p["act"]) @ p["down"].T


def route(h, p, f):
    """One token: -> [(expert, weight)].  Sigmoid scores; the correction joins them for the choice only; experts in groups of
    neighbours, a group's score the sum of its two largest choice scores, only the best `keep` groups stay eligible."""
    r = f["router"]
    E, top = r["experts"], r["top"]
    s = sigmoid(h @ p["router"].T)
    choice = s + p["correction"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = E // groups["count"]
    score = []
    for g in range(groups["count"]):
        part = sorted((float(c) for c in choice[g * per:(g + 1) * per]), reverse=True)
        score.append(sum(part[:2]))
    kept = sorted(range(groups["count"]), key=lambda g: (-score[g], g))[:groups["keep"]]
    eligible = [e for e in range(E) if e // per in kept]
    chosen = sorted(eligible, key=lambda e: (-float(choice[e]), e))[:top]
    total = sum(s[e] for e in chosen) + 1e-20
    return [(e, s[e] / total * r["scale"]) for e in chosen]


def routed_ff(h, p, f):
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in route(h[t], p, f):
            q = f"e{e}."
            out[t] = out[t] + wt * ((silu(h[t] @ p[q + "gate"].T) * (h[t] @ p[q + "up"].T)) @ p[q + "down"].T)
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


class Decoder:
    """A Fogizen decoder over one sequence: forward(tokens) continues from what earlier calls left."""

    def __init__(self, cfg, tensors, dt=torch.float64):
        self.cfg, self.dt = cfg, dt
        self.w = {k: (v.to(dt) if v.is_floating_point() else v) for k, v in tensors.items()}
        W = cfg["width"]
        self.state = []
        for e in cfg["layers"]:
            if e["type"] != "parallel":
                raise NotImplementedError(e["type"])
            self.state.append(dict(left=new_attention_state(e["mixer"]["left"], dt), right=new_recurrence_state(e["mixer"]["right"], dt),
                                   h=torch.zeros(W, dtype=dt), a=torch.zeros(W, dtype=dt)))
        self.pos = 0
        self.previous = None

    def forward(self, tokens, trace=None):
        """-> logits [n, vocab]; trace (a list) receives the stream after every layer."""
        cfg, w = self.cfg, self.w
        eps = cfg["norm"]["eps"]
        n = len(tokens)
        positions = list(range(self.pos, self.pos + n))
        self.pos += n
        x = embed(tokens, self.previous, w, cfg)
        self.previous = tokens[-1]
        for i, e in enumerate(cfg["layers"]):
            p, st = f"l{i}.", self.state[i]
            h = unit_rms(x, eps) * w[p + "norm1"]
            a = shifted(h, st["h"], w[p + "shift"])
            y = two_sided_mixer(a, st["a"], sub(w, p + "mix."), e["mixer"], eps, positions, st)
            st["h"], st["a"] = h[-1].clone(), a[-1].clone()
            f = e.get("mlp")
            if f is not None:
                y = y + (dense_ff(h, sub(w, p + "mlp.")) if f["kind"] == "dense" else routed_ff(h, sub(w, p + "mlp."), f))
            x = x + y
            if trace is not None:
                trace.append(x.clone())
        return (unit_rms(x, eps) * w["final.norm"]) @ w["head"].T
