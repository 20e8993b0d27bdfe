"""A numpy stand-in for libb200hybrid.so that works on host memory -- TEST INFRASTRUCTURE ONLY.

It has the entry points of include/b200_hybrid.h with the same argument lists and addresses rows, pages and state slots the
way the header says, in float32 only (dtype B200H_F32), with the arithmetic written row by row in numpy.  With it the host
side of a hybrid decoder (turbomind/hybrid.py, the engine, the scheduler's blocks and slots, bin/trace_run) runs without a
GPU: a wrong page address, slot offset or row mapping shows on the CPU.  The CUDA kernels themselves are compared with
oracle/gulozen.py on a device (tests/test_hybrid_gpu.py)."""
import ctypes as C

import numpy as np

F32 = 2


def _a(ptr, count, ctype=C.c_float):
    if isinstance(ptr, C.c_void_p):
        ptr = ptr.value
    return np.ctypeslib.as_array(C.cast(int(ptr), C.POINTER(ctype)), shape=(int(count),))


def _f(ptr, *shape):
    return _a(ptr, int(np.prod(shape))).reshape(shape)


def _i(ptr, count):
    return _a(ptr, count, C.c_int)


def _rows(ptr, n, ld, cols):
    """[n, cols] view of a float matrix with row stride ld."""
    return np.lib.stride_tricks.as_strided(_a(ptr, (n - 1) * ld + cols), (n, cols), (4 * ld, 4))


def _unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True, dtype=np.float32) + np.float32(eps))


def _sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


class EmulatedHybridLib:
    def b200h_last_error(self):
        return b""

    def b200h_embed(self, tokens, table, scale, out, n, width, dtype, stream):
        assert dtype == F32
        tok = _i(tokens, n)
        tab = _a(table, (int(tok.max()) + 1) * width).reshape(-1, width)
        _f(out, n, width)[:] = tab[tok] * np.float32(scale)
        return 0

    def b200h_causal_conv(self, x, w, state, slot_stride, tok_seq, cu_q, seq_slot, out, n, batch, width, taps, dtype, stream):
        X, Wt, O = _f(x, n, width), _f(w, width, taps), _f(out, n, width)
        cu, slots = _i(cu_q, batch + 1), _i(seq_slot, batch)
        for s in range(batch):
            lo, hi = cu[s], cu[s + 1]
            if lo == hi:
                continue
            st = _f(int(state) + 4 * int(slots[s]) * slot_stride, taps - 1, width)
            full = np.concatenate([st, X[lo:hi]], 0)
            for t in range(hi - lo):
                acc = X[lo + t].copy()
                for j in range(taps):
                    acc += Wt[:, j] * full[t + j]
                O[lo + t] = acc
            st[:] = full[full.shape[0] - (taps - 1):]
        return 0

    def b200h_residual_group_norm(self, x, m, m_is_f32, parts, w, n, width, groups, eps, x_t, dtype, stream):
        X, M, Wn = _f(x, n, width), _f(m, n, parts, width), _f(w, width)
        v = M[:, 0].copy()
        for p in range(1, parts):
            v += M[:, p]
        y = _unit(v.reshape(n, groups, width // groups), eps).reshape(n, width) * Wn
        X += y
        if x_t:
            _f(x_t, n, width)[:] = X
        return 0

    def b200h_group_norm_rows(self, x, rows, w, count, width, groups, eps, out, dtype, stream):
        idx = _i(rows, count) if rows else np.arange(count)
        X = _f(x, int(idx.max()) + 1, width)[idx]
        _f(out, count, width)[:] = _unit(X.reshape(count, groups, width // groups), eps).reshape(count, width) * _f(w, width)
        return 0

    def b200h_depth_mix(self, x, hist, hist_stride, coef, terms, count, stream):
        X, c = _a(x, count), _a(coef, terms)
        Hs = [_a(int(hist) + 4 * j * hist_stride, count) for j in range(terms)]
        Hs[terms - 1][:] = X
        acc = np.zeros(count, np.float32)
        for j in range(terms):
            acc += c[j] * Hs[j]
        X[:] = acc
        return 0

    @staticmethod
    def _rot(v, pos, a):
        if a.rot.pairs == 0:
            return v.copy()
        f = _a(a.rot.freqs, a.rot.pairs, C.c_double)
        ang = float(pos) * f
        c, s = (np.cos(ang) * a.rot.magnitude).astype(np.float32), (np.sin(ang) * a.rot.magnitude).astype(np.float32)
        out = v.copy()
        u, w = v[..., 0:2 * a.rot.pairs:2], v[..., 1:2 * a.rot.pairs:2]
        out[..., 0:2 * a.rot.pairs:2] = u * c - w * s
        out[..., 1:2 * a.rot.pairs:2] = w * c + u * s
        return out

    @staticmethod
    def _page(a, seq, pos):
        cu = _i(a.cu_blocks, seq + 2)
        ptrs = _a(a.block_ptrs, cu[seq + 1], C.c_int64)
        base = int(ptrs[cu[seq] + pos // a.block_len]) + a.layer_off
        at = pos % a.block_len
        return _f(base + 4 * at * a.kv_rank, a.kv_rank), _f(base + a.rot_off + 4 * at * a.rot_dim, a.rot_dim)

    def b200h_latent_prep(self, args):
        a = args._obj
        assert a.dtype == F32
        dq, dkv = _rows(a.dq, a.n, a.ld_dq, a.q_rank), _rows(a.dkv, a.n, a.ld_dkv, a.kv_rank + a.rot_dim)
        _f(a.cq, a.n, a.q_rank)[:] = _unit(dq, a.eps) * _f(a.q_norm, a.q_rank)
        seqs, poss = _i(a.tok_seq, a.n), _i(a.tok_pos, a.n)
        for t in range(a.n):
            c, kr = self._page(a, int(seqs[t]), int(poss[t]))
            c[:] = _unit(dkv[t, :a.kv_rank], a.eps) * _f(a.kv_norm, a.kv_rank)
            kr[:] = self._rot(dkv[t, a.kv_rank:], poss[t], a)
        return 0

    def b200h_rotate_query(self, args):
        a = args._obj
        H, D, R = a.heads, a.dim, a.rot_dim
        q = _rows(a.q, a.n, a.ld_q, H * (D + R)).reshape(a.n, H, D + R)
        out, poss = _f(a.q_rot, a.n, H, R), _i(a.tok_pos, a.n)
        for t in range(a.n):
            out[t] = self._rot(q[t, :, D:], int(poss[t]), a)
        return 0

    def b200h_latent_attention(self, args):
        a = args._obj
        H, R, Ck = a.heads, a.rot_dim, a.kv_rank
        q_lat, q_rot, sink = _f(a.q_lat, a.n, H, Ck), _f(a.q_rot, a.n, H, R), _f(a.sink, H)
        out = _f(a.o_heads, H, a.n, Ck)
        seqs, poss = _i(a.tok_seq, a.n), _i(a.tok_pos, a.n)
        for t in range(a.n):
            s, pos = int(seqs[t]), int(poss[t])
            cs, krs = zip(*[self._page(a, s, j) for j in range(pos + 1)])
            cs, krs = np.stack(cs), np.stack(krs)
            for h in range(H):
                sc = (cs @ q_lat[t, h] + krs @ q_rot[t, h]) * np.float32(a.scale)
                top = max(float(sc.max()), float(sink[h]))
                e = np.exp(sc - top)
                out[h, t] = (e / (e.sum() + np.exp(sink[h] - top))) @ cs
        return 0

    def b200h_head_gate(self, o, gate, ld_gate, n, heads, vdim, y, dtype, stream):
        O = _f(o, heads, n, vdim).transpose(1, 0, 2).reshape(n, heads * vdim)
        _f(y, n, heads * vdim)[:] = O * _sigmoid(_rows(gate, n, ld_gate, heads * vdim))
        return 0

    def b200h_decay_attention(self, q, k, v, ld, decay, state, slot_stride, cu_q, seq_slot, batch, heads, dim, vdim, out, dtype, stream):
        cu, slots, lam = _i(cu_q, batch + 1), _i(seq_slot, batch), _a(decay, heads)
        n = int(cu[batch])
        silu = lambda z: z * _sigmoid(z)
        Q, K = silu(_rows(q, n, ld, heads * dim)).reshape(n, heads, dim), silu(_rows(k, n, ld, heads * dim)).reshape(n, heads, dim)
        Vv = silu(_rows(v, n, ld, heads * vdim)).reshape(n, heads, vdim)
        O = _f(out, n, heads, vdim)
        for s in range(batch):
            S = _f(int(state) + 4 * int(slots[s]) * slot_stride, heads, vdim, dim)
            for t in range(cu[s], cu[s + 1]):
                for h in range(heads):
                    S[h] = lam[h] * S[h] + np.outer(Vv[t, h], K[t, h])
                    O[t, h] = S[h] @ Q[t, h]
        return 0

    def b200h_gated_rms(self, o, w, gate, ld_gate, n, count, eps, y, dtype, stream):
        _f(y, n, count)[:] = _unit(_f(o, n, count), eps) * _f(w, count) * _sigmoid(_rows(gate, n, ld_gate, count))
        return 0

    def b200h_route(self, x, router, n, width, experts, top, ids, wts, stream):
        return self.b200h_route_scored(x, F32, router, n, width, experts, top, 0, ids, wts, stream)

    def b200h_route_scored(self, x, x_dtype, router, n, width, experts, top, score_fn, ids, wts, stream):
        assert x_dtype == F32
        z = _f(x, n, width) @ _f(router, experts, width).T
        if score_fn == 1:
            order = np.argsort(-z, -1, kind="stable")[:, :top]          # chosen on the logits: the sigmoid keeps their order
            _i(ids, n * top).reshape(n, top)[:] = order
            _f(wts, n, top)[:] = _sigmoid(np.take_along_axis(z, order, -1))
            return 0
        else:
            e = np.exp(z - z.max(-1, keepdims=True))
            sc = e / e.sum(-1, keepdims=True)
        order = np.argsort(-sc, -1, kind="stable")[:, :top]
        _i(ids, n * top).reshape(n, top)[:] = order
        _f(wts, n, top)[:] = np.take_along_axis(sc, order, -1)
        return 0

    def b200h_experts(self, args):
        a = args._obj
        n, top, width, ff, E = a.n, a.top, a.width, a.ff, a.experts
        X, idx, wt = _f(a.x, n, width), _i(a.ids, n * top).reshape(n, top), _f(a.wts, n, top)
        U, Dn = _f(a.up, E, ff, width), _f(a.down, E, width, ff)
        G = _f(a.gate, E, ff, width) if a.act == 0 else None
        O = _f(a.out, n, top, width)
        for t in range(n):
            for k in range(top):
                e = idx[t, k]
                xin = X[t] * wt[t, k] if a.scale_input else X[t]
                if a.act == 0:
                    g = G[e] @ xin
                    mid = g * _sigmoid(g) * (U[e] @ xin)
                else:
                    mid = np.maximum(U[e] @ xin, 0) ** 2
                O[t, k] = (Dn[e] @ mid) * (np.float32(1) if a.scale_input else wt[t, k])
        return 0

    def b200h_silu_mul(self, g, u, out, count, dtype, stream):
        G_, U_ = _a(g, count).copy(), _a(u, count).copy()
        _a(out, count)[:] = G_ * _sigmoid(G_) * U_
        return 0

    def b200h_weighted_scatter(self, src, slot, wts, out, rows, width, dtype, stream):
        S_, to = _f(src, rows, width), _i(slot, rows)
        wt = _a(wts, rows) if wts else np.ones(rows, np.float32)
        _f(out, rows, width)[to] = wt[to][:, None] * S_
        return 0

    # ---- pre-norm blocks
    def b200h_add_rows(self, x, table, idx, fixed, n, width, dtype, stream):
        assert dtype == F32
        X = _f(x, n, width)
        which = _i(idx, n) if idx else np.full(n, fixed)
        tab = _f(table, int(which.max()) + 1, width)
        X += tab[which]
        return 0

    def b200h_residual_norm(self, x, m, extra, w, n, width, eps, h, dtype, stream):
        X = _f(x, n, width)
        if m:
            X += _f(m, n, width)
        if extra:
            X += _f(extra, width)
        if h:
            _f(h, n, width)[:] = _unit(X, eps) * _f(w, width)
        return 0

    def b200h_relu2(self, x, count, dtype, stream):
        X = _a(x, count)
        X[:] = np.maximum(X, 0) ** 2
        return 0

    @staticmethod
    def _kv(a, seq, pos):
        """The cache entry of (seq, pos): key [kv_heads, dim] and value [kv_heads, vdim] views."""
        cu = _i(a.cu_blocks, seq + 2)
        ptrs = _a(a.block_ptrs, cu[seq + 1], C.c_int64)
        base = int(ptrs[cu[seq] + pos // a.block_len]) + a.layer_off
        at = pos % a.block_len
        G, D, V = a.kv_heads, a.dim, a.vdim
        return _f(base + 4 * at * G * D, G, D), _f(base + a.v_off + 4 * at * G * V, G, V)

    def b200h_window_prep(self, args):
        a = args._obj
        assert a.dtype == F32
        H, G, D, V = a.heads, a.kv_heads, a.dim, a.vdim
        q, k, v = _rows(a.q, a.n, a.ld, H * D), _rows(a.k, a.n, a.ld, G * D), _rows(a.v, a.n, a.ld, G * V)
        if a.bias:
            b = _f(a.bias, (H + G) * D + G * V)
            q, k, v = q + b[:H * D], k + b[H * D:(H + G) * D], v + b[(H + G) * D:]
        _f(a.qn, a.n, H * D)[:] = _unit(q, a.eps) * _f(a.q_norm, H * D) if a.q_norm else q
        kn = _unit(k, a.eps) * _f(a.k_norm, G * D) if a.k_norm else k
        seqs, poss = _i(a.tok_seq, a.n), _i(a.tok_pos, a.n)
        for t in range(a.n):
            kd, vd = self._kv(a, int(seqs[t]), int(poss[t]))
            kd[:] = kn[t].reshape(G, D)
            vd[:] = v[t].reshape(G, V)
        return 0

    def b200h_window_attention(self, args):
        a = args._obj
        H, G, D, V = a.heads, a.kv_heads, a.dim, a.vdim
        rep = H // G
        qn = _f(a.qn, a.n, H, D)
        y = _f(a.y, a.n, H * V)
        gate = _rows(a.gate, a.n, a.ld_gate, H if a.gate_heads else H * V) if a.gate else None
        seqs, poss = _i(a.tok_seq, a.n), _i(a.tok_pos, a.n)
        for t in range(a.n):
            s, pos = int(seqs[t]), int(poss[t])
            lo = max(0, pos - a.window + 1) if a.window > 0 else 0
            if a.chunk > 0:
                lo = max(lo, pos // a.chunk * a.chunk)
            ks, vs = zip(*[self._kv(a, s, j) for j in range(lo, pos + 1)])
            ks, vs = np.stack(ks), np.stack(vs)                                    # [L, G, D], [L, G, V]
            dist = (pos - np.arange(lo, pos + 1)).astype(np.float32)
            wts = np.zeros((H, len(dist)), np.float32)
            raw = np.zeros((H, len(dist)), np.float32)
            for h in range(H):
                sc = (ks[:, h // rep] @ qn[t, h]) * np.float32(a.scale)
                if a.softcap > 0:
                    sc = a.softcap * np.tanh(sc / a.softcap)
                if a.r1:
                    sc = sc - _f(a.r1, H)[h] * np.log1p(_f(a.r2, H)[h] * dist)
                raw[h] = sc
            if a.talk and a.talk_scores:
                raw = _f(a.talk, H, H) @ raw
            for h in range(H):
                sc = raw[h]
                if a.sink:
                    mx = max(float(sc.max()), float(_f(a.sink, H)[h]))
                    e = np.exp(sc - mx)
                    wts[h] = e / (e.sum() + np.exp(_f(a.sink, H)[h] - mx))
                else:
                    e = np.exp(sc - sc.max())
                    wts[h] = e / e.sum()
            if a.talk and not a.talk_scores:
                wts = _f(a.talk, H, H) @ wts
            out = np.stack([wts[h] @ vs[:, h // rep] for h in range(H)])
            if gate is not None:
                out = out * (_sigmoid(gate[t])[:, None] if a.gate_heads else _sigmoid(gate[t]).reshape(H, V))
            y[t] = out.reshape(H * V)
        return 0

    def b200h_head_rope_prep(self, args, rot):
        a, r = args._obj, rot._obj
        assert a.dtype == F32
        H, G, D, V = a.heads, a.kv_heads, a.dim, a.vdim
        q, k, v = _rows(a.q, a.n, a.ld, H * D), _rows(a.k, a.n, a.ld, G * D), _rows(a.v, a.n, a.ld, G * V)
        if a.bias:
            b = _f(a.bias, (H + G) * D + G * V)
            q, k, v = q + b[:H * D], k + b[H * D:(H + G) * D], v + b[(H + G) * D:]
        q, k = q.reshape(a.n, H, D), k.reshape(a.n, G, D)
        if a.q_norm:
            q = _unit(q, a.eps) * _f(a.q_norm, D)
        if a.k_norm:
            k = _unit(k, a.eps) * _f(a.k_norm, D)

        class WithRot:
            pass
        holder = WithRot()
        holder.rot = r
        seqs, poss = _i(a.tok_seq, a.n), _i(a.tok_pos, a.n)
        qn = _f(a.qn, a.n, H, D)
        for t in range(a.n):
            qn[t] = self._rot(q[t], int(poss[t]), holder)
            kd, vd = self._kv(a, int(seqs[t]), int(poss[t]))
            kd[:] = self._rot(k[t], int(poss[t]), holder)
            vd[:] = v[t].reshape(G, V)
        return 0

    # ---- shared-norm blocks: hashed bigram embedding, side norms + residual, token shift, channel-decay recurrence
    def b200h_embed_hashed(self, tokens, table, second, buckets, mul_prev, mul_cur, prev, slot_stride, tok_seq, tok_pos, cu_q, seq_slot, out,
                           n, batch, width, dtype, stream):
        assert dtype == F32
        tok, seqs, poss = _i(tokens, n), _i(tok_seq, n), _i(tok_pos, n)
        cu, slots = _i(cu_q, batch + 1), _i(seq_slot, batch)
        tab = _a(table, (int(tok.max()) + 1) * width).reshape(-1, width)
        sec = _f(second, buckets + 1, width)
        O = _f(out, n, width)
        for t in range(n):
            s = int(seqs[t])
            row = buckets
            if poss[t] > 0:
                before = int(tok[t - 1]) if t > cu[s] else int(_i(int(prev) + 4 * int(slots[s]) * slot_stride, 1)[0])
                row = (before * mul_prev + int(tok[t]) * mul_cur) % buckets
            O[t] = tab[tok[t]] + sec[row]
        for s in range(batch):
            if cu[s] < cu[s + 1]:
                _i(int(prev) + 4 * int(slots[s]) * slot_stride, 1)[0] = tok[cu[s + 1] - 1]
        return 0

    def b200h_branch_residual_norm(self, x, left, right, wl, wr, branch_scale, ff, ff_is_f32, parts, w, n, width, eps, h, hf, dtype, stream):
        X = _f(x, n, width)
        if left:
            X += np.float32(branch_scale) * (_unit(_f(left, n, width), eps) * _f(wl, width) + _unit(_f(right, n, width), eps) * _f(wr, width))
        if ff:
            F = _f(ff, n, parts, width)
            for p in range(parts):
                X += F[:, p]
        if w:
            v = _unit(X, eps) * _f(w, width)
            if h:
                _f(h, n, width)[:] = v
            if hf:
                _f(hf, n, width)[:] = v
        return 0

    def b200h_token_shift(self, h, shift, mu, nmu, state, slot_stride, tok_seq, cu_q, seq_slot, n, batch, width, a, blends, dtype, stream):
        Hm = _f(h, n, width)
        sh = _f(shift, width) if shift else np.zeros(width, np.float32)
        M = _f(mu, nmu, width) if nmu else None
        cu, slots = _i(cu_q, batch + 1), _i(seq_slot, batch)
        A = _f(a, n, width) if a else None
        B = _f(blends, nmu, n, width) if nmu else None
        for s in range(batch):
            lo, hi = cu[s], cu[s + 1]
            if lo == hi:
                continue
            st = _f(int(state) + 4 * int(slots[s]) * slot_stride, 2, width)
            hp, ap = st[0].copy(), st[1].copy()
            for t in range(lo, hi):
                cur = Hm[t] + (hp - Hm[t]) * sh
                if A is not None:
                    A[t] = cur
                for m in range(nmu):
                    B[m, t] = cur + (ap - cur) * M[m]
                hp, ap = Hm[t].copy(), cur
            st[0], st[1] = hp, ap
        return 0

    def b200h_channel_decay_scan(self, r, k, v, ld, d, w0, bonus, state, slot_stride, cu_q, seq_slot, n, batch, heads, dim, vdim, decay, out,
                                 dtype, stream):
        R, K, Vv = _rows(r, n, ld, heads * dim), _rows(k, n, ld, heads * dim), _rows(v, n, ld, heads * vdim)
        Wd = np.exp(-np.exp(_f(d, n, heads * dim) + _f(w0, heads * dim)))
        U = _f(bonus, heads, dim)
        O = _f(out, n, heads, vdim)
        cu, slots = _i(cu_q, batch + 1), _i(seq_slot, batch)
        for s in range(batch):
            S = _f(int(state) + 4 * int(slots[s]) * slot_stride, heads, vdim, dim)            # [head][value][key]
            for t in range(cu[s], cu[s + 1]):
                for hh in range(heads):
                    kk, rr = K[t, hh * dim:(hh + 1) * dim], R[t, hh * dim:(hh + 1) * dim]
                    kv = np.outer(Vv[t, hh * vdim:(hh + 1) * vdim], kk)
                    O[t, hh] = (S[hh] + kv * U[hh]) @ rr
                    S[hh] = S[hh] * Wd[t, hh * dim:(hh + 1) * dim] + kv
        return 0

    def b200h_group_norm_gate(self, o, w, gate, ld_gate, n, count, groups, act, eps, y, dtype, stream):
        G = _rows(gate, n, ld_gate, count)
        g = G * _sigmoid(G) if act == 1 else _sigmoid(G)
        _f(y, n, count)[:] = _unit(_f(o, n, groups, count // groups), eps).reshape(n, count) * _f(w, count) * g
        return 0

    def b200h_xielu(self, x, count, params, dtype, stream):
        X, pr = _a(x, count), _a(params, 2)
        sp = lambda z: np.log1p(np.exp(-abs(z))) + max(z, 0.0)
        pos, neg = np.float32(sp(float(pr[0]))), np.float32(0.5 + sp(float(pr[1])))
        z = X.copy()
        X[:] = np.where(z > 0, pos * z * z + 0.5 * z, neg * (np.expm1(np.minimum(z, 0)) - z) + 0.5 * z)
        return 0

    def b200h_tanh(self, x, count, dtype, stream):
        X = _a(x, count)
        X[:] = np.tanh(X)
        return 0

    def b200h_route_grouped(self, x, x_dtype, router, correction, n, width, experts, top, groups, keep, group_top, renorm, scale, ids, wts,
                            stream):
        assert x_dtype == F32
        sc = _sigmoid(_f(x, n, width) @ _f(router, experts, width).T)
        ch = sc + _f(correction, experts) if correction else sc.copy()
        per = experts // groups
        if groups > 1 and keep < groups:
            gs = -np.sort(-ch.reshape(n, groups, per), -1)[:, :, :group_top].sum(-1)
            kept = np.argsort(-gs, -1, kind="stable")[:, :keep]
            mask = np.zeros((n, groups), bool)
            np.put_along_axis(mask, kept, True, -1)
            ch = np.where(np.repeat(mask, per, -1), ch, -np.inf)
        order = np.argsort(-ch, -1, kind="stable")[:, :top]
        chosen = np.take_along_axis(sc, order, -1)
        if renorm:
            chosen = chosen / (chosen.sum(-1, keepdims=True) + np.float32(1e-20))
        _i(ids, n * top).reshape(n, top)[:] = order
        _f(wts, n, top)[:] = chosen * np.float32(scale)
        return 0

    # ---- parallel blocks, convolved rotary attention, state-space mixer
    def b200h_parallel_residual_norm(self, x, mix, ff, parts, mult, add, extra, w1, w2, n, width, eps, h1, h2, h2f, dtype, stream):
        X = _f(x, n, width)
        if mix or ff:
            y = _f(mix, n, width).copy() if mix else np.zeros((n, width), np.float32)
            if ff:
                y += _f(ff, n, parts, width).sum(1)
            X += np.float32(mult) * y
        if add:
            X += _f(add, n, width)
        if extra:
            X += _f(extra, width)
        for h, w in ((h1, w1), (h2, w2), (h2f, w2)):
            if h:
                _f(h, n, width)[:] = _unit(X, eps) * _f(w, width)
        return 0

    @staticmethod
    def _conv_rows(U, Wt, bias, state, slot_stride, cu, slots, batch, taps):
        """Causal taps over every entry's rows with its state in front; advances the state.  -> [n, channels]."""
        n, ch = U.shape
        out = np.zeros((n, ch), np.float32)
        for s in range(batch):
            lo, hi = cu[s], cu[s + 1]
            if lo == hi:
                continue
            st = _f(int(state) + 4 * int(slots[s]) * slot_stride, taps - 1, ch)
            full = np.concatenate([st, U[lo:hi]], 0)
            for t in range(hi - lo):
                acc = np.zeros(ch, np.float32) if bias is None else bias.copy()
                for j in range(taps):
                    acc += Wt[:, j] * full[t + j]
                out[lo + t] = acc
            st[:] = full[full.shape[0] - (taps - 1):]
        return out

    def b200h_short_conv(self, u, ld, w, bias, act, state, slot_stride, tok_seq, cu_q, seq_slot, out, n, batch, channels, taps, dtype, stream):
        assert dtype == F32
        y = self._conv_rows(_rows(u, n, ld, channels), _f(w, channels, taps), _f(bias, channels) if bias else None, state, slot_stride,
                            _i(cu_q, batch + 1), _i(seq_slot, batch), batch, taps)
        _f(out, n, channels)[:] = y * _sigmoid(y) if act == 1 else y
        return 0

    def b200h_ssm_scan(self, xbc, dt, ld_dt, dt_bias, a_log, skip, state, slot_stride, cu_q, seq_slot, n, batch, heads, vdim, nstate,
                       groups, steps, out, dtype, stream):
        cu, slots = _i(cu_q, batch + 1), _i(seq_slot, batch)
        assert n == int(cu[batch]) and steps
        inner, gn = heads * vdim, groups * nstate
        X = _f(xbc, n, inner + 2 * gn)
        DT = _rows(dt, n, ld_dt, heads) + _f(dt_bias, heads)
        DT = (np.maximum(DT, 0) + np.log1p(np.exp(-np.abs(DT)))).astype(np.float32)
        rate, D, O = np.exp(_f(a_log, heads)), _f(skip, heads), _f(out, n, heads, vdim)
        for s in range(batch):
            S = _f(int(state) + 4 * int(slots[s]) * slot_stride, heads, vdim, nstate)
            for t in range(cu[s], cu[s + 1]):
                for h in range(heads):
                    g = h // (heads // groups)
                    xv = X[t, h * vdim:(h + 1) * vdim]
                    B, Cm = X[t, inner + g * nstate:inner + (g + 1) * nstate], X[t, inner + gn + g * nstate:inner + gn + (g + 1) * nstate]
                    S[h] = np.exp(-rate[h] * DT[t, h]) * S[h] + DT[t, h] * np.outer(xv, B)
                    O[t, h] = S[h] @ Cm + D[h] * xv
        return 0

    def b200h_gate_group_norm(self, y, gate, ld_gate, w, n, count, groups, eps, out, dtype, stream):
        z = _rows(gate, n, ld_gate, count)
        v = _f(y, n, count) * (z * _sigmoid(z))
        _f(out, n, count)[:] = _unit(v.reshape(n, groups, count // groups), eps).reshape(n, count) * _f(w, count)
        return 0

    def b200h_conv_rope_prep(self, args):
        a = args._obj
        assert a.dtype == F32
        H, G, D = a.heads, a.kv_heads, a.dim
        ch = (H + G) * D
        y = self._conv_rows(_rows(a.qk, a.n, a.ld, ch), _f(a.conv, ch, a.taps), None, a.state, a.slot_stride, _i(a.cu_q, a.batch + 1),
                            _i(a.seq_slot, a.batch), a.batch, a.taps)
        seqs, poss = _i(a.tok_seq, a.n), _i(a.tok_pos, a.n)
        qn = _f(a.qn, a.n, H, D)

        class _Geo:          # what _kv reads
            cu_blocks, block_ptrs, block_len, layer_off, v_off, kv_heads, dim, vdim = a.cu_blocks, a.block_ptrs, a.block_len, a.layer_off, a.v_off, G, D, D
        for t in range(a.n):
            heads = y[t].reshape(H + G, D)
            kd, vd = self._kv(_Geo, int(seqs[t]), int(poss[t]))
            vd[:] = heads[H:]
            turned = _unit(self._rot(heads, int(poss[t]), a), a.eps)
            qn[t] = turned[:H]
            kd[:] = turned[H:]
        return 0

    def b200h_softcap(self, x, count, cap, stream):
        X = _a(x, count)
        X[:] = np.float32(cap) * np.tanh(X / np.float32(cap))
        return 0

    def b200h_scaled_relu2(self, u, scale, rows, cols, dtype, stream):
        U = _f(u, rows, cols)
        sc = _a(scale, rows)[:, None] if scale else np.float32(1)
        U[:] = np.maximum(U * sc, 0) ** 2
        return 0

    def b200h_argmax(self, logits, ld, rows, vocab, out, stream):
        _i(out, rows)[:] = _rows(logits, rows, ld, vocab).argmax(-1)
        return 0
