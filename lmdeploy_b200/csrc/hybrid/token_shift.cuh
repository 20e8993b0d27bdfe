// Kernels of parallel blocks with ONE norm and a token shift, and of the recurrence with a decay per key channel and token:
// an embedding that adds a hashed row of a second table chosen by the previous token, the join of two side-by-side mixers (each
// RMS-normed over the width, averaged) and the feed-forward into the stream fused with the next norm, the token shift and the
// recurrence's five blends of a row with its predecessor, the recurrence itself, a per-head unit norm with a gate after it, and
// two small activations.
// Included by hybrid_ops.cu inside namespace b200h, after its helpers (to_f / from_f / block_sum / warp_sum / silu_f / sigmoid_f).
//
// State of a sequence (floats of its slot): the id of its last token (an int in a float's place); per run the last row of the
// normed stream h and of the shifted row a (2 * width floats); per run the recurrence's [heads, vdim, dim] matrix.  A fresh slot
// is zeroed, and zeros are what a sequence's first token blends with.

__device__ __forceinline__ float softplus32(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// out[t] = table[tokens[t]] + second[row], row = (previous * mul_prev + tokens[t] * mul_cur) mod buckets, or `buckets` (the last
// row) at position 0.  The token before an entry's first row is the int at prev + seq_slot[s] * slot_stride.
template <typename T>
__global__ void embed_hashed_kernel(const int* __restrict__ tokens, const T* __restrict__ table, const T* __restrict__ second, int buckets,
                                    int mul_prev, int mul_cur, const float* __restrict__ prev, int64_t slot_stride,
                                    const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ cu_q,
                                    const int* __restrict__ seq_slot, float* __restrict__ out, int width)
{
    const int t = blockIdx.x, s = tok_seq[t], tok = tokens[t];
    int64_t row = buckets;
    if (tok_pos[t] > 0) {
        const int before = t > cu_q[s] ? tokens[t - 1] : *reinterpret_cast<const int*>(prev + (int64_t)seq_slot[s] * slot_stride);
        row = ((int64_t)before * mul_prev + (int64_t)tok * mul_cur) % buckets;
        if (row < 0) row += buckets;
    }
    const T* a = table + (size_t)tok * width;
    const T* b = second + (size_t)row * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)t * width + i] = to_f(a[i]) + to_f(b[i]);
}

// the last token of every entry of the step becomes its slot's previous token (after embed_hashed_kernel has read the old one)
__global__ void last_token_kernel(const int* __restrict__ tokens, float* __restrict__ prev, int64_t slot_stride, const int* __restrict__ cu_q,
                                  const int* __restrict__ seq_slot, int batch)
{
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= batch || cu_q[s] == cu_q[s + 1]) return;
    *reinterpret_cast<int*>(prev + (int64_t)seq_slot[s] * slot_stride) = tokens[cu_q[s + 1] - 1];
}

// x[t] += branch_scale * (left[t] / rms(left[t]) * wl + right[t] / rms(right[t]) * wr) + sum_p ff[t, p];  then
// hf[t] = x[t] / rms(x[t]) * w (float) and h[t] the same as T.  left / right (T [n, width]; both or neither), ff (TF = T or float,
// [n, parts, width]), w with h / hf are optional.  One block per row; every sum is float.
template <typename T, typename TF>
__global__ void branch_residual_norm_kernel(float* __restrict__ x, const T* __restrict__ left, const T* __restrict__ right,
                                            const float* __restrict__ wl, const float* __restrict__ wr, float branch_scale,
                                            const TF* __restrict__ ff, int parts, const float* __restrict__ w, int width, float eps,
                                            T* __restrict__ h, float* __restrict__ hf)
{
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * width;
    float rl = 0.f, rr = 0.f;
    if (left) {
        float sl = 0.f, sr = 0.f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float a = to_f(left[base + i]), b = to_f(right[base + i]);
            sl += a * a;
            sr += b * b;
        }
        sl = block_sum(sl, red);
        sr = block_sum(sr, red);
        rl = 1.0f / sqrtf(sl / (float)width + eps);
        rr = 1.0f / sqrtf(sr / (float)width + eps);
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = x[base + i];
        if (left || ff) {
            float y = 0.f;
            if (left) y = branch_scale * (to_f(left[base + i]) * rl * wl[i] + to_f(right[base + i]) * rr * wr[i]);
            for (int p = 0; p < parts; ++p) y += to_f(ff[((size_t)blockIdx.x * parts + p) * width + i]);
            v += y;
            x[base + i] = v;
        }
        ss += v * v;
    }
    if (!w) return;
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = x[base + i] * r * w[i];               // written above by this same thread
        if (h) h[base + i] = from_f<T>(v);
        if (hf) hf[base + i] = v;
    }
}

// the shifted row: cur + (before - cur) * s
__device__ __forceinline__ float shift_blend(float cur, float before, float s) { return fmaf(before - cur, s, cur); }

// Row t of entry s, local index j = t - cu_q[s]:  a_t = blend(h_t, h_(t-1), shift), and for every m < nmu
// blends[m][t] = blend(a_t, a_(t-1), mu[m]).  Rows before the step's first come from the slot: state = [h_last | a_last].
// h: float [n, width];  a (optional) and blends: T.  shift == nullptr: the row is not shifted (a_t = h_t).
template <typename T>
__global__ void token_shift_kernel(const float* __restrict__ h, const float* __restrict__ shift, const float* __restrict__ mu, int nmu,
                                   const float* __restrict__ state, int64_t slot_stride, const int* __restrict__ tok_seq,
                                   const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int n, int width, T* __restrict__ a,
                                   T* __restrict__ blends)
{
    const int t = blockIdx.x, s = tok_seq[t], j = t - cu_q[s];
    const float* st = state + (int64_t)seq_slot[s] * slot_stride;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float sh = shift ? shift[i] : 0.f;
        const float h0 = h[(size_t)t * width + i];
        const float h1 = j >= 1 ? h[(size_t)(t - 1) * width + i] : st[i];
        const float a0 = shift_blend(h0, h1, sh);
        float a1;
        if (j >= 1) {
            const float h2 = j >= 2 ? h[(size_t)(t - 2) * width + i] : st[i];
            a1 = shift_blend(h1, h2, sh);
        } else {
            a1 = st[width + i];
        }
        if (a) a[(size_t)t * width + i] = from_f<T>(a0);
        for (int m = 0; m < nmu; ++m)
            blends[((size_t)m * n + t) * width + i] = from_f<T>(shift_blend(a0, a1, mu[(size_t)m * width + i]));
    }
}

// the slot's [h_last | a_last] after the step; one thread per (entry, channel) reads the old state before it writes
__global__ void token_shift_state_kernel(const float* __restrict__ h, const float* __restrict__ shift, float* __restrict__ state,
                                         int64_t slot_stride, const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int width)
{
    const int s = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    const int first = cu_q[s], last = cu_q[s + 1];
    if (i >= width || first == last) return;
    float* st = state + (int64_t)seq_slot[s] * slot_stride;
    const float h0 = h[(size_t)(last - 1) * width + i];
    const float h1 = last - first >= 2 ? h[(size_t)(last - 2) * width + i] : st[i];
    st[i] = h0;
    st[width + i] = shift_blend(h0, h1, shift ? shift[i] : 0.f);
}

// decay[t, c] = exp(-exp(d[t, c] + w0[c])): float, once per (row, channel)
__global__ void channel_decay_kernel(const float* __restrict__ d, const float* __restrict__ w0, int channels, int64_t count,
                                     float* __restrict__ decay)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) decay[i] = expf(-expf(d[i] + w0[i % channels]));
}

// Per head, with S a [dim, vdim] float matrix per sequence:  o_t = (S + diag(u) k_t v_t^T)^T r_t,  S <- diag(w_t) S + k_t v_t^T.
// One block owns 32 value columns of one (sequence, head); its warps split the key channels, 16 each: lane j of warp w keeps
// S[16 w .. 16 w + 15, j] in registers, so a row costs no shuffle per column.  With c = sum_i r_i u_i k_i (the bonus term, common to
// all columns) a warp's part of a row is  sum_(its i) r_i S_ij + v_j c_(its i);  then S_ij <- w_i S_ij + k_i v_j.  The parts of R
// rows meet in shared memory, one block barrier per R rows (the parts are double-buffered), and warp u % warps writes row u.
// r_t, k_t and w_t of a warp's channels pass through the warp's own shared memory [3][R][16] (every lane reads them as 16-byte
// broadcasts); the next R rows' global loads are in flight while the current ones are computed.
// r, k, v: T with row stride ld; decay: float [n, heads * dim].  State layout per head: [vdim][dim] floats.
// blockDim = (32, ceil(dim / 16)); grid = (heads * ceil(vdim / 32), batch).  Channels past dim hold zeros and stay zero.
template <typename T, int R>
__global__ void __launch_bounds__(512) channel_decay_scan_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                                                                int64_t ld, const float* __restrict__ decay, const float* __restrict__ bonus,
                                                                float* __restrict__ state, int64_t slot_stride, const int* __restrict__ cu_q,
                                                                const int* __restrict__ seq_slot, int heads, int dim, int vdim,
                                                                float* __restrict__ out)
{
    constexpr int CK = 16, E = R * CK / 32;                   // key channels per warp; staged elements per lane and array
    static_assert(R * CK % 32 == 0 && 32 % CK == 0, "a warp stages whole rows");
    extern __shared__ __align__(16) float cds_smem[];
    const int lane = threadIdx.x, w = threadIdx.y, KW = blockDim.y, groups = (vdim + 31) / 32;
    const int s = blockIdx.y, first = cu_q[s], last = cu_q[s + 1];
    if (first == last) return;                                // the whole block leaves
    const int h = blockIdx.x / groups, col = (blockIdx.x - h * groups) * 32 + lane, c0 = w * CK;
    const bool live = col < vdim;
    float* rs = cds_smem + (size_t)w * 3 * R * CK;
    float* ks = rs + R * CK;
    float* wd = ks + R * CK;
    float* part = cds_smem + (size_t)KW * 3 * R * CK;         // [2][KW][R][32]
    float* sp = state + (int64_t)seq_slot[s] * slot_stride + ((size_t)h * vdim + (live ? col : 0)) * dim + c0;
    float S[CK];
    const bool vec = dim % 4 == 0 && (reinterpret_cast<uintptr_t>(sp) & 15) == 0;
#pragma unroll
    for (int i = 0; i < CK; i += 4) {
        if (vec && live && c0 + i < dim) {
            const float4 q = *reinterpret_cast<const float4*>(sp + i);
            S[i] = q.x; S[i + 1] = q.y; S[i + 2] = q.z; S[i + 3] = q.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) S[i + e] = (live && c0 + i + e < dim) ? sp[i + e] : 0.f;
        }
    }
    // staged element e of a lane: row (e * 32 + lane) / CK of the group, the warp's channel (e * 32 + lane) % CK
    const int my_d = c0 + lane % CK, my_u = lane / CK;
    const bool my_in = my_d < dim;
    const float ub = my_in ? bonus[(size_t)h * dim + my_d] : 0.f;
    const size_t hd = (size_t)heads * dim, my_at = (size_t)h * dim + my_d;
    float rr[E], kk[E], ww[E], vv[R];
    // the loads of rows [t0, t0 + R) into registers (zeros past the sequence's last row and past dim)
#define B200H_CDS_LOAD(t0)                                                                                        \
    _Pragma("unroll") for (int e = 0; e < E; ++e) {                                                               \
        const int u = e * (32 / CK) + my_u;                                                                       \
        const bool in = my_in && (t0) + u < last;                                                                 \
        const size_t t = (size_t)((t0) + u);                                                                      \
        rr[e] = in ? to_f(r[t * ld + my_at]) : 0.f;                                                               \
        kk[e] = in ? to_f(k[t * ld + my_at]) : 0.f;                                                               \
        ww[e] = in ? decay[t * hd + my_at] : 0.f;                                                                 \
    }                                                                                                             \
    _Pragma("unroll") for (int u = 0; u < R; ++u)                                                                 \
        vv[u] = (live && (t0) + u < last) ? to_f(v[(size_t)((t0) + u) * ld + (size_t)h * vdim + col]) : 0.f;
    B200H_CDS_LOAD(first)
    int p = 0;
    for (int t0 = first; t0 < last; t0 += R, p ^= 1) {
        float cc[R], vc[R];
        __syncwarp();                                        // the previous rows' readers are done with the warp's shared memory
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int at = e * 32 + lane;                    // = row * CK + channel
            rs[at] = rr[e];
            ks[at] = kk[e];
            wd[at] = ww[e];
            float c = rr[e] * ub * kk[e];                    // the bonus term of this warp's channels: summed over the CK lanes of a row
#pragma unroll
            for (int o = CK / 2; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
#pragma unroll
            for (int q = 0; q < 32 / CK; ++q) cc[e * (32 / CK) + q] = __shfl_sync(0xffffffffu, c, q * CK);
        }
#pragma unroll
        for (int u = 0; u < R; ++u) vc[u] = vv[u];
        __syncwarp();
        B200H_CDS_LOAD(t0 + R)                               // in flight while the staged rows are computed
        float* mine = part + ((size_t)(p * KW + w) * R) * 32 + lane;
#pragma unroll
        for (int u = 0; u < R; ++u) {
            if (t0 + u < last) {
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
                const float vj = vc[u];
#pragma unroll
                for (int i = 0; i < CK; i += 4) {
                    const float4 r4 = *reinterpret_cast<const float4*>(rs + u * CK + i);
                    const float4 k4 = *reinterpret_cast<const float4*>(ks + u * CK + i);
                    const float4 w4 = *reinterpret_cast<const float4*>(wd + u * CK + i);
                    a0 = fmaf(r4.x, S[i], a0);     S[i] = fmaf(w4.x, S[i], k4.x * vj);
                    a1 = fmaf(r4.y, S[i + 1], a1); S[i + 1] = fmaf(w4.y, S[i + 1], k4.y * vj);
                    a2 = fmaf(r4.z, S[i + 2], a2); S[i + 2] = fmaf(w4.z, S[i + 2], k4.z * vj);
                    a3 = fmaf(r4.w, S[i + 3], a3); S[i + 3] = fmaf(w4.w, S[i + 3], k4.w * vj);
                }
                mine[u * 32] = fmaf(vj, cc[u], (a0 + a1) + (a2 + a3));
            }
        }
        __syncthreads();
        for (int u = w; u < R; u += KW) {
            if (t0 + u < last && live) {
                float o = 0.f;
                for (int q = 0; q < KW; ++q) o += part[((size_t)(p * KW + q) * R + u) * 32 + lane];
                out[((size_t)(t0 + u) * heads + h) * vdim + col] = o;
            }
        }
    }
#undef B200H_CDS_LOAD
    if (!live) return;
#pragma unroll
    for (int i = 0; i < CK; i += 4) {
        if (vec && c0 + i < dim) {
            *reinterpret_cast<float4*>(sp + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (c0 + i + e < dim) sp[i + e] = S[i + e];
        }
    }
}

// y[t] = unit_rms_per_group(o[t]) * w * act(gate[t]) as T: the norm comes before the gate; `groups` equal parts of `count` columns;
// act 0: sigmoid, 1: silu.
template <typename T>
__global__ void group_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, const T* __restrict__ gate, int64_t ld_gate,
                                       int count, int groups, int act, float eps, T* __restrict__ y)
{
    __shared__ float red[32];
    const int t = blockIdx.x, g = blockIdx.y, gw = count / groups;
    const float* ot = o + (size_t)t * count + (size_t)g * gw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gw; i += blockDim.x) ss += ot[i] * ot[i];
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)gw + eps);
    for (int i = threadIdx.x; i < gw; i += blockDim.x) {
        const float z = to_f(gate[(size_t)t * ld_gate + (size_t)g * gw + i]);
        y[(size_t)t * count + (size_t)g * gw + i] = from_f<T>(ot[i] * r * w[(size_t)g * gw + i] * (act ? silu_f(z) : sigmoid_f(z)));
    }
}

// The same for groups of at most a few hundred columns (a head): one block per row, a WARP per group at a time -- the group's
// values stay in the lanes' registers between the sum of squares and the scaling, and nothing waits at a block barrier.
// NV = ceil(group width / 32) values per lane.
template <typename T, int NV>
__global__ void __launch_bounds__(256) group_norm_gate_warp_kernel(const float* __restrict__ o, const float* __restrict__ w,
                                                                  const T* __restrict__ gate, int64_t ld_gate, int count, int groups, int act,
                                                                  float eps, T* __restrict__ y)
{
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5, gw = count / groups;
    for (int g = warp; g < groups; g += nw) {
        const size_t at = (size_t)g * gw;
        const float* ot = o + (size_t)t * count + at;
        float v[NV], ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) { const int c = i * 32 + lane; v[i] = c < gw ? ot[c] : 0.f; ss += v[i] * v[i]; }
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)gw + eps);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = i * 32 + lane;
            if (c < gw) {
                const float z = to_f(gate[(size_t)t * ld_gate + at + c]);
                y[(size_t)t * count + at + c] = from_f<T>(v[i] * r * w[at + c] * (act ? silu_f(z) : sigmoid_f(z)));
            }
        }
    }
}

// x <- z > 0 ? softplus(p) z^2 + z / 2 : (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2, in place (T); params = {p, q} (float, device)
template <typename T>
__global__ void xielu_kernel(T* __restrict__ x, int64_t count, const float* __restrict__ params)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float z = to_f(x[i]);
    const float pos = softplus32(params[0]), neg = 0.5f + softplus32(params[1]);
    x[i] = from_f<T>(z > 0.f ? fmaf(pos * z, z, 0.5f * z) : fmaf(neg, expm1f(z) - z, 0.5f * z));
}

// x <- tanh(x) in place (T)
template <typename T>
__global__ void tanh_kernel(T* __restrict__ x, int64_t count)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) x[i] = from_f<T>(tanhf(to_f(x[i])));
}
