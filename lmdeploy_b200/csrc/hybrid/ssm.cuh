// Kernels of the selective state-space mixer: a short causal convolution per channel over strided projection columns (with
// the sequence's last taps-1 inputs as state), the per-head recurrence with a scalar decay per head and token, and the gated
// RMS norm in groups that follows it.
// Included by hybrid_ops.cu inside namespace b200h, after its helpers (to_f / from_f / block_sum / warp_sum / silu_f).
//
// Number formats: the projection (T) is read once; the convolution's output, step sizes, decays, the state and the
// recurrence's output are float.  State of a sequence: [taps-1, channels] floats of convolution inputs (oldest first) and
// [heads, vdim, state] floats of the recurrence.

// y[t, c] = act(bias[c] + sum_j w[c, j] * u[t - taps + 1 + j, c]) as float.  u is T with row stride ld; rows before the step's first
// row of the sequence come from its state, zeros at a sequence's start because a fresh slot is zeroed.  act: 0 none, 1 silu.
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ u, int64_t ld, const float* __restrict__ w, const float* __restrict__ bias, int act,
                                  const float* __restrict__ state, int64_t slot_stride, const int* __restrict__ tok_seq,
                                  const int* __restrict__ cu_q, const int* __restrict__ seq_slot, float* __restrict__ out, int channels, int taps)
{
    const int t = blockIdx.x, s = tok_seq[t], first = cu_q[s], local = t - first;
    const float* st = state + (int64_t)seq_slot[s] * slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float acc = bias ? bias[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = local - (taps - 1) + j;
            const float v = src >= 0 ? to_f(u[(size_t)(first + src) * ld + c]) : st[(size_t)(src + taps - 1) * channels + c];
            acc = fmaf(w[c * taps + j], v, acc);
        }
        out[(size_t)t * channels + c] = act == 1 ? silu_f(acc) : acc;
    }
}

// The state after the step: the last taps-1 inputs of (old state ++ this step's rows).  One thread owns a (sequence, channel)
// pair, reads all it needs and then writes, so a step shorter than taps-1 shifts the state correctly.
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ u, int64_t ld, float* __restrict__ state, int64_t slot_stride,
                                        const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int channels, int taps)
{
    const int s = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    const int first = cu_q[s], n = cu_q[s + 1] - first;
    if (c >= channels || n == 0) return;
    float* st = state + (int64_t)seq_slot[s] * slot_stride;
    float keep[B200H_MAX_TAPS];
    for (int k = 0; k < taps - 1; ++k) {
        const int src = n + k - (taps - 1);
        keep[k] = src >= 0 ? to_f(u[(size_t)(first + src) * ld + c]) : st[(size_t)(src + taps - 1) * channels + c];
    }
    for (int k = 0; k < taps - 1; ++k) st[(size_t)k * channels + c] = keep[k];
}

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// steps[t, h] = (dt, a) with dt = softplus(dt_raw[t, h] + dt_bias[h]) and a = exp(-exp(A_log[h]) * dt): computed once per (row, head)
// instead of once per value column of the head.
template <typename T>
__global__ void ssm_steps_kernel(const T* __restrict__ dt, int64_t ld_dt, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                 int heads, int64_t count, float2* __restrict__ steps)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const int64_t t = i / heads;
    const int h = (int)(i - t * heads);
    const float d = softplus_f(to_f(dt[t * ld_dt + h]) + dt_bias[h]);
    steps[i] = make_float2(d, expf(-expf(a_log[h]) * d));
}

// Per head S <- a_t S + dt_t B_t x_t^T, y_t = S^T C_t + D x_t, (dt_t, a_t) from ssm_steps_kernel.
// The columns of S (one per value channel) are independent: one warp owns NC value columns of one (sequence, head), lane l keeps
// rows l, l + 32, ... of those columns in registers and walks the sequence's rows of this step in order; B_t and C_t are read once
// for the warp's NC columns.
// xbc: float [n, inner + 2 * groups * N] = x | B | C after convolution and silu.
template <int NW, int NC>
__global__ void ssm_scan_kernel(const float* __restrict__ xbc, const float2* __restrict__ steps, const float* __restrict__ skip,
                                float* __restrict__ state, int64_t slot_stride, const int* __restrict__ cu_q,
                                const int* __restrict__ seq_slot, int heads, int vdim, int N, int groups, float* __restrict__ out)
{
    const int col = (blockIdx.x * blockDim.y + threadIdx.y) * NC, h = blockIdx.y, s = blockIdx.z, lane = threadIdx.x;
    if (col >= vdim) return;
    const int first = cu_q[s], last = cu_q[s + 1];
    if (first == last) return;
    const int inner = heads * vdim, channels = inner + 2 * groups * N, grp = h / (heads / groups);
    float* sp = state + (int64_t)seq_slot[s] * slot_stride + ((size_t)h * vdim + col) * N;
    float st[NC][NW];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < NW; ++i) { const int d = i * 32 + lane; st[c][i] = d < N ? sp[(size_t)c * N + d] : 0.f; }
    const float dskip = skip[h];
    const size_t x_at = (size_t)h * vdim + col, b_at = (size_t)inner + (size_t)grp * N, c_at = b_at + (size_t)groups * N;
    // four rows at a time: their loads do not depend on the state, only the four updates are in order
    for (int t0 = first; t0 < last; t0 += 4) {
        float ba[4][NW], ca[4][NW], xa[4][NC];
        float2 sd[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (t0 + u < last) {                      // a step of one row (decode) loads one row
                const float* row = xbc + (size_t)(t0 + u) * channels;
#pragma unroll
                for (int c = 0; c < NC; ++c) xa[u][c] = row[x_at + c];
                sd[u] = steps[(size_t)(t0 + u) * heads + h];
#pragma unroll
                for (int i = 0; i < NW; ++i) {
                    const int d = i * 32 + lane;
                    ba[u][i] = d < N ? row[b_at + d] : 0.f;
                    ca[u][i] = d < N ? row[c_at + d] : 0.f;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (t0 + u < last) {
                float part[NC];
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const float dx = sd[u].x * xa[u][c];
                    part[c] = 0.f;
#pragma unroll
                    for (int i = 0; i < NW; ++i) {
                        st[c][i] = fmaf(sd[u].y, st[c][i], ba[u][i] * dx);          // rows past N hold zeros and stay zero
                        part[c] = fmaf(st[c][i], ca[u][i], part[c]);
                    }
                }
#pragma unroll
                for (int c = 0; c < NC; ++c) part[c] = warp_sum(part[c]);
                if (lane == 0) {
#pragma unroll
                    for (int c = 0; c < NC; ++c) out[(size_t)(t0 + u) * inner + x_at + c] = part[c] + dskip * xa[u][c];
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < NW; ++i) { const int d = i * 32 + lane; if (d < N) sp[(size_t)c * N + d] = st[c][i]; }
}

// out[t] = unit_rms_per_group(y[t] * silu(gate[t])) * w as T: the gate comes before the norm; `groups` equal parts of `count` columns.
template <typename T>
__global__ void gate_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate, int64_t ld_gate, const float* __restrict__ w,
                                       int count, int groups, float eps, T* __restrict__ out)
{
    __shared__ float red[32];
    const int t = blockIdx.x, g = blockIdx.y, gw = count / groups;
    const float* yt = y + (size_t)t * count + g * gw;
    const T* gt = gate + (size_t)t * ld_gate + g * gw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gw; i += blockDim.x) { const float v = yt[i] * silu_f(to_f(gt[i])); ss += v * v; }
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)gw + eps);
    for (int i = threadIdx.x; i < gw; i += blockDim.x)
        out[(size_t)t * count + g * gw + i] = from_f<T>(yt[i] * silu_f(to_f(gt[i])) * r * w[g * gw + i]);
}
