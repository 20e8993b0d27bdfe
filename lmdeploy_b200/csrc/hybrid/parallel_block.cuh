// Kernels of parallel hybrid blocks (both sublayers read the same stream, their outputs join it together): the residual add
// fused with the two offset norms of the next layer, the preparation of an attention whose query and key pass a short
// convolution, a rotation and then a weightless per-head RMS norm and whose values are its keys, and two small epilogues.
// Included by hybrid_ops.cu inside namespace b200h, after ssm.cuh (short_conv_state_kernel) and the Rotary struct.

// x[t] += mult * (mix[t] + sum_p ff[t, p]) + add[t] + extra;  h1[t] = x[t] / rms(x[t]) * w1,  h2[t] = x[t] / rms(x[t]) * w2  (as T).
// mix (T [n, width]), ff (float [n, parts, width]), add (float [n, width]), extra (T [width]), h1 and h2 are optional; the two norms
// share one root mean square.  w1 / w2 hold the full factor (one plus the stored deviation).  h2f (optional): the second norm's
// result as float as well, for a router that reads it unrounded.
template <typename T>
__global__ void parallel_residual_norm_kernel(float* __restrict__ x, const T* __restrict__ mix, const float* __restrict__ ff, int parts,
                                              float mult, const float* __restrict__ add, const T* __restrict__ extra,
                                              const float* __restrict__ w1, const float* __restrict__ w2, int width, float eps,
                                              T* __restrict__ h1, T* __restrict__ h2, float* __restrict__ h2f)
{
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = x[base + i];
        if (mix || ff) {
            float y = mix ? to_f(mix[base + i]) : 0.f;
            for (int p = 0; p < parts; ++p) y += ff[((size_t)blockIdx.x * parts + p) * width + i];
            v = fmaf(mult, y, v);
        }
        if (add) v += add[base + i];
        if (extra) v += to_f(extra[i]);
        x[base + i] = v;
        ss += v * v;
    }
    if (!h1 && !h2) return;
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = x[base + i] * r;               // written above by this same thread
        if (h1) h1[base + i] = from_f<T>(v * w1[i]);
        if (h2) h2[base + i] = from_f<T>(v * w2[i]);
        if (h2f) h2f[base + i] = v * w2[i];
    }
}

// One block per row.  qk: T [n, ld] = heads * dim query columns, then kv_heads * dim key columns (one stacked projection).
//   1. every channel passes its short causal convolution (conv float [channels, taps]; earlier rows of the step, or the sequence's
//      state = its last taps-1 projected rows);
//   2. a key/value head's convolved key is its VALUE: stored in the cache as T before anything else touches it;
//   3. pairs (2i, 2i+1), i < rot.pairs, of every head turn by position * freqs[i];
//   4. every head is divided by its root mean square (no weight): queries -> qn (float), keys -> the cache (T).
// Shared memory: channels floats, then 2 * rot.pairs floats of cos / sin.
template <typename T>
__global__ void conv_rope_prep_kernel(const T* __restrict__ qk, int64_t ld, const float* __restrict__ conv, int taps,
                                      const float* __restrict__ state, int64_t slot_stride, const int* __restrict__ tok_seq,
                                      const int* __restrict__ tok_pos, const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
                                      Rotary rot, int heads, int kv_heads, int dim, float eps, const int64_t* __restrict__ block_ptrs,
                                      const int* __restrict__ cu_blocks, int64_t layer_off, int64_t v_off, int block_len,
                                      float* __restrict__ qn)
{
    extern __shared__ __align__(16) float prep_smem[];
    const int t = blockIdx.x, s = tok_seq[t], pos = tok_pos[t], first = cu_q[s], local = t - first;
    const int HD = heads * dim, GD = kv_heads * dim, channels = HD + GD;
    float* buf = prep_smem;
    float* cs = prep_smem + channels;
    float* sn = cs + rot.pairs;
    for (int i = threadIdx.x; i < rot.pairs; i += blockDim.x) {
        double sv, cv;
        sincos((double)pos * rot.freqs[i], &sv, &cv);
        cs[i] = (float)cv * rot.magnitude;
        sn[i] = (float)sv * rot.magnitude;
    }
    __syncthreads();
    const float* st = state + (int64_t)seq_slot[s] * slot_stride;
    char* page = reinterpret_cast<char*>(block_ptrs[cu_blocks[s] + pos / block_len]) + layer_off;
    const int at = pos % block_len;
    T* k_dst = reinterpret_cast<T*>(page) + (size_t)at * GD;
    T* v_dst = reinterpret_cast<T*>(page + v_off) + (size_t)at * GD;
    // one item per (head, pair of dimensions); a head of odd size ends in a lone dimension, which never turns
    const int per_head = (dim + 1) / 2;
    for (int i = threadIdx.x; i < (heads + kv_heads) * per_head; i += blockDim.x) {
        const int hh = i / per_head, pair = i - hh * per_head, c = hh * dim + 2 * pair;
        const bool two = 2 * pair + 1 < dim;
        float a = 0.f, b = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int src = local - (taps - 1) + j;
            float ua, ub = 0.f;
            if (src >= 0) {
                const T* row = qk + (size_t)(first + src) * ld + c;
                ua = to_f(row[0]);
                if (two) ub = to_f(row[1]);
            } else {
                const float* row = st + (size_t)(src + taps - 1) * channels + c;
                ua = row[0];
                if (two) ub = row[1];
            }
            a = fmaf(conv[c * taps + j], ua, a);
            if (two) b = fmaf(conv[(c + 1) * taps + j], ub, b);
        }
        if (c >= HD) {
            v_dst[c - HD] = from_f<T>(a);
            if (two) v_dst[c - HD + 1] = from_f<T>(b);
        }
        if (pair < rot.pairs) {                          // 2 * rot.pairs <= dim: a turning pair is always whole
            const float ra = a * cs[pair] - b * sn[pair], rb = b * cs[pair] + a * sn[pair];
            a = ra;
            b = rb;
        }
        buf[c] = a;
        if (two) buf[c + 1] = b;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int h = warp; h < heads + kv_heads; h += nw) {
        const float* v = buf + (size_t)h * dim;
        float ss = 0.f;
        for (int d = lane; d < dim; d += 32) ss += v[d] * v[d];
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)dim + eps);
        if (h < heads)
            for (int d = lane; d < dim; d += 32) qn[(size_t)t * HD + (size_t)h * dim + d] = v[d] * r;
        else
            for (int d = lane; d < dim; d += 32) k_dst[(size_t)(h - heads) * dim + d] = from_f<T>(v[d] * r);
    }
}

// x <- cap * tanh(x / cap) in place (float, `count` elements)
__global__ void softcap_kernel(float* __restrict__ x, int64_t count, float cap)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) x[i] = cap * tanhf(x[i] / cap);
}

// u[r, :] <- relu(scale[r] * u[r, :])^2 in place (T [rows, cols]; scale float [rows] or nullptr: 1)
template <typename T>
__global__ void scaled_relu2_kernel(T* __restrict__ u, const float* __restrict__ scale, int cols, int64_t count)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float v = fmaxf(to_f(u[i]) * (scale ? scale[i / cols] : 1.0f), 0.f);
    u[i] = from_f<T>(v * v);
}
