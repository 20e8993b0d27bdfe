// Kernels of pre-norm hybrid blocks: table rows added to the stream, residual add fused with an RMS norm, softmax attention
// with grouped key/value heads over a sliding window or within chunks of a paged cache (capped scores, a logarithmic distance
// penalty, the heads' weight rows recombined by a matrix after the softmax or their scores before it, a sink, an output gate per
// column or per head), the preparation of an attention that norms per head and rotates, and the squared-relu activation.
// Included by hybrid_ops.cu inside namespace b200h, after its helpers (to_f / from_f / block_sum / sigmoid_f).
//
// Cache entry of position p of a sequence, inside its page (page address + layer_off): the normed key as T at
// [p % block_len][kv_heads * dim], and, v_off bytes further, the value as T at [p % block_len][kv_heads * vdim].
//
// Attention runs in two passes over a row's visible keys [window_first(pos), pos] -- the window's first key, or the first key of
// the row's chunk --, both cut into `splits` equal key ranges so that a step of few rows still fills the SMs:
//   pass 1 (window_stats_kernel, one block per row block, key/value head and range): scores of the heads that share the key/value
//          head, written to a scratch [row, head, key - first visible key], and their running maximum and denominator;
//   pass 2 (window_pv_kernel, one block per row block and range): the ranges' (maximum, denominator) pairs are merged per head, the
//          scores of ALL heads of the row are read back, turned into final softmax weights, recombined across heads
//          (weight'_h = sum_g talk[h, g] weight_g -- this couples every head of a row, hence one block for all of them) and
//          applied to the values of each head's own key/value head;
//   window_out_kernel sums the ranges' partial outputs, applies sigmoid(gate) and writes T.
// A design that mixes the heads' SCORES runs window_mix_scores_kernel between the passes (scores mixed in place, maxima and
// denominators recomputed from the mixed scores) and pass 2 without its recombination.
// A block takes `rows` consecutive rows of the step; those of one sequence (consecutive positions) walk their keys together, so a
// cached key or value is read and converted once for all of them (prompt portions: 4 rows; a step of single tokens: 1).
// Scores, softmax, recombination and the weighted value sums are float whatever T is.

constexpr int kMaxPairs = 8;            // most (row, head) pairs handled per walk over a key: the kernels' template parameter NP

// x[t] += table[idx ? idx[t] : fixed]
template <typename T>
__global__ void add_rows_kernel(float* __restrict__ x, const T* __restrict__ table, const int* __restrict__ idx, int fixed, int width)
{
    const int t = blockIdx.x;
    const T* row = table + (size_t)(idx ? idx[t] : fixed) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) x[(size_t)t * width + i] += to_f(row[i]);
}

// x[t] += m[t] (+ extra); h[t] = x[t] / rms(x[t]) * w.  m, extra and h are optional.
template <typename T>
__global__ void residual_norm_kernel(float* __restrict__ x, const T* __restrict__ m, const T* __restrict__ extra,
                                     const float* __restrict__ w, int width, float eps, float* __restrict__ h)
{
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = x[base + i];
        if (m) v += to_f(m[base + i]);
        if (extra) v += to_f(extra[i]);
        if (m || extra) x[base + i] = v;
        ss += v * v;
    }
    if (!h) return;
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) h[base + i] = x[base + i] * r * w[i];
}

// x <- relu(x)^2 in place
template <typename T>
__global__ void relu2_kernel(T* __restrict__ x, int64_t count)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float v = fmaxf(to_f(x[i]), 0.f);
    x[i] = from_f<T>(v * v);
}

// One block per row: the projections' biases are added (float), the query is normed over all its heads at once (-> qn, float), the
// key likewise and written to the row's cache entry as T, the value is written to the cache.  wq / wk == nullptr: no norm of that
// projection; bias (q | k | v entries, float) == nullptr: none.
template <typename T>
__global__ void window_prep_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int64_t ld, int q_cols,
                                   int k_cols, int v_cols, const float* __restrict__ bias, const float* __restrict__ wq,
                                   const float* __restrict__ wk, float eps, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                   const int64_t* __restrict__ block_ptrs, const int* __restrict__ cu_blocks, int64_t layer_off, int64_t v_off,
                                   int block_len, float* __restrict__ qn)
{
    __shared__ float red[32];
    const int t = blockIdx.x, s = tok_seq[t], pos = tok_pos[t];
    const float* bq = bias;
    const float* bk = bias ? bias + q_cols : nullptr;
    const float* bv = bias ? bias + q_cols + k_cols : nullptr;
    const T* qr = q + (size_t)t * ld;
    float r = 1.0f;
    if (wq) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < q_cols; i += blockDim.x) { const float a = to_f(qr[i]) + (bq ? bq[i] : 0.f); ss += a * a; }
        ss = block_sum(ss, red);
        r = 1.0f / sqrtf(ss / (float)q_cols + eps);
    }
    for (int i = threadIdx.x; i < q_cols; i += blockDim.x) {
        const float a = to_f(qr[i]) + (bq ? bq[i] : 0.f);
        qn[(size_t)t * q_cols + i] = wq ? a * r * wq[i] : a;
    }
    char* page = reinterpret_cast<char*>(block_ptrs[cu_blocks[s] + pos / block_len]) + layer_off;
    const int at = pos % block_len;
    const T* kr = k + (size_t)t * ld;
    T* k_dst = reinterpret_cast<T*>(page) + (size_t)at * k_cols;
    r = 1.0f;
    if (wk) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < k_cols; i += blockDim.x) { const float a = to_f(kr[i]) + (bk ? bk[i] : 0.f); ss += a * a; }
        ss = block_sum(ss, red);
        r = 1.0f / sqrtf(ss / (float)k_cols + eps);
    }
    for (int i = threadIdx.x; i < k_cols; i += blockDim.x) {
        const float a = to_f(kr[i]) + (bk ? bk[i] : 0.f);
        k_dst[i] = from_f<T>(wk ? a * r * wk[i] : a);
    }
    const T* vr = v + (size_t)t * ld;
    T* v_dst = reinterpret_cast<T*>(page + v_off) + (size_t)at * v_cols;
    for (int i = threadIdx.x; i < v_cols; i += blockDim.x) v_dst[i] = from_f<T>(to_f(vr[i]) + (bv ? bv[i] : 0.f));
}

struct WindowGeom {
    int n, heads, kv_heads, dim, vdim, block_len, window, splits;
    int chunk;                // > 0: a row sees only the keys of its own chunk of this many positions, counted from position 0
    int rows;                 // rows of the step per block (consecutive rows; a block walks the keys once for those of one sequence)
    int tile;                 // keys per tile of pass 2, a multiple of 4, at most 256
    float scale, softcap;
    const float* r1;          // [heads] or nullptr: no distance penalty
    const float* r2;
    const float* talk;        // [heads, heads] or nullptr: heads are not recombined
    const float* sink;        // [heads] or nullptr: a score per head that joins the softmax denominator and carries no value
    const int* tok_seq;
    const int* tok_pos;
    const int64_t* block_ptrs;
    const int* cu_blocks;
    int64_t layer_off, v_off;
    float* scores;            // [rows of the step, heads, score_ld]: score of a row's key j at index j - (the row's first visible key)
    int score_ld;
};

// first visible key of a row at position pos
__device__ __forceinline__ int window_first(const WindowGeom& g, int pos)
{
    const int lo = g.window > 0 ? max(0, pos - g.window + 1) : 0;
    return g.chunk > 0 ? max(lo, pos / g.chunk * g.chunk) : lo;
}

// The key range `z` of consecutive rows of one sequence at positions first .. last: [j0, j1).  Every row masks the keys of the
// range that it does not see.
__device__ __forceinline__ void window_range(const WindowGeom& g, int first, int last, int z, int& j0, int& j1)
{
    const int lo = window_first(g, first);
    const int per = (last - lo + g.splits) / g.splits;         // ceil((last - lo + 1) / splits)
    j0 = lo + z * per;
    j1 = min(last + 1, j0 + per);
}

__device__ __forceinline__ bool window_sees(const WindowGeom& g, int pos, int j)
{
    return j <= pos && j >= window_first(g, pos);
}

// score of head `head` for a key at distance `dist` behind the query, from the raw dot product
__device__ __forceinline__ float window_score(const WindowGeom& g, float dot, int head, int dist)
{
    float s = dot * g.scale;
    if (g.softcap > 0.f) s = g.softcap * tanhf(s / g.softcap);
    if (g.r1) s -= g.r1[head] * log1pf(g.r2[head] * (float)dist);
    return s;
}

// dot products of one cached key with `cnt` (<= NP) queries that lie `dim` floats apart in shared memory.  VEC: 16-byte
// reads of the key and of the queries (dim * sizeof(T) is a multiple of 16 and everything is 16-byte aligned).
template <typename T, bool VEC, int NP>
__device__ __forceinline__ void key_dots(const T* __restrict__ key, const float* __restrict__ qs, int dim, int cnt, float* acc)
{
#pragma unroll
    for (int u = 0; u < NP; ++u) acc[u] = 0.f;
    if (VEC) {
        constexpr int N = 16 / (int)sizeof(T);
#pragma unroll 4                  // four 16-byte reads of the key in flight
        for (int d = 0; d < dim; d += N) {
            const uint4 raw = *reinterpret_cast<const uint4*>(key + d);
            const T* e = reinterpret_cast<const T*>(&raw);
            float kv[N];
#pragma unroll
            for (int i = 0; i < N; ++i) kv[i] = to_f(e[i]);
#pragma unroll
            for (int u = 0; u < NP; ++u) {
                if (u < cnt) {
                    const float4* qu = reinterpret_cast<const float4*>(qs + u * dim + d);
#pragma unroll
                    for (int i = 0; i < N / 4; ++i) {
                        const float4 q4 = qu[i];
                        acc[u] = fmaf(q4.x, kv[4 * i], acc[u]);
                        acc[u] = fmaf(q4.y, kv[4 * i + 1], acc[u]);
                        acc[u] = fmaf(q4.z, kv[4 * i + 2], acc[u]);
                        acc[u] = fmaf(q4.w, kv[4 * i + 3], acc[u]);
                    }
                }
            }
        }
    } else {
        for (int d = 0; d < dim; ++d) {
            const float kv = to_f(key[d]);
#pragma unroll
            for (int u = 0; u < NP; ++u)
                if (u < cnt) acc[u] = fmaf(qs[u * dim + d], kv, acc[u]);
        }
    }
}

// address of position j's cache entry of the layer (its key row; the value row lies v_off bytes + its own row offset further)
__device__ __forceinline__ const char* window_page(const WindowGeom& g, const int64_t* pages, int j)
{
    return reinterpret_cast<const char*>(pages[j / g.block_len]) + g.layer_off;
}

// (m, l) <- merge of two running (maximum, denominator) pairs
__device__ __forceinline__ void merge_ml(float& m, float& l, float om, float ol)
{
    const float mx = fmaxf(m, om);
    l = l * expf(m - mx) + ol * expf(om - mx);
    m = mx;
}

// Pass 1.  grid (row blocks, kv_heads, splits), up to 128 threads: thread i walks keys j0 + i, j0 + i + blockDim, ... of the range
// for all (row, head) pairs of the block's rows that belong to one sequence and of the heads that share key/value head blockIdx.y.
template <typename T, bool VEC, int NP>
__global__ void __launch_bounds__(128) window_stats_kernel(const float* __restrict__ qn, WindowGeom g, float* __restrict__ ml)
{
    extern __shared__ __align__(16) float win_smem[];
    __shared__ float red_m[4][kMaxPairs], red_l[4][kMaxPairs];
    const int c = blockIdx.y, z = blockIdx.z, tid = threadIdx.x, nw = blockDim.x >> 5;
    const int H = g.heads, D = g.dim, rep = H / g.kv_heads;
    const int t0 = blockIdx.x * g.rows, t1 = min(g.n, t0 + g.rows);
    float* qs = win_smem;                                                    // [rows * rep][dim]
    // VEC: one key row per thread after the queries, rows 16 bytes apart from a multiple of 128 so that the 16-byte reads of a
    // quarter warp fall into different banks
    char* stage = reinterpret_cast<char*>(win_smem + (size_t)g.rows * rep * D) + (size_t)tid * (D * sizeof(T) + 16);
    const size_t k_row = (size_t)g.kv_heads * D;
    for (int ta = t0; ta < t1;) {
        const int s = g.tok_seq[ta];
        int tb = ta + 1;
        while (tb < t1 && g.tok_seq[tb] == s) ++tb;
        const int nr = tb - ta, pos = g.tok_pos[ta], pairs = nr * rep;
        __syncthreads();
        for (int i = tid; i < pairs * D; i += blockDim.x) {
            const int u = i / D, d = i - u * D, r = u / rep, hh = u - r * rep;
            qs[i] = qn[((size_t)(ta + r) * H + c * rep + hh) * D + d];
        }
        __syncthreads();
        int j0, j1;
        window_range(g, pos, pos + nr - 1, z, j0, j1);
        const int64_t* pages = g.block_ptrs + g.cu_blocks[s];
        for (int ub = 0; ub < pairs; ub += NP) {
            const int cnt = min(NP, pairs - ub);
            float m[NP], l[NP];
#pragma unroll
            for (int u = 0; u < NP; ++u) { m[u] = -1e30f; l[u] = 0.f; }
            for (int j = j0 + tid; j < j1; j += blockDim.x) {
                const T* key = reinterpret_cast<const T*>(window_page(g, pages, j)) + (size_t)(j % g.block_len) * k_row + (size_t)c * D;
                if (VEC) {
                    // the thread's key travels to its own row of shared memory by asynchronous 16-byte copies: all of them are in
                    // flight at once and hold no registers; only the issuing thread reads the row, so its own wait suffices
                    const unsigned dst = (unsigned)__cvta_generic_to_shared(stage);
                    for (int b = 0; b < D * (int)sizeof(T); b += 16)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + b), "l"(reinterpret_cast<const char*>(key) + b) : "memory");
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                    key = reinterpret_cast<const T*>(stage);
                }
                float acc[NP];
                key_dots<T, VEC, NP>(key, qs + (size_t)ub * D, D, cnt, acc);
#pragma unroll
                for (int u = 0; u < NP; ++u) {
                    if (u < cnt) {
                        const int r = (ub + u) / rep, hh = (ub + u) - r * rep;
                        if (window_sees(g, pos + r, j)) {
                            const float sc = window_score(g, acc[u], c * rep + hh, pos + r - j);
                            g.scores[((size_t)(ta + r) * H + c * rep + hh) * g.score_ld + (j - window_first(g, pos + r))] = sc;
                            merge_ml(m[u], l[u], sc, 1.0f);
                        }
                    }
                }
            }
            // across the block: lanes of a warp by shuffles, the warps through shared memory
#pragma unroll
            for (int u = 0; u < NP; ++u) {
                for (int o = 16; o > 0; o >>= 1) {
                    const float om = __shfl_xor_sync(0xffffffffu, m[u], o), ol = __shfl_xor_sync(0xffffffffu, l[u], o);
                    merge_ml(m[u], l[u], om, ol);
                }
            }
            __syncthreads();
            if ((tid & 31) == 0) {
#pragma unroll
                for (int u = 0; u < NP; ++u) { red_m[tid >> 5][u] = m[u]; red_l[tid >> 5][u] = l[u]; }
            }
            __syncthreads();
            if (tid < cnt) {
                float mm = red_m[0][tid], ll = red_l[0][tid];
                for (int w = 1; w < nw; ++w) merge_ml(mm, ll, red_m[w][tid], red_l[w][tid]);
                const int r = (ub + tid) / rep, hh = (ub + tid) - r * rep;
                float* dst = ml + (((size_t)(ta + r) * H + c * rep + hh) * g.splits + z) * 2;
                dst[0] = mm;
                dst[1] = ll;
            }
        }
        ta = tb;
    }
}

// CW (1 or 4) consecutive values of a cached row as float
template <typename T, int CW> __device__ __forceinline__ void load_cols(const T* __restrict__ src, float* out);
template <> __device__ __forceinline__ void load_cols<float, 1>(const float* __restrict__ src, float* out) { out[0] = src[0]; }
template <> __device__ __forceinline__ void load_cols<bf16, 1>(const bf16* __restrict__ src, float* out) { out[0] = to_f(src[0]); }
template <> __device__ __forceinline__ void load_cols<float, 4>(const float* __restrict__ src, float* out)
{
    const float4 v = *reinterpret_cast<const float4*>(src);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <> __device__ __forceinline__ void load_cols<bf16, 4>(const bf16* __restrict__ src, float* out)
{
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
    out[0] = to_f(e[0]); out[1] = to_f(e[1]); out[2] = to_f(e[2]); out[3] = to_f(e[3]);
}

__device__ __forceinline__ int pad4(int v) { return (v + 3) & ~3; }

// Pass 2.  grid (row blocks, splits), 256 threads.  Shared memory: the tile's value row addresses [tile], then floats
// mx [rows * heads] | linv [rows * heads] | talk [heads][heads] | p [rows * heads][tile] | p2 [rows * heads][tile] |
// o [rows * heads][vdim] (every part padded to a multiple of four floats).
// CW: value columns per thread and walk (4: 8- or 16-byte reads of the values).  NP: (row, head) pairs per walk over a value -- 2 for
// a step of single tokens with two heads per key/value head, which keeps registers low and more blocks resident.
template <typename T, int CW, int NP>
__global__ void __launch_bounds__(256) window_pv_kernel(WindowGeom g, const float* __restrict__ ml, float* __restrict__ o_part)
{
    extern __shared__ __align__(16) unsigned char win_raw[];
    const int z = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
    const int H = g.heads, G = g.kv_heads, rep = H / G, V = g.vdim, KT = g.tile;
    const char** vrow = reinterpret_cast<const char**>(win_raw);
    float* mx = reinterpret_cast<float*>(win_raw + (size_t)KT * sizeof(char*));
    float* linv = mx + pad4(g.rows * H);
    float* talk = linv + pad4(g.rows * H);
    float* p = talk + (g.talk ? pad4(H * H) : 0);
    float* p2 = g.talk ? p + (size_t)g.rows * H * KT : p;
    float* o = p2 + (size_t)g.rows * H * KT;
    if (g.talk)
        for (int i = tid; i < H * H; i += nt) talk[i] = g.talk[i];
    const int t0 = blockIdx.x * g.rows, t1 = min(g.n, t0 + g.rows);
    const size_t v_row = (size_t)G * V * sizeof(T);
    for (int ta = t0; ta < t1;) {
        const int s = g.tok_seq[ta];
        int tb = ta + 1;
        while (tb < t1 && g.tok_seq[tb] == s) ++tb;
        const int nr = tb - ta, pos = g.tok_pos[ta], pairs = nr * rep;
        __syncthreads();
        for (int i = tid; i < nr * H * V; i += nt) o[i] = 0.f;
        for (int i = tid; i < nr * H; i += nt) {
            const float* src = ml + ((size_t)ta * H + i) * g.splits * 2;
            float mm = src[0], ll = src[1];
            for (int k = 1; k < g.splits; ++k) merge_ml(mm, ll, src[2 * k], src[2 * k + 1]);
            if (g.sink) merge_ml(mm, ll, g.sink[i % H], 1.0f);
            mx[i] = mm;
            linv[i] = 1.0f / ll;
        }
        int j0, j1;
        window_range(g, pos, pos + nr - 1, z, j0, j1);
        const int64_t* pages = g.block_ptrs + g.cu_blocks[s];
        for (int jt = j0; jt < j1; jt += KT) {
            const int kt = min(KT, j1 - jt), kt4 = pad4(kt);
            __syncthreads();                      // the previous tile's readers are done; mx / o of this segment are in place
            for (int jj = tid; jj < kt; jj += nt) {
                const int j = jt + jj;
                vrow[jj] = window_page(g, pages, j) + g.v_off + (size_t)(j % g.block_len) * v_row;
            }
            // final softmax weights of every (row, head) for the tile's keys (zero for a key the row does not see and for the
            // keys that pad the tile to a multiple of four), from the scores pass 1 left
            for (int item = tid; item < nr * H * kt4; item += nt) {
                const int rh = item / kt4, jj = item - rh * kt4, j = jt + jj, r = rh / H;
                float w = 0.f;
                if (jj < kt && window_sees(g, pos + r, j))
                    w = expf(g.scores[((size_t)ta * H + rh) * g.score_ld + (j - window_first(g, pos + r))] - mx[rh]) * linv[rh];
                p[(size_t)rh * KT + jj] = w;
            }
            __syncthreads();
            if (g.talk) {
                for (int item = tid; item < nr * H * kt4; item += nt) {
                    const int rh = item / kt4, jj = item - rh * kt4, r = rh / H, h = rh - r * H;
                    const float* pr = p + (size_t)r * H * KT + jj;
                    float a = 0.f;
                    for (int k = 0; k < H; ++k) a = fmaf(talk[h * H + k], pr[(size_t)k * KT], a);
                    p2[(size_t)rh * KT + jj] = a;
                }
                __syncthreads();
            }
            // weighted value sums: one (key/value head, CW value columns) item per thread and walk, each value read once for the
            // rows and heads that share it, four keys per step
            const int ncg = V / CW;
            for (int item = tid; item < G * ncg; item += nt) {
                const int c = item / ncg, col = (item - c * ncg) * CW;
                for (int ub = 0; ub < pairs; ub += NP) {
                    const int cnt = min(NP, pairs - ub);
                    float acc[NP][CW];
                    int rhs[NP];
#pragma unroll
                    for (int u = 0; u < NP; ++u) {
                        const int r = (ub + u) / rep;
                        rhs[u] = r * H + c * rep + (ub + u) - r * rep;
#pragma unroll
                        for (int k = 0; k < CW; ++k) acc[u][k] = 0.f;
                    }
#pragma unroll 2                  // eight value reads in flight
                    for (int jj = 0; jj < kt; jj += 4) {
                        float vv[4][CW];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (jj + q < kt) load_cols<T, CW>(reinterpret_cast<const T*>(vrow[jj + q]) + (size_t)c * V + col, vv[q]);
                            else {
#pragma unroll
                                for (int k = 0; k < CW; ++k) vv[q][k] = 0.f;
                            }
                        }
#pragma unroll
                        for (int u = 0; u < NP; ++u) {
                            if (u < cnt) {
                                const float4 w4 = *reinterpret_cast<const float4*>(p2 + (size_t)rhs[u] * KT + jj);
#pragma unroll
                                for (int k = 0; k < CW; ++k)
                                    acc[u][k] += (w4.x * vv[0][k] + w4.y * vv[1][k]) + (w4.z * vv[2][k] + w4.w * vv[3][k]);
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < NP; ++u) {
                        if (u < cnt) {
                            float* dst = o + (size_t)rhs[u] * V + col;
                            if (CW == 4) {                     // one 16-byte read and write per lane: no bank conflicts
                                float4 cur = *reinterpret_cast<float4*>(dst);
                                cur.x += acc[u][0]; cur.y += acc[u][CW > 1 ? 1 : 0]; cur.z += acc[u][CW > 2 ? 2 : 0]; cur.w += acc[u][CW > 3 ? 3 : 0];
                                *reinterpret_cast<float4*>(dst) = cur;
                            } else {
#pragma unroll
                                for (int k = 0; k < CW; ++k) dst[k] += acc[u][k];
                            }
                        }
                    }
                }
            }
        }
        __syncthreads();
        float* dst = o_part + ((size_t)ta * g.splits + z) * H * V;          // row r of the segment: ((ta + r) * splits + z) * H * V
        for (int i = tid; i < nr * H * V; i += nt) {
            const int r = i / (H * V);
            dst[(size_t)r * g.splits * H * V + (i - r * H * V)] = o[i];
        }
        ta = tb;
    }
}

// y[t, i] = (sum over ranges of o_part[t, z, i]) * sigmoid(gate[t, i / gate_div]) as T (gate_div 1: a gate per column; vdim: one per head)
template <typename T>
__global__ void window_out_kernel(const float* __restrict__ o_part, int splits, int cols, const T* __restrict__ gate, int64_t ld_gate,
                                  int gate_div, T* __restrict__ y)
{
    const int t = blockIdx.x, i = blockIdx.y * blockDim.x + threadIdx.x;          // one column per thread
    if (i >= cols) return;
    const float* src = o_part + (size_t)t * splits * cols + i;
    float a = 0.f;
#pragma unroll 8
    for (int z = 0; z < splits; ++z) a += src[(size_t)z * cols];
    if (gate) a *= sigmoid_f(to_f(gate[(size_t)t * ld_gate + i / gate_div]));
    y[(size_t)t * cols + i] = from_f<T>(a);
}

// Scores mixed ACROSS heads before the softmax: for every row and visible key, s'_h = sum_g talk[h, g] s_g, in place in the
// scratch pass 1 left, then every (row, head)'s running maximum and denominator over the mixed scores of the block's key range
// (pass 2 merges the ranges).  grid (rows, splits): a block takes key range blockIdx.y of ONE row -- the ranges pass 1 used when it
// cut a row's keys (one row per block there), the whole row otherwise; a tile of keys of all heads passes through shared memory:
// talk [heads][heads] | tile [heads][keys] floats.
__global__ void __launch_bounds__(256) window_mix_scores_kernel(WindowGeom g, const float* __restrict__ talk, int tile, float* __restrict__ ml)
{
    extern __shared__ __align__(16) float mix_smem[];
    const int t = blockIdx.x, z = blockIdx.y, H = g.heads, tid = threadIdx.x, nt = blockDim.x;
    const int pos = g.tok_pos[t], lo = window_first(g, pos);
    int j0, j1;
    window_range(g, pos, pos, z, j0, j1);
    j0 -= lo;                                                 // the scratch is indexed from the row's first visible key
    j1 -= lo;
    float* tk = mix_smem;
    float* raw = mix_smem + H * H;
    float* row = g.scores + (size_t)t * H * g.score_ld;
    for (int i = tid; i < H * H; i += nt) tk[i] = talk[i];
    for (int jt = j0; jt < j1; jt += tile) {
        const int kt = min(tile, j1 - jt);
        __syncthreads();
        for (int i = tid; i < H * kt; i += nt) { const int h = i / kt, jj = i - h * kt; raw[h * tile + jj] = row[(size_t)h * g.score_ld + jt + jj]; }
        __syncthreads();
        for (int i = tid; i < H * kt; i += nt) {
            const int h = i / kt, jj = i - h * kt;
            float a = 0.f;
            for (int k = 0; k < H; ++k) a = fmaf(tk[h * H + k], raw[k * tile + jj], a);
            row[(size_t)h * g.score_ld + jt + jj] = a;
        }
    }
    __syncthreads();
    const int lane = tid & 31, warp = tid >> 5, nw = nt >> 5;
    for (int h = warp; h < H; h += nw) {
        float m = -1e30f, l = 0.f;
        for (int j = j0 + lane; j < j1; j += 32) merge_ml(m, l, row[(size_t)h * g.score_ld + j], 1.0f);
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, m, o), ol = __shfl_xor_sync(0xffffffffu, l, o);
            merge_ml(m, l, om, ol);
        }
        if (lane == 0) {
            float* dst = ml + (((size_t)t * H + h) * g.splits + z) * 2;
            dst[0] = m;
            dst[1] = l;
        }
    }
}

// One block per row, for an attention whose query and key are normed PER HEAD and then rotated:
//   1. the projections' biases are added (float);
//   2. every head of q and of k is divided by its root mean square over `dim` and multiplied by a weight of `dim` entries that all
//      heads share (wq / wk; nullptr: no norm of that projection);
//   3. pairs (2i, 2i+1), i < rot.pairs, of every head turn by position * freqs[i];
//   4. queries -> qn (float), keys and (biased) values -> the row's cache entry as T.
// Shared memory: (heads + kv_heads) * dim floats, then 2 * rot.pairs floats of cos / sin.
template <typename T>
__global__ void head_rope_prep_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int64_t ld, int heads,
                                      int kv_heads, int dim, int vdim, const float* __restrict__ bias, const float* __restrict__ wq,
                                      const float* __restrict__ wk, float eps, Rotary rot, const int* __restrict__ tok_seq,
                                      const int* __restrict__ tok_pos, const int64_t* __restrict__ block_ptrs,
                                      const int* __restrict__ cu_blocks, int64_t layer_off, int64_t v_off, int block_len,
                                      float* __restrict__ qn)
{
    extern __shared__ __align__(16) float hr_smem[];
    const int t = blockIdx.x, s = tok_seq[t], pos = tok_pos[t];
    const int HD = heads * dim, GD = kv_heads * dim, GV = kv_heads * vdim;
    float* buf = hr_smem;
    float* cs = hr_smem + HD + GD;
    float* sn = cs + rot.pairs;
    for (int i = threadIdx.x; i < rot.pairs; i += blockDim.x) {
        double sv, cv;
        sincos((double)pos * rot.freqs[i], &sv, &cv);
        cs[i] = (float)cv * rot.magnitude;
        sn[i] = (float)sv * rot.magnitude;
    }
    for (int i = threadIdx.x; i < HD + GD; i += blockDim.x) {
        const float a = i < HD ? to_f(q[(size_t)t * ld + i]) : to_f(k[(size_t)t * ld + i - HD]);
        buf[i] = a + (bias ? bias[i] : 0.f);
    }
    __syncthreads();
    char* page = reinterpret_cast<char*>(block_ptrs[cu_blocks[s] + pos / block_len]) + layer_off;
    const int at = pos % block_len;
    T* k_dst = reinterpret_cast<T*>(page) + (size_t)at * GD;
    T* v_dst = reinterpret_cast<T*>(page + v_off) + (size_t)at * GV;
    for (int i = threadIdx.x; i < GV; i += blockDim.x) v_dst[i] = from_f<T>(to_f(v[(size_t)t * ld + i]) + (bias ? bias[HD + GD + i] : 0.f));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int h = warp; h < heads + kv_heads; h += nw) {
        float* x = buf + (size_t)h * dim;
        const float* wn = h < heads ? wq : wk;
        if (wn) {
            float ss = 0.f;
            for (int d = lane; d < dim; d += 32) ss += x[d] * x[d];
            ss = warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)dim + eps);
            for (int d = lane; d < dim; d += 32) x[d] = x[d] * r * wn[d];
        }
        __syncwarp();
        // one lane per pair of dimensions; a turning pair is whole (2 * rot.pairs <= dim), the rest pass unchanged
        for (int d = 2 * lane; d < dim; d += 64) {
            const bool two = d + 1 < dim;
            float a = x[d], b = two ? x[d + 1] : 0.f;
            if (d / 2 < rot.pairs) {
                const float ra = a * cs[d / 2] - b * sn[d / 2], rb = b * cs[d / 2] + a * sn[d / 2];
                a = ra;
                b = rb;
            }
            if (h < heads) {
                qn[(size_t)t * HD + (size_t)h * dim + d] = a;
                if (two) qn[(size_t)t * HD + (size_t)h * dim + d + 1] = b;
            } else {
                k_dst[(size_t)(h - heads) * dim + d] = from_f<T>(a);
                if (two) k_dst[(size_t)(h - heads) * dim + d + 1] = from_f<T>(b);
            }
        }
    }
}
