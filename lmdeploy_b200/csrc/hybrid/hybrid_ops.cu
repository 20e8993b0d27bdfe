// Operators of hybrid decoders (latent attention with a sink, decayed linear attention, routed experts, grouped RMS norm,
// short causal convolution, depth-weighted residual history; window_attention.cuh: pre-norm blocks and windowed attention;
// ssm.cuh, parallel_block.cuh: the state-space mixer, parallel blocks and convolved rotary attention) behind a C ABI of
// their own: libb200hybrid.so.
//
// Number formats.  T is the activation / weight type of the matrix products (float or bf16).  Everything the designs want in
// 32 bits is float here whatever T is: the residual stream and its history, every norm, rotary angles (double), attention
// scores and the online softmax, recurrent state, router scores.  Kernels read T only where a projection wrote it.
//
// Token addressing.  A step carries `n` rows; row t belongs to sequence tok_seq[t] of the batch and sits at position
// tok_pos[t] of that sequence.  cu_q[s] is the first row of sequence s (rows of a sequence are consecutive and in order).
// Paged cache: block_ptrs[cu_blocks[s] + p / block_len] is the address of the page that holds position p of sequence s;
// a layer's region starts layer_off bytes into the page.  Recurrent state: state + seq_slot[s] * slot_stride + layer offset.
#include "../../../include/b200_hybrid.h"
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200h {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over the block; every thread gets the result.  blockDim.x is a multiple of 32, at most 1024.
__device__ __forceinline__ float block_sum(float v, float* red)
{
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();                       // red may still be read from an earlier call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = 0.f;
    for (int i = 0; i < nw; ++i) r += red[i];
    return r;
}

// ------------------------------------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float scale, float* __restrict__ out,
                             int width)
{
    const int t = blockIdx.x;
    const T* row = table + (size_t)tokens[t] * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)t * width + i] = to_f(row[i]) * scale;
}

// ------------------------------------------------------------------------------------------------ short causal convolution
// out[t] = x[t] + sum_j w[:, j] * x[t - taps + 1 + j]; rows before the step's first come from the sequence's state
// (its last taps-1 inputs, oldest first), zeros at a sequence's start because a fresh slot is zeroed.
template <typename T>
__global__ void conv_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ state,
                            int64_t slot_stride, const int* __restrict__ tok_seq, const int* __restrict__ cu_q,
                            const int* __restrict__ seq_slot, T* __restrict__ out, int width, int taps)
{
    const int t = blockIdx.x, s = tok_seq[t], first = cu_q[s], local = t - first;
    const float* st = state + (int64_t)seq_slot[s] * slot_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = x[(size_t)t * width + c];
        for (int j = 0; j < taps; ++j) {
            const int src = local - (taps - 1) + j;
            const float v = src >= 0 ? x[(size_t)(first + src) * width + c] : st[(size_t)(src + taps - 1) * width + c];
            acc += w[c * taps + j] * v;
        }
        out[(size_t)t * width + c] = from_f<T>(acc);
    }
}

// The state after the step: the last taps-1 inputs of (old state ++ this step's rows).  One thread owns a (sequence, channel)
// pair, reads all it needs and then writes, so a step shorter than taps-1 shifts the state correctly.
__global__ void conv_state_kernel(const float* __restrict__ x, float* __restrict__ state, int64_t slot_stride,
                                  const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int width, int taps)
{
    const int s = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    const int first = cu_q[s], n = cu_q[s + 1] - first;
    if (c >= width || n == 0) return;
    float* st = state + (int64_t)seq_slot[s] * slot_stride;
    float keep[B200H_MAX_TAPS];
    for (int k = 0; k < taps - 1; ++k) {
        const int src = n + k - (taps - 1);
        keep[k] = src >= 0 ? x[(size_t)(first + src) * width + c] : st[(size_t)(src + taps - 1) * width + c];
    }
    for (int k = 0; k < taps - 1; ++k) st[(size_t)k * width + c] = keep[k];
}

// ------------------------------------------------------------------------------------------------ grouped RMS norm
// x[t] += w * unit_rms_per_group(sum_p m[t, p]); optionally also writes x as T (the next projection's input).
template <typename TI, typename T>
__global__ void residual_group_norm_kernel(float* __restrict__ x, const TI* __restrict__ m, int parts, const float* __restrict__ w,
                                           int width, int groups, float eps, T* __restrict__ x_t)
{
    __shared__ float red[32];
    const int t = blockIdx.x, g = blockIdx.y, gw = width / groups;
    const TI* mt = m + (size_t)t * parts * width + g * gw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gw; i += blockDim.x) {
        float v = 0.f;
        for (int p = 0; p < parts; ++p) v += to_f(mt[(size_t)p * width + i]);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)gw + eps);
    for (int i = threadIdx.x; i < gw; i += blockDim.x) {
        float v = 0.f;
        for (int p = 0; p < parts; ++p) v += to_f(mt[(size_t)p * width + i]);
        const size_t at = (size_t)t * width + g * gw + i;
        const float y = x[at] + v * r * w[g * gw + i];
        x[at] = y;
        if (x_t) x_t[at] = from_f<T>(y);
    }
}

// out[r] = w * unit_rms_per_group(x[rows[r]]) as T (rows == nullptr: row r).
template <typename T>
__global__ void group_norm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                                       int width, int groups, float eps, T* __restrict__ out)
{
    __shared__ float red[32];
    const int r = blockIdx.x, g = blockIdx.y, gw = width / groups;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * width + g * gw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gw; i += blockDim.x) ss += xr[i] * xr[i];
    ss = block_sum(ss, red);
    const float k = 1.0f / sqrtf(ss / (float)gw + eps);
    for (int i = threadIdx.x; i < gw; i += blockDim.x) out[(size_t)r * width + g * gw + i] = from_f<T>(xr[i] * k * w[g * gw + i]);
}

// ------------------------------------------------------------------------------------------------ depth-weighted history
// hist[terms-1] <- x (the layer's result); x <- sum_j coef[j] * hist[j], j ascending.
__global__ void depth_mix_kernel(float* __restrict__ x, float* __restrict__ hist, int64_t hist_stride, const float* __restrict__ coef,
                                 int terms, int64_t count)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float last = x[i];
    hist[(int64_t)(terms - 1) * hist_stride + i] = last;
    float acc = 0.f;
    for (int j = 0; j < terms - 1; ++j) acc += coef[j] * hist[(int64_t)j * hist_stride + i];
    x[i] = acc + coef[terms - 1] * last;
}

// ------------------------------------------------------------------------------------------------ latent attention
struct Rotary {
    const double* freqs;      // angle per position of pair i, i < pairs
    int pairs;                // rotated pairs; dimensions from 2 * pairs on pass unchanged
    float magnitude;          // factor on cos and sin
};

__device__ __forceinline__ void rotate_pair(float u, float v, int pos, double f, float mag, float& ru, float& rv)
{
    double sn, cs;
    sincos((double)pos * f, &sn, &cs);
    const float c = (float)cs * mag, s = (float)sn * mag;
    ru = u * c - v * s;
    rv = v * c + u * s;
}

// One block per row: the query latent is normed (-> cq as T), the key/value latent is normed and written to the row's cache
// entry as T, the shared rotated key part is rotated and written to the cache as float.
template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ dq, int64_t ld_dq, int q_rank, const float* __restrict__ wq,
                                   const T* __restrict__ dkv, int64_t ld_dkv, int kv_rank, int rot_dim, const float* __restrict__ wkv,
                                   float eps, Rotary rot, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                   const int64_t* __restrict__ block_ptrs, const int* __restrict__ cu_blocks, int64_t layer_off,
                                   int block_len, int64_t rot_off, T* __restrict__ cq)
{
    __shared__ float red[32];
    const int t = blockIdx.x, s = tok_seq[t], pos = tok_pos[t];
    const T* q = dq + (size_t)t * ld_dq;
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { const float v = to_f(q[i]); ss += v * v; }
    ss = block_sum(ss, red);
    float r = 1.0f / sqrtf(ss / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[(size_t)t * q_rank + i] = from_f<T>(to_f(q[i]) * r * wq[i]);

    const T* kv = dkv + (size_t)t * ld_dkv;
    char* page = reinterpret_cast<char*>(block_ptrs[cu_blocks[s] + pos / block_len]) + layer_off;
    const int at = pos % block_len;
    T* c_dst = reinterpret_cast<T*>(page) + (size_t)at * kv_rank;
    float* r_dst = reinterpret_cast<float*>(page + rot_off) + (size_t)at * rot_dim;
    ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) { const float v = to_f(kv[i]); ss += v * v; }
    ss = block_sum(ss, red);
    r = 1.0f / sqrtf(ss / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) c_dst[i] = from_f<T>(to_f(kv[i]) * r * wkv[i]);
    const T* kr = kv + kv_rank;
    for (int i = threadIdx.x; i < rot.pairs; i += blockDim.x)
        rotate_pair(to_f(kr[2 * i]), to_f(kr[2 * i + 1]), pos, rot.freqs[i], rot.magnitude, r_dst[2 * i], r_dst[2 * i + 1]);
    for (int i = 2 * rot.pairs + threadIdx.x; i < rot_dim; i += blockDim.x) r_dst[i] = to_f(kr[i]);
}

// The rotated part of every head's query, rotated: q_rot[t, h, :] (float).  The plain part is carried into the latent's
// coordinates by a batched GEMM (q_lat[t, h, :] = uk_h^T q_plain[t, h, :], so that q_lat . c == q_plain . (uk_h c) and no per-head
// key is ever materialised); the attention kernel applies the score scale.
template <typename T>
__global__ void rotate_query_kernel(const T* __restrict__ q, int64_t ld_q, int heads, int dim, int rot_dim, Rotary rot,
                                    const int* __restrict__ tok_pos, float* __restrict__ q_rot)
{
    const int t = blockIdx.x, pos = tok_pos[t];
    for (int h = threadIdx.y; h < heads; h += blockDim.y) {
        const T* qr = q + (size_t)t * ld_q + (size_t)h * (dim + rot_dim) + dim;
        float* out = q_rot + ((size_t)t * heads + h) * rot_dim;
        for (int i = threadIdx.x; i < rot.pairs; i += blockDim.x)
            rotate_pair(to_f(qr[2 * i]), to_f(qr[2 * i + 1]), pos, rot.freqs[i], rot.magnitude, out[2 * i], out[2 * i + 1]);
        for (int i = 2 * rot.pairs + threadIdx.x; i < rot_dim; i += blockDim.x) out[i] = to_f(qr[i]);
    }
}

// Causal attention of one (row, head, key range) per warp over the cached latents: score_j = q_lat . c_j + q_rot . kr_j, online
// softmax, o_lat = sum_j w_j c_j.  Lane l owns the latent coordinates l, l + 32, ...; a key's latent is loaded once and used for
// the score and for the weighted sum; four keys are in flight per iteration (independent dot products and reductions).  The
// warps of a block are heads of the same row: thirty-two keys at a time are staged in shared memory once for all of them.
// The keys of a row are cut into `splits` ranges of whole pages (blockIdx.z); range 0 starts its running maximum at the
// sink (a term exp(sink_h) in the denominator with no value), the others empty.  Every range leaves an unnormalised partial
// (max, denominator, weighted sum) that latent_out_kernel merges -- prompt portions run with one range, a step of single
// decoded tokens with several, so that a few rows still fill the SMs.
constexpr int kKeyTile = 32;           // keys staged in shared memory at a time, shared by the heads of the block

// Copy `bytes` (a multiple of `unit`) from global to shared memory with the whole block: 16-byte pieces when both allow it.
__device__ __forceinline__ void stage(void* dst, const void* src, int bytes, int unit, int tid, int nthreads)
{
    if (unit % 16 == 0) {
        for (int i = tid; i < bytes / 16; i += nthreads) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else if (unit % 4 == 0) {
        for (int i = tid; i < bytes / 4; i += nthreads) reinterpret_cast<unsigned*>(dst)[i] = reinterpret_cast<const unsigned*>(src)[i];
    } else {
        for (int i = tid; i < bytes / 2; i += nthreads)
            reinterpret_cast<unsigned short*>(dst)[i] = reinterpret_cast<const unsigned short*>(src)[i];
    }
}

template <typename T, int NC, int NR>
__global__ void __launch_bounds__(256, 2) latent_attention_kernel(const float* __restrict__ q_lat, const float* __restrict__ q_rot, const float* __restrict__ sink,
                                        int heads, int kv_rank, int rot_dim, const int* __restrict__ tok_seq,
                                        const int* __restrict__ tok_pos, const int64_t* __restrict__ block_ptrs,
                                        const int* __restrict__ cu_blocks, int64_t layer_off, int block_len, int64_t rot_off,
                                        int splits, float scale, float* __restrict__ o_lat, float* __restrict__ ml)
{
    extern __shared__ __align__(16) unsigned char tile_raw[];
    const int c_row = kv_rank * (int)sizeof(T), r_row = rot_dim * (int)sizeof(float);
    T* cs = reinterpret_cast<T*>(tile_raw);                                                       // [kKeyTile][kv_rank]
    float* rs = reinterpret_cast<float*>(tile_raw + (kKeyTile * c_row + 15) / 16 * 16);           // [kKeyTile][rot_dim]
    const int t = blockIdx.x, z = blockIdx.z, lane = threadIdx.x;
    const int tid = threadIdx.y * 32 + lane, nthreads = blockDim.y * 32;
    const int h_raw = blockIdx.y * blockDim.y + threadIdx.y;
    const bool live = h_raw < heads;                  // a warp past the last head still helps staging and meets the barriers
    const int h = live ? h_raw : heads - 1;
    const int s = tok_seq[t], pos = tok_pos[t];
    float ql[NC], qr[NR], acc[NC];
    const float* qlp = q_lat + ((size_t)t * heads + h) * kv_rank;
    const float* qrp = q_rot + ((size_t)t * heads + h) * rot_dim;
#pragma unroll
    for (int i = 0; i < NC; ++i) { const int c = i * 32 + lane; ql[i] = c < kv_rank ? qlp[c] : 0.f; acc[i] = 0.f; }
#pragma unroll
    for (int i = 0; i < NR; ++i) { const int c = i * 32 + lane; qr[i] = c < rot_dim ? qrp[c] : 0.f; }
    float m = z == 0 ? sink[h] : -1e30f, l = z == 0 ? 1.0f : 0.0f;
    const int64_t* pages = block_ptrs + cu_blocks[s];
    const int n_pages = pos / block_len + 1, per = (n_pages + splits - 1) / splits;
    const int p_lo = z * per, p_hi = min(n_pages, p_lo + per);
    for (int pg = p_lo; pg < p_hi; ++pg) {
        const char* page = reinterpret_cast<const char*>(pages[pg]) + layer_off;
        const int cnt = min(block_len, pos + 1 - pg * block_len);
        for (int j0 = 0; j0 < cnt; j0 += kKeyTile) {
            const int kt = min(kKeyTile, cnt - j0);
            __syncthreads();
            stage(cs, page + (size_t)j0 * c_row, kt * c_row, c_row, tid, nthreads);
            stage(rs, page + rot_off + (size_t)j0 * r_row, kt * r_row, r_row, tid, nthreads);
            __syncthreads();
            if (!live) continue;
            int j = 0;
            for (; j + 4 <= kt; j += 4) {
                float cv[4][NC], part[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    part[u] = 0.f;
#pragma unroll
                    for (int i = 0; i < NC; ++i) {
                        const int c = i * 32 + lane;
                        cv[u][i] = c < kv_rank ? to_f(cs[(j + u) * kv_rank + c]) : 0.f;
                        part[u] = fmaf(ql[i], cv[u][i], part[u]);
                    }
#pragma unroll
                    for (int i = 0; i < NR; ++i) {
                        const int c = i * 32 + lane;
                        if (c < rot_dim) part[u] = fmaf(qr[i], rs[(j + u) * rot_dim + c], part[u]);
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) part[u] += __shfl_xor_sync(0xffffffffu, part[u], o);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) part[u] *= scale;
                const float mn = fmaxf(fmaxf(fmaxf(m, part[0]), fmaxf(part[1], part[2])), part[3]);
                const float alpha = expf(m - mn);
                float p[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) p[u] = expf(part[u] - mn);
                l = l * alpha + ((p[0] + p[1]) + (p[2] + p[3]));
#pragma unroll
                for (int i = 0; i < NC; ++i)
                    acc[i] = acc[i] * alpha + ((p[0] * cv[0][i] + p[1] * cv[1][i]) + (p[2] * cv[2][i] + p[3] * cv[3][i]));
                m = mn;
            }
            for (; j < kt; ++j) {
                float cv[NC], part = 0.f;
#pragma unroll
                for (int i = 0; i < NC; ++i) {
                    const int c = i * 32 + lane;
                    cv[i] = c < kv_rank ? to_f(cs[j * kv_rank + c]) : 0.f;
                    part = fmaf(ql[i], cv[i], part);
                }
#pragma unroll
                for (int i = 0; i < NR; ++i) {
                    const int c = i * 32 + lane;
                    if (c < rot_dim) part = fmaf(qr[i], rs[j * rot_dim + c], part);
                }
                const float sc = warp_sum(part) * scale;
                const float mn = fmaxf(m, sc);
                const float alpha = expf(m - mn), p = expf(sc - mn);
                l = l * alpha + p;
#pragma unroll
                for (int i = 0; i < NC; ++i) acc[i] = acc[i] * alpha + p * cv[i];
                m = mn;
            }
        }
    }
    if (!live) return;
    const size_t at = ((size_t)t * heads + h) * splits + z;
    float* out = o_lat + at * kv_rank;
#pragma unroll
    for (int i = 0; i < NC; ++i) { const int c = i * 32 + lane; if (c < kv_rank) out[c] = acc[i]; }
    if (lane == 0) { ml[2 * at] = m; ml[2 * at + 1] = l; }
}

// Merge of the key ranges' partials into the normalised weighted latent sum, stored as T head-major [heads, n, kv_rank]: the
// operand of the batched GEMM that expands it to values (o[h] = o_lat[h] uv_h^T).
template <typename T>
__global__ void latent_merge_kernel(const float* __restrict__ o_lat, const float* __restrict__ ml, int splits, int n, int heads,
                                    int kv_rank, T* __restrict__ out)
{
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t at = ((size_t)t * heads + h) * splits;
    float top = ml[2 * at];
    for (int z = 1; z < splits; ++z) top = fmaxf(top, ml[2 * (at + z)]);
    float den = 0.f;
    for (int z = 0; z < splits; ++z) den += expf(ml[2 * (at + z)] - top) * ml[2 * (at + z) + 1];
    const float inv = 1.0f / den;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
        float v = 0.f;
        for (int z = 0; z < splits; ++z) v += expf(ml[2 * (at + z)] - top) * o_lat[(at + z) * kv_rank + c];
        out[((size_t)h * n + t) * kv_rank + c] = from_f<T>(v * inv);
    }
}

// y[t, h*vdim + v] = o[h, t, v] * sigmoid(gate[t, h*vdim + v]) as T; o float head-major [heads, n, vdim].
template <typename T>
__global__ void head_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int64_t ld_gate, int n, int heads, int vdim,
                                 T* __restrict__ y)
{
    const int t = blockIdx.x, cols = heads * vdim;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const int h = i / vdim, v = i - h * vdim;
        y[(size_t)t * cols + i] = from_f<T>(o[((size_t)h * n + t) * vdim + v] * sigmoid_f(to_f(gate[(size_t)t * ld_gate + i])));
    }
}

// ------------------------------------------------------------------------------------------------ decayed linear attention
// Per head S <- decay * S + k v^T, o = S^T q with q, k, v = silu(projection).  The columns of S are independent, so one warp
// owns one (sequence, head, value column): lane l keeps rows l, l + 32, ... of that column in registers and walks the
// sequence's rows of this step in order.  State layout per head: [vdim][dim] floats.
template <typename T, int NW>
__global__ void decay_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int64_t ld,
                                  const float* __restrict__ decay, float* __restrict__ state, int64_t slot_stride,
                                  const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int heads, int dim, int vdim,
                                  float* __restrict__ out)
{
    const int col = blockIdx.x * blockDim.y + threadIdx.y, h = blockIdx.y, s = blockIdx.z, lane = threadIdx.x;
    if (col >= vdim) return;
    const int first = cu_q[s], last = cu_q[s + 1];
    if (first == last) return;
    float* sp = state + (int64_t)seq_slot[s] * slot_stride + ((size_t)h * vdim + col) * dim;
    float st[NW];
#pragma unroll
    for (int i = 0; i < NW; ++i) { const int d = i * 32 + lane; st[i] = d < dim ? sp[d] : 0.f; }
    const float lam = decay[h];
    // four rows at a time: their q, k, v loads and activations do not depend on the state, only the four updates are in order
    for (int t0 = first; t0 < last; t0 += 4) {
        float qa[4][NW], ka[4][NW], va[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (t0 + u < last) {                      // a step of one row (decode) loads and activates one row
                const int t = t0 + u;
                const T* qt = q + (size_t)t * ld + (size_t)h * dim;
                const T* kt = k + (size_t)t * ld + (size_t)h * dim;
                va[u] = to_f(v[(size_t)t * ld + (size_t)h * vdim + col]);
#pragma unroll
                for (int i = 0; i < NW; ++i) {
                    const int d = i * 32 + lane;
                    qa[u][i] = d < dim ? to_f(qt[d]) : 0.f;
                    ka[u][i] = d < dim ? to_f(kt[d]) : 0.f;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (t0 + u < last) {
                va[u] = silu_f(va[u]);
#pragma unroll
                for (int i = 0; i < NW; ++i) { qa[u][i] = silu_f(qa[u][i]); ka[u][i] = silu_f(ka[u][i]); }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (t0 + u < last) {
                float part = 0.f;
#pragma unroll
                for (int i = 0; i < NW; ++i) {
                    st[i] = fmaf(lam, st[i], ka[u][i] * va[u]);          // rows past dim hold zeros and stay zero
                    part = fmaf(st[i], qa[u][i], part);
                }
                part = warp_sum(part);
                if (lane == 0) out[((size_t)(t0 + u) * heads + h) * vdim + col] = part;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < NW; ++i) { const int d = i * 32 + lane; if (d < dim) sp[d] = st[i]; }
}

// y[t] = unit_rms(o[t]) * w * sigmoid(gate[t]) as T over the concatenated heads.
template <typename T>
__global__ void gated_rms_kernel(const float* __restrict__ o, const float* __restrict__ w, const T* __restrict__ gate, int64_t ld_gate,
                                 int count, float eps, T* __restrict__ y)
{
    __shared__ float red[32];
    const int t = blockIdx.x;
    const float* ot = o + (size_t)t * count;
    float ss = 0.f;
    for (int i = threadIdx.x; i < count; i += blockDim.x) ss += ot[i] * ot[i];
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)count + eps);
    for (int i = threadIdx.x; i < count; i += blockDim.x)
        y[(size_t)t * count + i] = from_f<T>(ot[i] * r * w[i] * sigmoid_f(to_f(gate[(size_t)t * ld_gate + i])));
}

// ------------------------------------------------------------------------------------------------ routed experts
// Router: logits = router x (float); scores = softmax over all experts (score_fn 0) or the sigmoid of every logit on its own
// (score_fn 1); the `top` largest (ties: the lower index), their scores as weights.  x is float or T.
template <typename TI>
__global__ void route_kernel(const TI* __restrict__ x, const float* __restrict__ router, int width, int experts, int top, int score_fn,
                             int* __restrict__ ids, float* __restrict__ wts)
{
    extern __shared__ float sm[];
    float* xs = sm;
    float* z = sm + width;
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = to_f(x[(size_t)t * width + i]);
    __syncthreads();
    for (int e = warp; e < experts; e += nw) {
        const float* row = router + (size_t)e * width;
        float part = 0.f;
        for (int i = lane; i < width; i += 32) part = fmaf(row[i], xs[i], part);
        part = warp_sum(part);
        if (lane == 0) z[e] = part;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float inv = 1.0f;
        if (score_fn == 1) {
            // the sigmoid is monotonic: the choice is made on the logits themselves (two large logits whose sigmoids both round
            // to one are still told apart), and only the chosen ones' sigmoids are taken
            for (int k = 0; k < top; ++k) {
                int best = -1;
                float bv = -INFINITY;
                for (int e = 0; e < experts; ++e)
                    if (z[e] > bv || best < 0) { bv = z[e]; best = e; }
                ids[(size_t)t * top + k] = best;
                wts[(size_t)t * top + k] = sigmoid_f(bv);
                z[best] = -INFINITY;
            }
            return;
        } else {
            float mx = z[0];
            for (int e = 1; e < experts; ++e) mx = fmaxf(mx, z[e]);
            float sum = 0.f;
            for (int e = 0; e < experts; ++e) { z[e] = expf(z[e] - mx); sum += z[e]; }
            inv = 1.0f / sum;
        }
        for (int k = 0; k < top; ++k) {
            int best = -1;
            float bv = -1.0f;
            for (int e = 0; e < experts; ++e)
                if (z[e] > bv) { bv = z[e]; best = e; }
            ids[(size_t)t * top + k] = best;
            wts[(size_t)t * top + k] = bv * inv;
            z[best] = -2.0f;
        }
    }
}

// Router with sigmoid scores s = sigmoid(router x) and a choice among GROUPS of neighbouring experts: the choice score of an
// expert is s + correction (correction nullptr: s); a group's score is the sum of its `group_top` largest choice scores; only the
// experts of the `keep` best groups can be chosen (ties: the lower index), the `top` with the largest choice scores are.  The
// weights are the chosen experts' s WITHOUT the correction, divided by their sum + 1e-20 when renorm, times scale.
// Shared memory: width floats of x, then experts logits, experts choice scores, groups group scores.
template <typename TI>
__global__ void route_grouped_kernel(const TI* __restrict__ x, const float* __restrict__ router, const float* __restrict__ correction,
                                     int width, int experts, int top, int groups, int keep, int group_top, int renorm, float scale,
                                     int* __restrict__ ids, float* __restrict__ wts)
{
    extern __shared__ float sm[];
    float* xs = sm;
    float* sc = sm + width;
    float* ch = sc + experts;
    float* gs = ch + experts;
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int i = threadIdx.x; i < width; i += blockDim.x) xs[i] = to_f(x[(size_t)t * width + i]);
    __syncthreads();
    for (int e = warp; e < experts; e += nw) {
        const float* row = router + (size_t)e * width;
        float part = 0.f;
        for (int i = lane; i < width; i += 32) part = fmaf(row[i], xs[i], part);
        part = warp_sum(part);
        if (lane == 0) {
            sc[e] = sigmoid_f(part);
            ch[e] = sc[e] + (correction ? correction[e] : 0.f);
        }
    }
    __syncthreads();
    const int per = experts / groups;
    if (groups > 1 && keep < groups) {
        // a group's score: its group_top largest choice scores, found by repeated selection (one thread per group)
        for (int g = threadIdx.x; g < groups; g += blockDim.x) {
            float total = 0.f, bound = INFINITY;
            int bound_at = -1;                          // the last one taken: equal values are taken in index order
            for (int k = 0; k < group_top && k < per; ++k) {
                float bv = -INFINITY;
                int best = -1;
                for (int e = 0; e < per; ++e) {
                    const float c = ch[g * per + e];
                    const bool after = c < bound || (c == bound && e > bound_at);
                    if (after && (best < 0 || c > bv)) { bv = c; best = e; }
                }
                total += bv;
                bound = bv;
                bound_at = best;
            }
            gs[g] = total;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            // groups that are NOT kept: the groups - keep worst (ties: the higher index goes first)
            for (int k = 0; k < groups - keep; ++k) {
                int worst = -1;
                float wv = INFINITY;
                for (int g = 0; g < groups; ++g)
                    if (gs[g] == gs[g] && (worst < 0 || gs[g] <= wv)) { wv = gs[g]; worst = g; }
                gs[worst] = nanf("");
                for (int e = 0; e < per; ++e) ch[worst * per + e] = -INFINITY;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < experts; ++e)
                if (ch[e] == ch[e] && (best < 0 || ch[e] > bv)) { bv = ch[e]; best = e; }
            ids[(size_t)t * top + k] = best;
            sum += sc[best];
            ch[best] = nanf("");                        // taken
        }
        const float f = (renorm ? 1.0f / (sum + 1e-20f) : 1.0f) * scale;
        for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] = sc[ids[(size_t)t * top + k]] * f;
    }
}

// Experts for a step of few rows, expert-major so that an expert's weights stream from HBM once whatever the number of rows
// that chose it.  Entry i = (row i / top, choice i % top).  expert_lists_kernel collects every expert's entries;
// expert_rows_kernel gives a block 32 weight rows of one expert and walks that expert's entries eight at a time: the
// eight input rows sit in shared memory as T, a warp takes one weight row at a time, every lane reads its 16-byte pieces of
// the row once and feeds eight float accumulators, and the warp reduces them.
//   MODE 1: out[i, r] = silu(w gate_e[r] . x) * (w up_e[r] . x) as T     (x = the row's stream as T, K = width, R = ff)
//   MODE 2: out[i, r] = relu(w up_e[r] . x)^2 as T                       (an expert without a gate matrix)
//   MODE 0: out[i, r] = w * (down_e[r] . mid[i]) as float                (K = ff, R = width)
// w = wts[i], or 1 when wts is nullptr: a design whose router score scales the expert's INPUT gives the score to the first
// product (the first map is linear, so scaling its result is scaling its input, without rounding the scaled input to T).
// The order of an expert's list depends on the atomics' order; every entry's result lands in its own place, so the numbers do not.
__global__ void expert_lists_kernel(const int* __restrict__ ids, int entries, int experts, int* __restrict__ counts, int* __restrict__ lists)
{
    extern __shared__ int cnt[];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < entries; i += blockDim.x) {
        const int e = ids[i];
        lists[(size_t)e * entries + atomicAdd(&cnt[e], 1)] = i;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = cnt[e];
}

constexpr int kExpertTile = 8;         // entries per pass over an expert's weight rows
constexpr int kExpertRows = 32;        // weight rows per block

template <typename T> struct Pack;     // 16 bytes of T
template <> struct Pack<bf16> { static constexpr int N = 8; };
template <> struct Pack<float> { static constexpr int N = 4; };

template <typename T>
__device__ __forceinline__ void load_pack(const T* p, float (&v)[Pack<T>::N]);
template <>
__device__ __forceinline__ void load_pack<bf16>(const bf16* p, float (&v)[8])
{
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void load_pack<float>(const float* p, float (&v)[4])
{
    const float4 raw = *reinterpret_cast<const float4*>(p);
    v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
}

template <typename T, int MODE, bool VEC, int TILE>
__global__ void __launch_bounds__(256, 3) expert_rows_kernel(const T* __restrict__ x, int x_div, const T* __restrict__ wa, const T* __restrict__ wb,
                                   const int* __restrict__ counts, const int* __restrict__ lists, int entries,
                                   const float* __restrict__ wts, int K, int R, void* __restrict__ out_)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr bool DUAL = MODE == 1;
    T* xs = reinterpret_cast<T*>(smem_raw);                     // [TILE][K]
    const int e = blockIdx.y, r0 = blockIdx.x * kExpertRows;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int count = counts[e];
    const int* list = lists + (size_t)e * entries;
    const T* wae = wa + (size_t)e * R * K;
    const T* wbe = DUAL ? wb + (size_t)e * R * K : nullptr;
    constexpr int P = Pack<T>::N;
    for (int base = 0; base < count; base += TILE) {
        const int live = min(TILE, count - base);
        __syncthreads();
        for (int u = 0; u < TILE; ++u) {
            const T* src = u < live ? x + (size_t)(list[base + u] / x_div) * K : nullptr;
            for (int i = threadIdx.x; i < K; i += blockDim.x) xs[(size_t)u * K + i] = src ? src[i] : from_f<T>(0.f);
        }
        __syncthreads();
        for (int r = r0 + warp; r < min(R, r0 + kExpertRows); r += nw) {
            float a[TILE], b[TILE];
#pragma unroll
            for (int u = 0; u < TILE; ++u) a[u] = b[u] = 0.f;
            const T* ra = wae + (size_t)r * K;
            const T* rb = DUAL ? wbe + (size_t)r * K : nullptr;
            if (VEC) {
                // 16-byte pieces of weights requested before any is used: two of the row and two of its twin, or four of a lone
                // first-stage row; the second stage requests two
                constexpr int NQ = MODE == 2 ? 4 : 2;
                for (int i = lane * P; i < K; i += 32 * NQ * P) {
                    float va[NQ][P], vb[DUAL ? NQ : 1][P];
#pragma unroll
                    for (int q2 = 0; q2 < NQ; ++q2) {
                        const int at = i + q2 * 32 * P;
                        if (at < K) {
                            load_pack<T>(ra + at, va[q2]);
                            if (DUAL) load_pack<T>(rb + at, vb[DUAL ? q2 : 0]);
                        }
                    }
#pragma unroll
                    for (int q2 = 0; q2 < NQ; ++q2) {
                        const int at = i + q2 * 32 * P;
                        if (at < K) {
#pragma unroll
                            for (int u = 0; u < TILE; ++u) {
                                float xv[P];
                                load_pack<T>(xs + (size_t)u * K + at, xv);
#pragma unroll
                                for (int k = 0; k < P; ++k) {
                                    a[u] = fmaf(va[q2][k], xv[k], a[u]);
                                    if (DUAL) b[u] = fmaf(vb[DUAL ? q2 : 0][k], xv[k], b[u]);
                                }
                            }
                        }
                    }
                }
            } else {
                for (int i = lane; i < K; i += 32) {
                    const float va = to_f(ra[i]), vb = DUAL ? to_f(rb[i]) : 0.f;
#pragma unroll
                    for (int u = 0; u < TILE; ++u) {
                        const float xv = to_f(xs[(size_t)u * K + i]);
                        a[u] = fmaf(va, xv, a[u]);
                        if (DUAL) b[u] = fmaf(vb, xv, b[u]);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < TILE; ++u) {
                a[u] = warp_sum(a[u]);
                if (DUAL) b[u] = warp_sum(b[u]);
            }
            if (lane < live) {
                float va = 0.f, vb = 0.f;
#pragma unroll
                for (int u = 0; u < TILE; ++u)
                    if (u == lane) { va = a[u]; vb = b[u]; }
                const int entry = list[base + lane];
                const float wt = wts ? wts[entry] : 1.0f;
                if (MODE == 1) reinterpret_cast<T*>(out_)[(size_t)entry * R + r] = from_f<T>(silu_f(wt * va) * (wt * vb));
                else if (MODE == 2) { const float a2 = fmaxf(wt * va, 0.f); reinterpret_cast<T*>(out_)[(size_t)entry * R + r] = from_f<T>(a2 * a2); }
                else reinterpret_cast<float*>(out_)[(size_t)entry * R + r] = wt * va;
            }
        }
    }
}

// The same experts for many rows (prompt portions): rows are grouped by expert on the host side of the step and every
// expert runs three plain GEMMs over its rows; these two kernels are what lies between them.
// mid = silu(g) * u, element by element, in float, stored as T.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ out, int64_t count)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = from_f<T>(silu_f(to_f(g[i])) * to_f(u[i]));
}

// out[slot[r]] = wts[slot[r]] * src[r]: row r of the expert-grouped result goes back to its (row, choice) place, weighted.
template <typename T>
__global__ void weighted_scatter_kernel(const T* __restrict__ src, const int* __restrict__ slot, const float* __restrict__ wts,
                                        float* __restrict__ out, int width)
{
    const int r = blockIdx.x, to = slot[r];
    const float wt = wts ? wts[to] : 1.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)to * width + i] = wt * to_f(src[(size_t)r * width + i]);
}

// ------------------------------------------------------------------------------------------------ arg-max of float rows
__global__ void argmax_kernel(const float* __restrict__ logits, int64_t ld, int vocab, int* __restrict__ out)
{
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x)
        if (row[i] > best) { best = row[i]; at = i; }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, at, o);
        if (ov > best || (ov == best && oi < at)) { best = ov; at = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = at; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < nw; ++i)
            if (bv[i] > best || (bv[i] == best && bi[i] < at)) { best = bv[i]; at = bi[i]; }
        out[blockIdx.x] = at == 0x7fffffff ? 0 : at;
    }
}

#include "window_attention.cuh"
#include "ssm.cuh"
#include "parallel_block.cuh"
#include "token_shift.cuh"

}  // namespace b200h

// ===================================================================================================== C ABI
using namespace b200h;

static thread_local const char* g_error = "";

static int fail(int code, const char* what)
{
    g_error = what;
    return code;
}

static int launched(const char* what)
{
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_error = cudaGetErrorString(e);
        (void)what;
        return (int)e;
    }
    return 0;
}

#define B200H_DISPATCH_T(dtype, ...)                                               \
    if ((dtype) == B200H_F32) { typedef float T; __VA_ARGS__; }                    \
    else if ((dtype) == B200H_BF16) { typedef bf16 T; __VA_ARGS__; }               \
    else return fail(B200H_ERR_UNSUPPORTED, "dtype: float32 (2) or bfloat16 (1)");

static Rotary make_rotary(const b200h_rotary* r)
{
    Rotary o;
    o.freqs = reinterpret_cast<const double*>(r->freqs);
    o.pairs = r->pairs;
    o.magnitude = r->magnitude;
    return o;
}

B200H_API const char* b200h_last_error(void) { return g_error; }

B200H_API int b200h_embed(const void* tokens, const void* table, float scale, void* out, int n, int width, int dtype, void* stream)
{
    if (!tokens || !table || !out || n < 0 || width <= 0) return fail(B200H_ERR_INVALID_ARG, "embed: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, embed_kernel<T><<<n, 256, 0, st>>>((const int*)tokens, (const T*)table, scale, (float*)out, width));
    return launched("embed");
}

B200H_API int b200h_causal_conv(const void* x, const void* w, void* state, int64_t slot_stride, const void* tok_seq, const void* cu_q,
                                const void* seq_slot, void* out, int n, int batch, int width, int taps, int dtype, void* stream)
{
    if (!x || !w || !state || !tok_seq || !cu_q || !seq_slot || !out || width <= 0 || batch <= 0)
        return fail(B200H_ERR_INVALID_ARG, "causal_conv: bad arguments");
    if (taps < 1 || taps > B200H_MAX_TAPS) return fail(B200H_ERR_UNSUPPORTED, "causal_conv: taps out of range");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, conv_kernel<T><<<n, 256, 0, st>>>((const float*)x, (const float*)w, (const float*)state, slot_stride,
                                                             (const int*)tok_seq, (const int*)cu_q, (const int*)seq_slot, (T*)out,
                                                             width, taps));
    if (taps > 1)
        conv_state_kernel<<<dim3((width + 127) / 128, batch), 128, 0, st>>>((const float*)x, (float*)state, slot_stride, (const int*)cu_q,
                                                                           (const int*)seq_slot, width, taps);
    return launched("causal_conv");
}

B200H_API int b200h_residual_group_norm(void* x, const void* m, int m_is_f32, int parts, const void* w, int n, int width, int groups,
                                        float eps, void* x_t, int dtype, void* stream)
{
    if (!x || !m || !w || width <= 0 || groups <= 0 || width % groups || parts < 1)
        return fail(B200H_ERR_INVALID_ARG, "residual_group_norm: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(n, groups);
    if (m_is_f32) {
        B200H_DISPATCH_T(dtype, residual_group_norm_kernel<float, T><<<grid, 256, 0, st>>>((float*)x, (const float*)m, parts, (const float*)w,
                                                                                          width, groups, eps, (T*)x_t));
    } else {
        B200H_DISPATCH_T(dtype, residual_group_norm_kernel<T, T><<<grid, 256, 0, st>>>((float*)x, (const T*)m, parts, (const float*)w, width,
                                                                                      groups, eps, (T*)x_t));
    }
    return launched("residual_group_norm");
}

B200H_API int b200h_group_norm_rows(const void* x, const void* rows, const void* w, int count, int width, int groups, float eps, void* out,
                                    int dtype, void* stream)
{
    if (!x || !w || !out || width <= 0 || groups <= 0 || width % groups) return fail(B200H_ERR_INVALID_ARG, "group_norm_rows: bad arguments");
    if (count == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, group_norm_rows_kernel<T><<<dim3(count, groups), 256, 0, st>>>((const float*)x, (const int*)rows, (const float*)w,
                                                                                          width, groups, eps, (T*)out));
    return launched("group_norm_rows");
}

B200H_API int b200h_depth_mix(void* x, void* hist, int64_t hist_stride, const void* coef, int terms, int64_t count, void* stream)
{
    if (!x || !hist || !coef || terms < 1) return fail(B200H_ERR_INVALID_ARG, "depth_mix: bad arguments");
    if (count == 0) return 0;
    depth_mix_kernel<<<(unsigned)((count + 255) / 256), 256, 0, (cudaStream_t)stream>>>((float*)x, (float*)hist, hist_stride,
                                                                                       (const float*)coef, terms, count);
    return launched("depth_mix");
}

B200H_API int b200h_latent_prep(const b200h_latent_args* a)
{
    if (!a || !a->dq || !a->dkv || !a->q_norm || !a->kv_norm || !a->cq || !a->block_ptrs || !a->tok_seq || !a->tok_pos || !a->cu_blocks)
        return fail(B200H_ERR_INVALID_ARG, "latent_prep: bad arguments");
    if (2 * a->rot.pairs > a->rot_dim) return fail(B200H_ERR_INVALID_ARG, "latent_prep: more rotated pairs than rot_dim holds");
    if (a->n == 0) return 0;
    cudaStream_t st = (cudaStream_t)a->stream;
    B200H_DISPATCH_T(a->dtype, latent_prep_kernel<T><<<a->n, 128, 0, st>>>(
        (const T*)a->dq, a->ld_dq, a->q_rank, (const float*)a->q_norm, (const T*)a->dkv, a->ld_dkv, a->kv_rank, a->rot_dim,
        (const float*)a->kv_norm, a->eps, make_rotary(&a->rot), (const int*)a->tok_seq, (const int*)a->tok_pos,
        (const int64_t*)a->block_ptrs, (const int*)a->cu_blocks, a->layer_off, a->block_len, a->rot_off, (T*)a->cq));
    return launched("latent_prep");
}

template <typename T>
static int launch_latent_attention(const b200h_latent_args* a, cudaStream_t st)
{
    const int hpb = a->heads < 8 ? a->heads : 8;
    const dim3 grid(a->n, (a->heads + hpb - 1) / hpb, a->splits), block(32, hpb);
    const size_t tile = (size_t)(kKeyTile * a->kv_rank * sizeof(T) + 15) / 16 * 16 + (size_t)kKeyTile * a->rot_dim * sizeof(float);
    const int nc = (a->kv_rank + 31) / 32, nr = (a->rot_dim + 31) / 32;
#define B200H_ATT(NC, NR)                                                                                                          \
    do {                                                                                                                           \
        if (tile > 48 * 1024)                                                                                                      \
            cudaFuncSetAttribute(latent_attention_kernel<T, NC, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile);      \
        latent_attention_kernel<T, NC, NR><<<grid, block, tile, st>>>((const float*)a->q_lat, (const float*)a->q_rot,              \
            (const float*)a->sink, a->heads, a->kv_rank, a->rot_dim, (const int*)a->tok_seq, (const int*)a->tok_pos,               \
            (const int64_t*)a->block_ptrs, (const int*)a->cu_blocks, a->layer_off, a->block_len, a->rot_off, a->splits, a->scale,  \
            (float*)a->o_lat, (float*)a->ml);                                                                                      \
    } while (0)
#define B200H_ATT_R(NC)                                    \
    if (nr <= 1) B200H_ATT(NC, 1);                         \
    else if (nr <= 2) B200H_ATT(NC, 2);                    \
    else B200H_ATT(NC, 4)
    if (nc <= 1) { B200H_ATT_R(1); }
    else if (nc <= 2) { B200H_ATT_R(2); }
    else if (nc <= 4) { B200H_ATT_R(4); }
    else if (nc <= 8) { B200H_ATT_R(8); }
    else { B200H_ATT_R(16); }
#undef B200H_ATT_R
#undef B200H_ATT
    return 0;
}

B200H_API int b200h_rotate_query(const b200h_latent_args* a)
{
    if (!a || !a->q || !a->q_rot || !a->tok_pos) return fail(B200H_ERR_INVALID_ARG, "rotate_query: bad arguments");
    if (2 * a->rot.pairs > a->rot_dim) return fail(B200H_ERR_INVALID_ARG, "rotate_query: more rotated pairs than rot_dim holds");
    if (a->n == 0) return 0;
    cudaStream_t st = (cudaStream_t)a->stream;
    B200H_DISPATCH_T(a->dtype, rotate_query_kernel<T><<<a->n, dim3(32, 8), 0, st>>>((const T*)a->q, a->ld_q, a->heads, a->dim, a->rot_dim,
                                                                                   make_rotary(&a->rot), (const int*)a->tok_pos,
                                                                                   (float*)a->q_rot));
    return launched("rotate_query");
}

B200H_API int b200h_latent_attention(const b200h_latent_args* a)
{
    if (!a || !a->sink || !a->q_lat || !a->q_rot || !a->o_lat || !a->o_heads || !a->block_ptrs || !a->tok_seq || !a->tok_pos ||
        !a->cu_blocks || !a->ml || a->splits < 1 || a->splits > 65535)
        return fail(B200H_ERR_INVALID_ARG, "latent_attention: bad arguments");
    if (a->kv_rank > 512 || a->rot_dim > 128) return fail(B200H_ERR_UNSUPPORTED, "latent_attention: kv_rank <= 512 and rot_dim <= 128");
    if (a->n == 0) return 0;
    cudaStream_t st = (cudaStream_t)a->stream;
    B200H_DISPATCH_T(a->dtype, launch_latent_attention<T>(a, st));
    B200H_DISPATCH_T(a->dtype, latent_merge_kernel<T><<<dim3(a->n, a->heads), 128, 0, st>>>((const float*)a->o_lat, (const float*)a->ml,
                                                                                           a->splits, a->n, a->heads, a->kv_rank,
                                                                                           (T*)a->o_heads));
    return launched("latent_attention");
}

B200H_API int b200h_head_gate(const void* o, const void* gate, int64_t ld_gate, int n, int heads, int vdim, void* y, int dtype, void* stream)
{
    if (!o || !gate || !y || heads <= 0 || vdim <= 0) return fail(B200H_ERR_INVALID_ARG, "head_gate: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, head_gate_kernel<T><<<n, 256, 0, st>>>((const float*)o, (const T*)gate, ld_gate, n, heads, vdim, (T*)y));
    return launched("head_gate");
}

B200H_API int b200h_decay_attention(const void* q, const void* k, const void* v, int64_t ld, const void* decay, void* state,
                                    int64_t slot_stride, const void* cu_q, const void* seq_slot, int batch, int heads, int dim, int vdim,
                                    void* out, int dtype, void* stream)
{
    if (!q || !k || !v || !decay || !state || !cu_q || !seq_slot || !out || batch <= 0 || heads <= 0)
        return fail(B200H_ERR_INVALID_ARG, "decay_attention: bad arguments");
    if (dim > 256) return fail(B200H_ERR_UNSUPPORTED, "decay_attention: dim <= 256");
    cudaStream_t st = (cudaStream_t)stream;
    const int cols = vdim < 8 ? vdim : 8;
    const dim3 grid((vdim + cols - 1) / cols, heads, batch), block(32, cols);
    const int nw = (dim + 31) / 32;
#define B200H_SCAN(NW)                                                                                                                   \
    decay_scan_kernel<T, NW><<<grid, block, 0, st>>>((const T*)q, (const T*)k, (const T*)v, ld, (const float*)decay, (float*)state,       \
                                                     slot_stride, (const int*)cu_q, (const int*)seq_slot, heads, dim, vdim, (float*)out)
    B200H_DISPATCH_T(dtype, if (nw <= 1) B200H_SCAN(1); else if (nw <= 2) B200H_SCAN(2); else if (nw <= 4) B200H_SCAN(4); else B200H_SCAN(8));
#undef B200H_SCAN
    return launched("decay_attention");
}

B200H_API int b200h_gated_rms(const void* o, const void* w, const void* gate, int64_t ld_gate, int n, int count, float eps, void* y,
                              int dtype, void* stream)
{
    if (!o || !w || !gate || !y || count <= 0) return fail(B200H_ERR_INVALID_ARG, "gated_rms: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, gated_rms_kernel<T><<<n, 256, 0, st>>>((const float*)o, (const float*)w, (const T*)gate, ld_gate, count, eps, (T*)y));
    return launched("gated_rms");
}

template <typename TI>
static void launch_route(const void* x, const void* router, int n, int width, int experts, int top, int score_fn, void* ids, void* wts,
                         size_t smem, cudaStream_t st)
{
    if (smem > 48 * 1024) cudaFuncSetAttribute(route_kernel<TI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    route_kernel<TI><<<n, 256, smem, st>>>((const TI*)x, (const float*)router, width, experts, top, score_fn, (int*)ids, (float*)wts);
}

B200H_API int b200h_route_scored(const void* x, int x_dtype, const void* router, int n, int width, int experts, int top, int score_fn,
                                 void* ids, void* wts, void* stream)
{
    if (!x || !router || !ids || !wts || experts <= 0 || top <= 0 || top > experts || score_fn < 0 || score_fn > 1)
        return fail(B200H_ERR_INVALID_ARG, "route: bad arguments");
    if (n == 0) return 0;
    const size_t smem = (size_t)(width + experts) * sizeof(float);
    if (smem > 200 * 1024) return fail(B200H_ERR_UNSUPPORTED, "route: width + experts exceeds shared memory");
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dtype == B200H_F32) launch_route<float>(x, router, n, width, experts, top, score_fn, ids, wts, smem, st);
    else if (x_dtype == B200H_BF16) launch_route<bf16>(x, router, n, width, experts, top, score_fn, ids, wts, smem, st);
    else return fail(B200H_ERR_UNSUPPORTED, "dtype: float32 (2) or bfloat16 (1)");
    return launched("route");
}

B200H_API int b200h_route(const void* x, const void* router, int n, int width, int experts, int top, void* ids, void* wts, void* stream)
{
    return b200h_route_scored(x, B200H_F32, router, n, width, experts, top, 0, ids, wts, stream);
}

template <typename T>
static void launch_expert_rows(const b200h_expert_args* a, cudaStream_t st)
{
    const int entries = a->n * a->top;
    const bool vec = a->width % Pack<T>::N == 0 && a->ff % Pack<T>::N == 0;
    const size_t sm_up = (size_t)kExpertTile * a->width * sizeof(T), sm_down = (size_t)kExpertTile * a->ff * sizeof(T);
    const dim3 g_up((a->ff + kExpertRows - 1) / kExpertRows, a->experts), g_down((a->width + kExpertRows - 1) / kExpertRows, a->experts);
    // the router's score goes to the first product when it scales the expert's input, to the last one otherwise
    const float* w_in = a->scale_input ? (const float*)a->wts : nullptr;
    const float* w_out = a->scale_input ? nullptr : (const float*)a->wts;
    // eight entries share a pass over an expert's weight rows; four where eight staged input rows would leave room for fewer than
    // three blocks per SM (the per-entry sums are the same either way)
#define B200H_ROWS_T(MODE, VEC, TILE, GRID, SM, X, DIV, WA, WB, WTS, K, R, OUT)                                                         \
    do {                                                                                                                               \
        if ((SM) > 48 * 1024)                                                                                                          \
            cudaFuncSetAttribute(expert_rows_kernel<T, MODE, VEC, TILE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SM));      \
        expert_rows_kernel<T, MODE, VEC, TILE><<<GRID, 256, SM, st>>>((const T*)(X), DIV, (const T*)(WA), (const T*)(WB),              \
                                                                     (const int*)a->counts, (const int*)a->lists, entries, WTS, K, R, OUT); \
    } while (0)
#define B200H_ROWS(MODE, VEC, GRID, SM, X, DIV, WA, WB, WTS, K, R, OUT)                                                                 \
    do {                                                                                                                               \
        if ((SM) > 72 * 1024) B200H_ROWS_T(MODE, VEC, 4, GRID, (SM) / 2, X, DIV, WA, WB, WTS, K, R, OUT);                               \
        else B200H_ROWS_T(MODE, VEC, 8, GRID, SM, X, DIV, WA, WB, WTS, K, R, OUT);                                                      \
    } while (0)
    if (a->act == 1) {
        if (vec) B200H_ROWS(2, true, g_up, sm_up, a->x, a->top, a->up, nullptr, w_in, a->width, a->ff, a->mid);
        else B200H_ROWS(2, false, g_up, sm_up, a->x, a->top, a->up, nullptr, w_in, a->width, a->ff, a->mid);
    } else {
        if (vec) B200H_ROWS(1, true, g_up, sm_up, a->x, a->top, a->gate, a->up, w_in, a->width, a->ff, a->mid);
        else B200H_ROWS(1, false, g_up, sm_up, a->x, a->top, a->gate, a->up, w_in, a->width, a->ff, a->mid);
    }
    if (vec) B200H_ROWS(0, true, g_down, sm_down, a->mid, 1, a->down, nullptr, w_out, a->ff, a->width, a->out);
    else B200H_ROWS(0, false, g_down, sm_down, a->mid, 1, a->down, nullptr, w_out, a->ff, a->width, a->out);
#undef B200H_ROWS
#undef B200H_ROWS_T
}

B200H_API int b200h_experts(const b200h_expert_args* a)
{
    if (!a || !a->x || !a->up || !a->down || !a->ids || !a->wts || !a->out || !a->mid || !a->counts || !a->lists ||
        a->ff <= 0 || a->experts <= 0 || a->top <= 0 || a->act < 0 || a->act > 1 || (a->act == 0 && !a->gate))
        return fail(B200H_ERR_INVALID_ARG, "experts: bad arguments");
    if (a->n == 0) return 0;
    const size_t widest = (size_t)kExpertTile * (a->width > a->ff ? a->width : a->ff) * (a->dtype == B200H_F32 ? 4 : 2);
    if (widest / 2 > 200 * 1024) return fail(B200H_ERR_UNSUPPORTED, "experts: four rows of width / ff exceed shared memory");
    if ((size_t)a->experts * sizeof(int) > 48 * 1024) return fail(B200H_ERR_UNSUPPORTED, "experts: more than 12288 experts");
    cudaStream_t st = (cudaStream_t)a->stream;
    expert_lists_kernel<<<1, 1024, a->experts * sizeof(int), st>>>((const int*)a->ids, a->n * a->top, a->experts, (int*)a->counts,
                                                                  (int*)a->lists);
    B200H_DISPATCH_T(a->dtype, launch_expert_rows<T>(a, st));
    return launched("experts");
}

B200H_API int b200h_silu_mul(const void* g, const void* u, void* out, int64_t count, int dtype, void* stream)
{
    if (!g || !u || !out || count < 0) return fail(B200H_ERR_INVALID_ARG, "silu_mul: bad arguments");
    if (count == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, silu_mul_kernel<T><<<(unsigned)((count + 255) / 256), 256, 0, st>>>((const T*)g, (const T*)u, (T*)out, count));
    return launched("silu_mul");
}

B200H_API int b200h_weighted_scatter(const void* src, const void* slot, const void* wts, void* out, int rows, int width, int dtype,
                                     void* stream)
{
    if (!src || !slot || !out || width <= 0) return fail(B200H_ERR_INVALID_ARG, "weighted_scatter: bad arguments");
    if (rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, weighted_scatter_kernel<T><<<rows, 256, 0, st>>>((const T*)src, (const int*)slot, (const float*)wts, (float*)out,
                                                                           width));
    return launched("weighted_scatter");
}

B200H_API int b200h_argmax(const void* logits, int64_t ld, int rows, int vocab, void* out, void* stream)
{
    if (!logits || !out || vocab <= 0) return fail(B200H_ERR_INVALID_ARG, "argmax: bad arguments");
    if (rows == 0) return 0;
    argmax_kernel<<<rows, 1024, 0, (cudaStream_t)stream>>>((const float*)logits, ld, vocab, (int*)out);
    return launched("argmax");
}


// ------------------------------------------------------------------------------------------------ pre-norm blocks
B200H_API int b200h_add_rows(void* x, const void* table, const void* idx, int fixed, int n, int width, int dtype, void* stream)
{
    if (!x || !table || n < 0 || width <= 0 || (!idx && fixed < 0)) return fail(B200H_ERR_INVALID_ARG, "add_rows: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, add_rows_kernel<T><<<n, 256, 0, st>>>((float*)x, (const T*)table, (const int*)idx, fixed, width));
    return launched("add_rows");
}

B200H_API int b200h_residual_norm(void* x, const void* m, const void* extra, const void* w, int n, int width, float eps, void* h,
                                  int dtype, void* stream)
{
    if (!x || n < 0 || width <= 0 || (h && !w)) return fail(B200H_ERR_INVALID_ARG, "residual_norm: bad arguments");
    if (n == 0 || (!m && !extra && !h)) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, residual_norm_kernel<T><<<n, 256, 0, st>>>((float*)x, (const T*)m, (const T*)extra, (const float*)w, width, eps,
                                                                      (float*)h));
    return launched("residual_norm");
}

B200H_API int b200h_relu2(void* x, int64_t count, int dtype, void* stream)
{
    if (!x || count < 0) return fail(B200H_ERR_INVALID_ARG, "relu2: bad arguments");
    if (count == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, relu2_kernel<T><<<(unsigned)((count + 255) / 256), 256, 0, st>>>((T*)x, count));
    return launched("relu2");
}

static int window_args_ok(const b200h_window_args* a, const char** why)
{
    if (!a || !a->tok_seq || !a->tok_pos || !a->block_ptrs || !a->cu_blocks || !a->qn) { *why = "window attention: bad arguments"; return 0; }
    if (a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads || a->dim <= 0 || a->vdim <= 0 || a->block_len <= 0 || a->window < 0 ||
        a->chunk < 0 || (a->talk_scores && !a->talk)) {
        *why = "window attention: heads must be a multiple of kv_heads, sizes positive";
        return 0;
    }
    return 1;
}

B200H_API int b200h_window_prep(const b200h_window_args* a)
{
    const char* why = "";
    if (!window_args_ok(a, &why)) return fail(B200H_ERR_INVALID_ARG, why);
    if (!a->q || !a->k || !a->v) return fail(B200H_ERR_INVALID_ARG, "window_prep: bad arguments");
    if (a->n == 0) return 0;
    cudaStream_t st = (cudaStream_t)a->stream;
    B200H_DISPATCH_T(a->dtype, window_prep_kernel<T><<<a->n, 256, 0, st>>>(
        (const T*)a->q, (const T*)a->k, (const T*)a->v, a->ld, a->heads * a->dim, a->kv_heads * a->dim, a->kv_heads * a->vdim,
        (const float*)a->bias, (const float*)a->q_norm, (const float*)a->k_norm, a->eps, (const int*)a->tok_seq, (const int*)a->tok_pos,
        (const int64_t*)a->block_ptrs, (const int*)a->cu_blocks, a->layer_off, a->v_off, a->block_len, (float*)a->qn));
    return launched("window_prep");
}

B200H_API int b200h_head_rope_prep(const b200h_window_args* a, const b200h_rotary* r)
{
    const char* why = "";
    if (!window_args_ok(a, &why)) return fail(B200H_ERR_INVALID_ARG, why);
    if (!a->q || !a->k || !a->v || !r || r->pairs < 0 || 2 * r->pairs > a->dim || (r->pairs && !r->freqs))
        return fail(B200H_ERR_INVALID_ARG, "head_rope_prep: bad arguments (2 * rot.pairs <= dim)");
    if (a->n == 0) return 0;
    cudaStream_t st = (cudaStream_t)a->stream;
    const Rotary rot = make_rotary(r);
    const size_t smem = ((size_t)(a->heads + a->kv_heads) * a->dim + 2 * (size_t)rot.pairs) * sizeof(float);
    if (smem > 200 * 1024) return fail(B200H_ERR_UNSUPPORTED, "head_rope_prep: (heads + kv_heads) * dim floats exceed an SM's shared memory");
    B200H_DISPATCH_T(a->dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(head_rope_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        head_rope_prep_kernel<T><<<a->n, 256, smem, st>>>(
            (const T*)a->q, (const T*)a->k, (const T*)a->v, a->ld, a->heads, a->kv_heads, a->dim, a->vdim, (const float*)a->bias,
            (const float*)a->q_norm, (const float*)a->k_norm, a->eps, rot, (const int*)a->tok_seq, (const int*)a->tok_pos,
            (const int64_t*)a->block_ptrs, (const int*)a->cu_blocks, a->layer_off, a->v_off, a->block_len, (float*)a->qn);
    });
    return launched("head_rope_prep");
}

static size_t window_pv_smem(const b200h_window_args* a, int rows, int tile)
{
    const size_t H = a->heads, rh = (size_t)rows * H;
    auto pad4 = [](size_t v) { return (v + 3) & ~(size_t)3; };
    const bool talk = a->talk && !a->talk_scores;           // pass 2 recombines weights only when the scores were not mixed before it
    return (size_t)tile * sizeof(char*) + sizeof(float) * (2 * pad4(rh) + (talk ? pad4(H * H) : 0) + (size_t)(talk ? 2 : 1) * rh * tile + rh * a->vdim);
}

struct WindowLaunch {
    int blocks, stats_threads;
    size_t stats_smem, pv_smem;
};

template <typename T, bool VEC, int CW, int NP>
static void launch_window_kernels(const b200h_window_args* a, const WindowGeom& g, const WindowLaunch& l, cudaStream_t st)
{
    if (l.stats_smem > 48 * 1024)
        cudaFuncSetAttribute(window_stats_kernel<T, VEC, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)l.stats_smem);
    if (l.pv_smem > 48 * 1024)
        cudaFuncSetAttribute(window_pv_kernel<T, CW, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)l.pv_smem);
    window_stats_kernel<T, VEC, NP><<<dim3(l.blocks, a->kv_heads, a->splits), l.stats_threads, l.stats_smem, st>>>((const float*)a->qn, g,
                                                                                                                   (float*)a->ml);
    if (a->talk_scores) {
        // between the passes: the scores of all heads of a row are mixed in place and their maxima and denominators recomputed
        const int H = a->heads;
        int tile = 128;
        while (tile > 8 && (size_t)H * (H + tile) * sizeof(float) > 96 * 1024) tile /= 2;
        const size_t smem = (size_t)H * (H + tile) * sizeof(float);
        if (smem > 48 * 1024) cudaFuncSetAttribute(window_mix_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        window_mix_scores_kernel<<<dim3(a->n, g.rows == 1 ? a->splits : 1), 256, smem, st>>>(g, (const float*)a->talk, tile, (float*)a->ml);
    }
    window_pv_kernel<T, CW, NP><<<dim3(l.blocks, a->splits), 256, l.pv_smem, st>>>(g, (const float*)a->ml, (float*)a->o_part);
}

template <typename T, bool VEC, int CW>
static int launch_window_attention(const b200h_window_args* a, WindowGeom g, cudaStream_t st)
{
    const int H = a->heads, rep = H / a->kv_heads;
    // Rows per block: four for prompt portions (one key range per row), one when the keys of a row are cut into ranges; 64 keys per
    // tile of pass 2.  Both shrink until a block fits half an SM's shared memory.
    const size_t budget = 100 * 1024;
    g.rows = (a->splits == 1 && a->n >= 4) ? 4 : 1;
    g.tile = 64;
    while (window_pv_smem(a, g.rows, g.tile) > budget && g.tile > 32) g.tile /= 2;
    while (window_pv_smem(a, g.rows, g.tile) > budget && g.rows > 1) g.rows /= 2;
    WindowLaunch l;
    // pass 1: a thread per key of the range, at most 128
    const int span = a->window > 0 && a->chunk > 0 ? (a->window < a->chunk ? a->window : a->chunk) : (a->window > 0 ? a->window : a->chunk);
    const int keys = span > 0 ? span + g.rows - 1 : 1 << 30, per = (keys + a->splits - 1) / a->splits;
    l.stats_threads = per <= 32 ? 32 : (per <= 64 ? 64 : 128);
    l.stats_smem = (size_t)g.rows * rep * a->dim * sizeof(float) + (VEC ? (size_t)l.stats_threads * (a->dim * sizeof(T) + 16) : 0);
    l.pv_smem = window_pv_smem(a, g.rows, g.tile);
    if (l.stats_smem > 200 * 1024 || l.pv_smem > 200 * 1024)
        return fail(B200H_ERR_UNSUPPORTED, "window_attention: heads * (dim + vdim + heads) floats exceed an SM's shared memory");
    l.blocks = (a->n + g.rows - 1) / g.rows;
    const int pairs = g.rows * rep;              // (row, head) pairs that share a key: walked NP at a time
    if (pairs <= 2) launch_window_kernels<T, VEC, CW, 2>(a, g, l, st);
    else if (pairs <= 4) launch_window_kernels<T, VEC, CW, 4>(a, g, l, st);
    else launch_window_kernels<T, VEC, CW, 8>(a, g, l, st);
    window_out_kernel<T><<<dim3(a->n, (H * a->vdim + 255) / 256), 256, 0, st>>>((const float*)a->o_part, a->splits, H * a->vdim, (const T*)a->gate,
                                                                                a->ld_gate, a->gate_heads ? a->vdim : 1, (T*)a->y);
    return 0;
}

B200H_API int b200h_window_attention(const b200h_window_args* a)
{
    const char* why = "";
    if (!window_args_ok(a, &why)) return fail(B200H_ERR_INVALID_ARG, why);
    if (!a->scores || a->score_ld < 1) return fail(B200H_ERR_INVALID_ARG, "window_attention: no score scratch");
    if (!a->ml || !a->o_part || !a->y || a->splits < 1 || a->splits > 65535 || a->kv_heads > 65535 || (a->r1 && !a->r2))
        return fail(B200H_ERR_INVALID_ARG, "window_attention: bad arguments");
    if (a->n == 0) return 0;
    WindowGeom g;
    g.n = a->n; g.rows = 1; g.tile = 32;
    g.heads = a->heads; g.kv_heads = a->kv_heads; g.dim = a->dim; g.vdim = a->vdim; g.block_len = a->block_len;
    g.window = a->window; g.splits = a->splits; g.scale = a->scale; g.softcap = a->softcap; g.chunk = a->chunk;
    // talk mixes the softmax WEIGHTS inside pass 2, or (talk_scores) the SCORES between the passes: pass 2 then sees no talk
    g.r1 = (const float*)a->r1; g.r2 = (const float*)a->r2; g.talk = a->talk_scores ? nullptr : (const float*)a->talk;
    g.sink = (const float*)a->sink;
    g.tok_seq = (const int*)a->tok_seq; g.tok_pos = (const int*)a->tok_pos;
    g.block_ptrs = (const int64_t*)a->block_ptrs; g.cu_blocks = (const int*)a->cu_blocks;
    g.layer_off = a->layer_off; g.v_off = a->v_off;
    g.scores = (float*)a->scores; g.score_ld = (int)a->score_ld;
    cudaStream_t st = (cudaStream_t)a->stream;
    const size_t esize = a->dtype == B200H_F32 ? 4 : 2;
    // 16-byte key reads / four value columns per read where sizes and offsets keep every read aligned
    const bool vec = (a->dim * esize) % 16 == 0 && a->layer_off % 16 == 0;
    const bool vec_v = a->vdim % 4 == 0 && a->layer_off % 16 == 0 && a->v_off % 16 == 0;
    int rc = 0;
    if (vec && vec_v) { B200H_DISPATCH_T(a->dtype, rc = (launch_window_attention<T, true, 4>(a, g, st))); }
    else if (vec) { B200H_DISPATCH_T(a->dtype, rc = (launch_window_attention<T, true, 1>(a, g, st))); }
    else if (vec_v) { B200H_DISPATCH_T(a->dtype, rc = (launch_window_attention<T, false, 4>(a, g, st))); }
    else { B200H_DISPATCH_T(a->dtype, rc = (launch_window_attention<T, false, 1>(a, g, st))); }
    if (rc) return rc;
    return launched("window_attention");
}


// ------------------------------------------------------------------------------------------------ parallel blocks, state-space mixer
B200H_API int b200h_parallel_residual_norm(void* x, const void* mix, const void* ff, int parts, float mult, const void* add, const void* extra,
                                           const void* w1, const void* w2, int n, int width, float eps, void* h1, void* h2, void* h2f,
                                           int dtype, void* stream)
{
    if (!x || n < 0 || width <= 0 || (h1 && !w1) || ((h2 || h2f) && !w2) || (h2f && !h2) || (ff && parts < 1))
        return fail(B200H_ERR_INVALID_ARG, "parallel_residual_norm: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, parallel_residual_norm_kernel<T><<<n, 256, 0, st>>>((float*)x, (const T*)mix, (const float*)ff, ff ? parts : 0, mult,
                                                                               (const float*)add, (const T*)extra, (const float*)w1,
                                                                               (const float*)w2, width, eps, (T*)h1, (T*)h2, (float*)h2f));
    return launched("parallel_residual_norm");
}

B200H_API int b200h_short_conv(const void* u, int64_t ld, const void* w, const void* bias, int act, void* state, int64_t slot_stride,
                               const void* tok_seq, const void* cu_q, const void* seq_slot, void* out, int n, int batch, int channels,
                               int taps, int dtype, void* stream)
{
    if (!u || !w || !state || !tok_seq || !cu_q || !seq_slot || !out || channels <= 0 || batch <= 0 || act < 0 || act > 1)
        return fail(B200H_ERR_INVALID_ARG, "short_conv: bad arguments");
    if (taps < 1 || taps > B200H_MAX_TAPS) return fail(B200H_ERR_UNSUPPORTED, "short_conv: taps 1..16");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(n, (channels + 1023) / 1024), sgrid((channels + 255) / 256, batch);
    B200H_DISPATCH_T(dtype, {
        short_conv_kernel<T><<<grid, 256, 0, st>>>((const T*)u, ld, (const float*)w, (const float*)bias, act, (const float*)state, slot_stride,
                                                   (const int*)tok_seq, (const int*)cu_q, (const int*)seq_slot, (float*)out, channels, taps);
        if (taps > 1)
            short_conv_state_kernel<T><<<sgrid, 256, 0, st>>>((const T*)u, ld, (float*)state, slot_stride, (const int*)cu_q, (const int*)seq_slot,
                                                            channels, taps);
    });
    return launched("short_conv");
}

B200H_API int b200h_ssm_scan(const void* xbc, const void* dt, int64_t ld_dt, const void* dt_bias, const void* a_log, const void* skip,
                             void* state, int64_t slot_stride, const void* cu_q, const void* seq_slot, int n, int batch, int heads, int vdim,
                             int nstate, int groups, void* steps, void* out, int dtype, void* stream)
{
    if (!xbc || !dt || !dt_bias || !a_log || !skip || !state || !cu_q || !seq_slot || !steps || !out || n < 0 || batch <= 0 || heads <= 0 ||
        vdim <= 0 || nstate <= 0 || groups <= 0 || heads % groups)
        return fail(B200H_ERR_INVALID_ARG, "ssm_scan: bad arguments");
    if (nstate > 256) return fail(B200H_ERR_UNSUPPORTED, "ssm_scan: state <= 256");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t count = (int64_t)n * heads;
    B200H_DISPATCH_T(dtype, ssm_steps_kernel<T><<<(unsigned)((count + 255) / 256), 256, 0, st>>>((const T*)dt, ld_dt, (const float*)dt_bias,
                                                                                               (const float*)a_log, heads, count, (float2*)steps));
    // two value columns per warp where the head has an even number of them (B and C are read once for both)
    const int nc = vdim % 2 == 0 ? 2 : 1, units = vdim / nc, warps = units < 8 ? units : 8;
    const dim3 grid((units + warps - 1) / warps, heads, batch), block(32, warps);
    const int nw = (nstate + 31) / 32;
#define B200H_SCAN(NW, NC)                                                                                                               \
    ssm_scan_kernel<NW, NC><<<grid, block, 0, st>>>((const float*)xbc, (const float2*)steps, (const float*)skip, (float*)state, slot_stride, \
                                                    (const int*)cu_q, (const int*)seq_slot, heads, vdim, nstate, groups, (float*)out)
#define B200H_SCAN_NW(NC) \
    do { if (nw <= 1) B200H_SCAN(1, NC); else if (nw <= 2) B200H_SCAN(2, NC); else if (nw <= 4) B200H_SCAN(4, NC); else B200H_SCAN(8, NC); } while (0)
    if (nc == 2) B200H_SCAN_NW(2); else B200H_SCAN_NW(1);
#undef B200H_SCAN_NW
#undef B200H_SCAN
    return launched("ssm_scan");
}

B200H_API int b200h_gate_group_norm(const void* y, const void* gate, int64_t ld_gate, const void* w, int n, int count, int groups, float eps,
                                    void* out, int dtype, void* stream)
{
    if (!y || !gate || !w || !out || count <= 0 || groups <= 0 || count % groups) return fail(B200H_ERR_INVALID_ARG, "gate_group_norm: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, gate_group_norm_kernel<T><<<dim3(n, groups), 256, 0, st>>>((const float*)y, (const T*)gate, ld_gate, (const float*)w,
                                                                                      count, groups, eps, (T*)out));
    return launched("gate_group_norm");
}

B200H_API int b200h_conv_rope_prep(const b200h_conv_prep_args* a)
{
    if (!a || !a->qk || !a->conv || !a->state || !a->qn || !a->tok_seq || !a->tok_pos || !a->cu_q || !a->seq_slot || !a->block_ptrs ||
        !a->cu_blocks || a->heads <= 0 || a->kv_heads <= 0 || a->dim <= 0 || a->block_len <= 0 || a->batch <= 0)
        return fail(B200H_ERR_INVALID_ARG, "conv_rope_prep: bad arguments");
    if (a->taps < 1 || a->taps > B200H_MAX_TAPS) return fail(B200H_ERR_UNSUPPORTED, "conv_rope_prep: taps 1..16");
    if (a->rot.pairs < 0 || 2 * a->rot.pairs > a->dim || (a->rot.pairs && !a->rot.freqs))
        return fail(B200H_ERR_INVALID_ARG, "conv_rope_prep: rotated pairs do not fit a head");
    if (a->n == 0) return 0;
    const int channels = (a->heads + a->kv_heads) * a->dim;
    const size_t smem = (size_t)(channels + 2 * a->rot.pairs) * sizeof(float);
    if (smem > 200 * 1024) return fail(B200H_ERR_UNSUPPORTED, "conv_rope_prep: (heads + kv_heads) * dim floats exceed shared memory");
    cudaStream_t st = (cudaStream_t)a->stream;
    const Rotary rot = make_rotary(&a->rot);
    const dim3 sgrid((channels + 255) / 256, a->batch);
    B200H_DISPATCH_T(a->dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(conv_rope_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        conv_rope_prep_kernel<T><<<a->n, 256, smem, st>>>((const T*)a->qk, a->ld, (const float*)a->conv, a->taps, (const float*)a->state,
                                                          a->slot_stride, (const int*)a->tok_seq, (const int*)a->tok_pos, (const int*)a->cu_q,
                                                          (const int*)a->seq_slot, rot, a->heads, a->kv_heads, a->dim, a->eps,
                                                          (const int64_t*)a->block_ptrs, (const int*)a->cu_blocks, a->layer_off, a->v_off,
                                                          a->block_len, (float*)a->qn);
        if (a->taps > 1)
            short_conv_state_kernel<T><<<sgrid, 256, 0, st>>>((const T*)a->qk, a->ld, (float*)a->state, a->slot_stride, (const int*)a->cu_q,
                                                            (const int*)a->seq_slot, channels, a->taps);
    });
    return launched("conv_rope_prep");
}

B200H_API int b200h_softcap(void* x, int64_t count, float cap, void* stream)
{
    if (!x || count < 0 || !(cap > 0.f)) return fail(B200H_ERR_INVALID_ARG, "softcap: bad arguments");
    if (count == 0) return 0;
    softcap_kernel<<<(unsigned)((count + 255) / 256), 256, 0, (cudaStream_t)stream>>>((float*)x, count, cap);
    return launched("softcap");
}

B200H_API int b200h_scaled_relu2(void* u, const void* scale, int rows, int cols, int dtype, void* stream)
{
    if (!u || rows < 0 || cols <= 0) return fail(B200H_ERR_INVALID_ARG, "scaled_relu2: bad arguments");
    if (rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t count = (int64_t)rows * cols;
    B200H_DISPATCH_T(dtype, scaled_relu2_kernel<T><<<(unsigned)((count + 255) / 256), 256, 0, st>>>((T*)u, (const float*)scale, cols, count));
    return launched("scaled_relu2");
}

// ------------------------------------------------------------------------------------------------ one-norm parallel blocks, token shift
B200H_API int b200h_embed_hashed(const void* tokens, const void* table, const void* second, int buckets, int mul_prev, int mul_cur, void* prev,
                                 int64_t slot_stride, const void* tok_seq, const void* tok_pos, const void* cu_q, const void* seq_slot,
                                 void* out, int n, int batch, int width, int dtype, void* stream)
{
    if (!tokens || !table || !second || !prev || !tok_seq || !tok_pos || !cu_q || !seq_slot || !out || n < 0 || batch <= 0 || width <= 0 ||
        buckets <= 0)
        return fail(B200H_ERR_INVALID_ARG, "embed_hashed: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, embed_hashed_kernel<T><<<n, 256, 0, st>>>((const int*)tokens, (const T*)table, (const T*)second, buckets, mul_prev,
                                                                     mul_cur, (const float*)prev, slot_stride, (const int*)tok_seq,
                                                                     (const int*)tok_pos, (const int*)cu_q, (const int*)seq_slot, (float*)out,
                                                                     width));
    last_token_kernel<<<(batch + 127) / 128, 128, 0, st>>>((const int*)tokens, (float*)prev, slot_stride, (const int*)cu_q, (const int*)seq_slot,
                                                         batch);
    return launched("embed_hashed");
}

B200H_API int b200h_branch_residual_norm(void* x, const void* left, const void* right, const void* wl, const void* wr, float branch_scale,
                                         const void* ff, int ff_is_f32, int parts, const void* w, int n, int width, float eps, void* h,
                                         void* hf, int dtype, void* stream)
{
    if (!x || n < 0 || width <= 0 || (!left != !right) || (left && (!wl || !wr)) || (ff && parts < 1) || ((h || hf) && !w))
        return fail(B200H_ERR_INVALID_ARG, "branch_residual_norm: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
#define B200H_JOIN(TF)                                                                                                                     \
    branch_residual_norm_kernel<T, TF><<<n, 256, 0, st>>>((float*)x, (const T*)left, (const T*)right, (const float*)wl, (const float*)wr,   \
                                                          branch_scale, (const TF*)ff, ff ? parts : 0, (const float*)w, width, eps, (T*)h,  \
                                                          (float*)hf)
    B200H_DISPATCH_T(dtype, if (ff_is_f32) B200H_JOIN(float); else B200H_JOIN(T));
#undef B200H_JOIN
    return launched("branch_residual_norm");
}

B200H_API int b200h_token_shift(const void* h, const void* shift, const void* mu, int nmu, void* state, int64_t slot_stride,
                                const void* tok_seq, const void* cu_q, const void* seq_slot, int n, int batch, int width, void* a,
                                void* blends, int dtype, void* stream)
{
    if (!h || !state || !tok_seq || !cu_q || !seq_slot || n < 0 || batch <= 0 || width <= 0 || nmu < 0 || (nmu && (!mu || !blends)))
        return fail(B200H_ERR_INVALID_ARG, "token_shift: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, token_shift_kernel<T><<<n, 256, 0, st>>>((const float*)h, (const float*)shift, (const float*)mu, nmu,
                                                                    (const float*)state, slot_stride, (const int*)tok_seq, (const int*)cu_q,
                                                                    (const int*)seq_slot, n, width, (T*)a, (T*)blends));
    token_shift_state_kernel<<<dim3((width + 255) / 256, batch), 256, 0, st>>>((const float*)h, (const float*)shift, (float*)state, slot_stride,
                                                                             (const int*)cu_q, (const int*)seq_slot, width);
    return launched("token_shift");
}

B200H_API int b200h_channel_decay_scan(const void* r, const void* k, const void* v, int64_t ld, const void* d, const void* w0,
                                       const void* bonus, void* state, int64_t slot_stride, const void* cu_q, const void* seq_slot, int n,
                                       int batch, int heads, int dim, int vdim, void* decay, void* out, int dtype, void* stream)
{
    if (!r || !k || !v || !d || !w0 || !bonus || !state || !cu_q || !seq_slot || !decay || !out || n < 0 || batch <= 0 || heads <= 0 ||
        dim <= 0 || vdim <= 0)
        return fail(B200H_ERR_INVALID_ARG, "channel_decay_scan: bad arguments");
    if (dim > 256) return fail(B200H_ERR_UNSUPPORTED, "channel_decay_scan: dim <= 256");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t count = (int64_t)n * heads * dim;
    channel_decay_kernel<<<(unsigned)((count + 255) / 256), 256, 0, st>>>((const float*)d, (const float*)w0, heads * dim, count, (float*)decay);
    // a block per (sequence, head, 32 value columns), a warp per 16 key channels
    const int groups = (vdim + 31) / 32, kw = (dim + 15) / 16;
    const dim3 grid(heads * groups, batch), block(32, kw);
    const size_t smem = (size_t)kw * (3 * 4 * 16 + 2 * 4 * 32) * sizeof(float);
    B200H_DISPATCH_T(dtype, (channel_decay_scan_kernel<T, 4><<<grid, block, smem, st>>>(
        (const T*)r, (const T*)k, (const T*)v, ld, (const float*)decay, (const float*)bonus, (float*)state, slot_stride, (const int*)cu_q,
        (const int*)seq_slot, heads, dim, vdim, (float*)out)));
    return launched("channel_decay_scan");
}

B200H_API int b200h_group_norm_gate(const void* o, const void* w, const void* gate, int64_t ld_gate, int n, int count, int groups, int act,
                                    float eps, void* y, int dtype, void* stream)
{
    if (!o || !w || !gate || !y || count <= 0 || groups <= 0 || count % groups || act < 0 || act > 1)
        return fail(B200H_ERR_INVALID_ARG, "group_norm_gate: bad arguments");
    if (n == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int gw = count / groups;
#define B200H_GNG(NV)                                                                                                                      \
    group_norm_gate_warp_kernel<T, NV><<<n, groups >= 8 ? 256 : 32 * groups, 0, st>>>((const float*)o, (const float*)w, (const T*)gate, ld_gate, \
                                                                                     count, groups, act, eps, (T*)y)
    if (gw <= 256) {            // a warp per group
        B200H_DISPATCH_T(dtype, if (gw <= 32) B200H_GNG(1); else if (gw <= 64) B200H_GNG(2); else if (gw <= 128) B200H_GNG(4); else B200H_GNG(8));
        return launched("group_norm_gate");
    }
#undef B200H_GNG
    B200H_DISPATCH_T(dtype, group_norm_gate_kernel<T><<<dim3(n, groups), 128, 0, st>>>((const float*)o, (const float*)w, (const T*)gate, ld_gate,
                                                                                      count, groups, act, eps, (T*)y));
    return launched("group_norm_gate");
}

B200H_API int b200h_xielu(void* x, int64_t count, const void* params, int dtype, void* stream)
{
    if (!x || !params || count < 0) return fail(B200H_ERR_INVALID_ARG, "xielu: bad arguments");
    if (count == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, xielu_kernel<T><<<(unsigned)((count + 255) / 256), 256, 0, st>>>((T*)x, count, (const float*)params));
    return launched("xielu");
}

B200H_API int b200h_tanh(void* x, int64_t count, int dtype, void* stream)
{
    if (!x || count < 0) return fail(B200H_ERR_INVALID_ARG, "tanh: bad arguments");
    if (count == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    B200H_DISPATCH_T(dtype, tanh_kernel<T><<<(unsigned)((count + 255) / 256), 256, 0, st>>>((T*)x, count));
    return launched("tanh");
}

template <typename TI>
static void launch_route_grouped(const void* x, const void* router, const void* correction, int n, int width, int experts, int top, int groups,
                                 int keep, int group_top, int renorm, float scale, void* ids, void* wts, size_t smem, cudaStream_t st)
{
    if (smem > 48 * 1024) cudaFuncSetAttribute(route_grouped_kernel<TI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    route_grouped_kernel<TI><<<n, 256, smem, st>>>((const TI*)x, (const float*)router, (const float*)correction, width, experts, top, groups, keep,
                                                  group_top, renorm, scale, (int*)ids, (float*)wts);
}

B200H_API int b200h_route_grouped(const void* x, int x_dtype, const void* router, const void* correction, int n, int width, int experts,
                                  int top, int groups, int keep, int group_top, int renorm, float scale, void* ids, void* wts, void* stream)
{
    if (!x || !router || !ids || !wts || experts <= 0 || top <= 0 || groups <= 0 || experts % groups || keep < 1 || keep > groups ||
        group_top < 1 || top > keep * (experts / groups))
        return fail(B200H_ERR_INVALID_ARG, "route_grouped: bad arguments (equal groups, top within the kept groups)");
    if (n == 0) return 0;
    const size_t smem = (size_t)(width + 2 * experts + groups) * sizeof(float);
    if (smem > 200 * 1024) return fail(B200H_ERR_UNSUPPORTED, "route_grouped: width + experts exceeds shared memory");
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dtype == B200H_F32)
        launch_route_grouped<float>(x, router, correction, n, width, experts, top, groups, keep, group_top, renorm, scale, ids, wts, smem, st);
    else if (x_dtype == B200H_BF16)
        launch_route_grouped<bf16>(x, router, correction, n, width, experts, top, groups, keep, group_top, renorm, scale, ids, wts, smem, st);
    else return fail(B200H_ERR_UNSUPPORTED, "dtype: float32 (2) or bfloat16 (1)");
    return launched("route_grouped");
}
