// Operators of hybrid (attention + recurrent) decoder models on mixed batches — include/atoma_hybrid.h.
//
// What is float32 whatever the activation format: the residual stream, every norm's statistics, attention
// scores and weights, the recurrent state with its gates, positions and angles (double here).  Reductions
// run in an order that depends only on the row and the launch geometry — never on what else is in the
// batch or on how a prompt was cut — so a position's result is reproducible across schedules.
//
// This file holds the row-wise operators, the general (any shape, any format) attention and scan
// kernels and the plain float32 GEMM; hybrid_attention.cu holds the tensor-core prefill and the split
// decode attention kernels.
#include "common.cuh"
#include "hybrid_common.cuh"

#include "atoma_hybrid.h"
#include "atoma_llama.h"

#include <algorithm>

namespace atoma {

int g_hybrid_debug = 0;
bool hyb_attn_split_reduce(const float *partial, void *out, int64_t T, int splits, int64_t n, uint32_t dtype, cudaStream_t stream);

namespace {

using namespace hybrid;

// ---------------------------------------------------------------------------------------------
// embedding + sinusoidal position signal
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) embed_sinusoid_kernel(const uint32_t *__restrict__ tokens,
                                                             const int64_t *__restrict__ positions,
                                                             const T *__restrict__ table, const double *__restrict__ inv_freq,
                                                             float *__restrict__ out, int width, int64_t vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int64_t tok = tokens[t];
    if (tok >= vocab) tok = vocab - 1;
    const double p = static_cast<double>(positions[t]);
    const T *row = table + tok * width;
    float *o = out + static_cast<int64_t>(t) * width;
    for (int i = threadIdx.x; 2 * i < width; i += blockDim.x) {
        double s, c;
        sincos(p * inv_freq[i], &s, &c);
        o[2 * i] = to_f(row[2 * i]) + static_cast<float>(s);
        if (2 * i + 1 < width) o[2 * i + 1] = to_f(row[2 * i + 1]) + static_cast<float>(c);
    }
}

// ---------------------------------------------------------------------------------------------
// norms
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kRowThreads) rmsnorm_rows_kernel(const float *__restrict__ x, const int32_t *__restrict__ rows,
                                                                   const float *__restrict__ weight, float offset,
                                                                   T *__restrict__ out, int width, float eps) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float *xr = x + static_cast<int64_t>(rows ? rows[r] : r) * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(width) + eps);
    T *o = out + static_cast<int64_t>(r) * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_f<T>(xr[c] * inv * (offset + weight[c]));
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads) postnorm_add_prenorm_kernel(const T *__restrict__ y, float *__restrict__ x,
                                                                           const float *__restrict__ w_post,
                                                                           const float *__restrict__ w_pre, T *__restrict__ h,
                                                                           int width, float eps, float offset) {
    extern __shared__ float row[];
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t base = static_cast<int64_t>(blockIdx.x) * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = to_f(y[base + c]);
        row[c] = v;
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(width) + eps);
    float s2 = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = x[base + c] + row[c] * inv * (offset + w_post[c]);
        x[base + c] = v;
        row[c] = v;
        s2 = fmaf(v, v, s2);
    }
    if (!w_pre) return;
    const float inv2 = 1.0f / sqrtf(block_sum(s2, red) / static_cast<float>(width) + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) h[base + c] = from_f<T>(row[c] * inv2 * (offset + w_pre[c]));
}

// ---------------------------------------------------------------------------------------------
// q/k norm over the whole projection + query temperature + cache write
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kRowThreads) qk_norm_cache_kernel(const T *__restrict__ qkv, const float *__restrict__ bias,
                                                                    const float *__restrict__ q_w, const float *__restrict__ k_w,
                                                                    const int64_t *__restrict__ positions,
                                                                    const int64_t *__restrict__ slots, T *__restrict__ q_out,
                                                                    T *__restrict__ k_cache, T *__restrict__ v_cache, int nq,
                                                                    int nk, int nv, float eps, float temp_coef, int64_t temp_every) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T *r = qkv + static_cast<int64_t>(t) * (nq + nk + nv);
    float sq = 0.f, sk = 0.f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) {
        const float v = to_f(r[c]) + (bias ? bias[c] : 0.f);
        sq = fmaf(v, v, sq);
    }
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
        const float v = to_f(r[nq + c]) + (bias ? bias[nq + c] : 0.f);
        sk = fmaf(v, v, sk);
    }
    const float iq = 1.0f / sqrtf(block_sum(sq, red) / static_cast<float>(nq) + eps);
    const float ik = 1.0f / sqrtf(block_sum(sk, red) / static_cast<float>(nk) + eps);
    float temp = 1.f;
    if (temp_every > 0) temp = 1.f + temp_coef * logf(static_cast<float>((positions[t] + 1) / temp_every + 1));
    for (int c = threadIdx.x; c < nq; c += blockDim.x) {
        const float v = to_f(r[c]) + (bias ? bias[c] : 0.f);
        q_out[static_cast<int64_t>(t) * nq + c] = from_f<T>(v * iq * q_w[c] * temp);
    }
    const int64_t slot = slots ? slots[t] : -1;
    if (slot < 0) return;
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
        const float v = to_f(r[nq + c]) + (bias ? bias[nq + c] : 0.f);
        k_cache[slot * nk + c] = from_f<T>(v * ik * k_w[c]);
    }
    for (int c = threadIdx.x; c < nv; c += blockDim.x)
        v_cache[slot * nv + c] = from_f<T>(to_f(r[nq + nk + c]) + (bias ? bias[nq + nk + c] : 0.f));
}

// ---------------------------------------------------------------------------------------------
// sigmoid attention, general kernel: one CTA per (query token, key split), keys in position order.
// With splits > 1 (decode steps over long contexts: few query tokens, many keys) every CTA writes the float32
// partial sums of its key range and attn_split_reduce_kernel adds them in split order — there is no softmax, so
// partial results simply add.
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float dot_row(const float *__restrict__ q, const T *__restrict__ k, int D) {
    float dot = 0.f;
    for (int d = 0; d < D; ++d) dot = fmaf(q[d], to_f(k[d]), dot);
    return dot;
}
// bfloat16 rows of a multiple of 8 elements: 16-byte loads
__device__ __forceinline__ float dot_row_vec(const float *__restrict__ q, const __nv_bfloat16 *__restrict__ k, int D) {
    float dot = 0.f;
    for (int d = 0; d < D; d += 8) {
        const uint4 v = *reinterpret_cast<const uint4 *>(k + d);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            dot = fmaf(q[d + 2 * i], f.x, dot);
            dot = fmaf(q[d + 2 * i + 1], f.y, dot);
        }
    }
    return dot;
}
constexpr int kGenThreads = 256;
constexpr int kGenKeys = 32;      // keys per pass
constexpr int kGenMaxOut = 32;    // outputs per thread: H * vdim <= 8192

template <typename T>
__global__ void __launch_bounds__(kGenThreads) sigmoid_attn_general_kernel(const atoma_sigmoid_attn_args a, int splits,
                                                                           float *__restrict__ partial) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int H = static_cast<int>(a.H), G = static_cast<int>(a.G), D = static_cast<int>(a.dim), Dv = static_cast<int>(a.vdim);
    const int rep = H / G;
    float *q_s = sm;                     // [H * D]
    float *w_s = q_s + H * D;            // [H][kGenKeys] raw weights
    float *m_s = w_s + H * kGenKeys;     // [H][kGenKeys] mixed weights
    float *talk_s = m_s + H * kGenKeys;  // [H * H]
    const int t = blockIdx.x;
    const int b = a.token_seq[t];
    const int p = static_cast<int>(a.positions[t]);
    const int32_t *bt = a.block_tables + static_cast<int64_t>(b) * a.max_blocks;
    const T *q = static_cast<const T *>(a.q) + static_cast<int64_t>(t) * H * D;
    const T *kc = static_cast<const T *>(a.k_cache);
    const T *vc = static_cast<const T *>(a.v_cache);
    const int bs = static_cast<int>(a.block_size);
    for (int i = threadIdx.x; i < H * D; i += kGenThreads) q_s[i] = to_f(q[i]);
    for (int i = threadIdx.x; i < H * H; i += kGenThreads) talk_s[i] = a.talk ? a.talk[i] : ((i / H == i % H) ? 1.f : 0.f);
    float acc[kGenMaxOut];
#pragma unroll
    for (int r = 0; r < kGenMaxOut; ++r) acc[r] = 0.f;
    __syncthreads();
    int k_lo = 0, k_hi = p + 1;
    if (splits > 1) {
        const int per = ((p + splits) / splits + kGenKeys - 1) / kGenKeys * kGenKeys;
        k_lo = min(p + 1, static_cast<int>(blockIdx.y) * per);
        k_hi = min(p + 1, k_lo + per);
    }
    const bool vec = sizeof(T) == 2 && D % 8 == 0;
    for (int j0 = k_lo; j0 < k_hi; j0 += kGenKeys) {
        for (int idx = threadIdx.x; idx < H * kGenKeys; idx += kGenThreads) {
            const int g = idx / kGenKeys, j = j0 + idx % kGenKeys;
            float w = 0.f;
            if (j < k_hi) {
                const int64_t slot = static_cast<int64_t>(bt[j / bs]) * bs + j % bs;
                const T *kr = kc + (slot * G + g / rep) * D;
                const float *qh = q_s + g * D;
                float dot;
                if (vec) dot = dot_row_vec(qh, reinterpret_cast<const __nv_bfloat16 *>(kr), D);
                else dot = dot_row<T>(qh, kr, D);
                w = sigmoid_weight(dot, a.scale, a.softcap, a.slopes ? a.slopes[g] : 0.f, static_cast<float>(p - j), a.head_bias[g]);
            }
            w_s[idx] = w;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < H * kGenKeys; idx += kGenThreads) {
            const int h = idx / kGenKeys, jj = idx % kGenKeys;
            float m = 0.f;
            for (int g = 0; g < H; ++g) m = fmaf(talk_s[h * H + g], w_s[g * kGenKeys + jj], m);
            m_s[idx] = m;
        }
        __syncthreads();
        const int nj = min(kGenKeys, k_hi - j0);
#pragma unroll
        for (int r = 0; r < kGenMaxOut; ++r) {
            const int od = threadIdx.x + r * kGenThreads;
            if (od < H * Dv) {
                const int h = od / Dv, d = od % Dv;
                float s = acc[r];
                for (int jj = 0; jj < nj; ++jj) {
                    const int j = j0 + jj;
                    const int64_t slot = static_cast<int64_t>(bt[j / bs]) * bs + j % bs;
                    s = fmaf(m_s[h * kGenKeys + jj], to_f(vc[(slot * G + h / rep) * Dv + d]), s);
                }
                acc[r] = s;
            }
        }
        __syncthreads();
    }
    if (partial) {
        float *o = partial + (static_cast<int64_t>(t) * splits + blockIdx.y) * H * Dv;
#pragma unroll
        for (int r = 0; r < kGenMaxOut; ++r) {
            const int od = threadIdx.x + r * kGenThreads;
            if (od < H * Dv) o[od] = acc[r];
        }
        return;
    }
    T *o = static_cast<T *>(a.out) + static_cast<int64_t>(t) * H * Dv;
#pragma unroll
    for (int r = 0; r < kGenMaxOut; ++r) {
        const int od = threadIdx.x + r * kGenThreads;
        if (od < H * Dv) o[od] = from_f<T>(acc[r]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) attn_split_reduce_kernel(const float *__restrict__ partial, T *__restrict__ out, int splits,
                                                                int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < splits; ++k) s += partial[(t * splits + k) * n + i];
        out[t * n + i] = from_f<T>(s);
    }
}

// ---------------------------------------------------------------------------------------------
// minGRU, sequential form: one thread per (sequence, channel), tokens in order
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) mingru_seq_kernel(const T *__restrict__ zxg, const float *__restrict__ bias,
                                                         float *__restrict__ state, const int32_t *__restrict__ slots,
                                                         const int32_t *__restrict__ query_start,
                                                         const int32_t *__restrict__ context_lens, T *__restrict__ out, int S) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= S) return;
    const int t0 = query_start[b], t1 = query_start[b + 1];
    if (t1 <= t0) return;
    float *st = state + static_cast<int64_t>(slots[b]) * S + c;
    float s = context_lens[b] > 0 ? *st : 0.f;
    const float bz = bias ? bias[c] : 0.f, bx = bias ? bias[S + c] : 0.f, bg = bias ? bias[2 * S + c] : 0.f;
    for (int t = t0; t < t1; ++t) {
        const T *r = zxg + static_cast<int64_t>(t) * 3 * S;
        float z, cand;
        mingru_gates(to_f(r[c]) + bz, to_f(r[S + c]) + bx, z, cand);
        s = (1.f - z) * s + z * cand;
        out[static_cast<int64_t>(t) * S + c] = from_f<T>(s * silu(to_f(r[2 * S + c]) + bg));
    }
    *st = s;
}

// minGRU, blocked scan for long portions.  The recurrence s <- a s + b (a = 1 - z, b = z cand) composes:
// (a2, b2) o (a1, b1) = (a2 a1, a2 b1 + b2).  A CTA owns 32 channels of one sequence; its 32 segment rows each fold
// a contiguous run of tokens, the segment summaries are chained in order, and each row then replays its run from
// its true start value and writes the gated output.
constexpr int kScanSeg = 32;
template <typename T>
__global__ void __launch_bounds__(32 * kScanSeg) mingru_scan_kernel(const T *__restrict__ zxg, const float *__restrict__ bias,
                                                                   float *__restrict__ state, const int32_t *__restrict__ slots,
                                                                   const int32_t *__restrict__ query_start,
                                                                   const int32_t *__restrict__ context_lens, T *__restrict__ out,
                                                                   int S) {
    __shared__ float sa[kScanSeg][33], sb[kScanSeg][33];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int lane = threadIdx.x, seg = threadIdx.y;
    const int c = blockIdx.x * 32 + lane;
    const int t0 = query_start[b], n = query_start[b + 1] - t0;
    if (n <= 0) return;
    const bool live = c < S;
    const int per = (n + kScanSeg - 1) / kScanSeg;
    const int lo = t0 + min(n, seg * per), hi = t0 + min(n, (seg + 1) * per);
    const float bz = (live && bias) ? bias[c] : 0.f, bx = (live && bias) ? bias[S + c] : 0.f, bg = (live && bias) ? bias[2 * S + c] : 0.f;
    float A = 1.f, B = 0.f;
    constexpr int kBatch = 8;   // tokens whose loads are issued together before any of them is used
    if (live)
        for (int t = lo; t < hi; t += kBatch) {
            T zr[kBatch], ur[kBatch];
#pragma unroll
            for (int i = 0; i < kBatch; ++i)
                if (t + i < hi) {
                    const T *r = zxg + static_cast<int64_t>(t + i) * 3 * S;
                    zr[i] = r[c];
                    ur[i] = r[S + c];
                }
#pragma unroll
            for (int i = 0; i < kBatch; ++i)
                if (t + i < hi) {
                    float z, cand;
                    mingru_gates(to_f(zr[i]) + bz, to_f(ur[i]) + bx, z, cand);
                    A = (1.f - z) * A;
                    B = (1.f - z) * B + z * cand;
                }
        }
    sa[seg][lane] = A;
    sb[seg][lane] = B;
    __syncthreads();
    float *st = state + (live ? static_cast<int64_t>(slots[b]) * S + c : 0);
    float s = (live && context_lens[b] > 0) ? *st : 0.f;
    for (int k = 0; k < seg; ++k) s = sa[k][lane] * s + sb[k][lane];
    if (!live) return;
    for (int t = lo; t < hi; t += kBatch) {
        T zr[kBatch], ur[kBatch], gr[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; ++i)
            if (t + i < hi) {
                const T *r = zxg + static_cast<int64_t>(t + i) * 3 * S;
                zr[i] = r[c];
                ur[i] = r[S + c];
                gr[i] = r[2 * S + c];
            }
#pragma unroll
        for (int i = 0; i < kBatch; ++i)
            if (t + i < hi) {
                float z, cand;
                mingru_gates(to_f(zr[i]) + bz, to_f(ur[i]) + bx, z, cand);
                s = (1.f - z) * s + z * cand;
                out[static_cast<int64_t>(t + i) * S + c] = from_f<T>(s * silu(to_f(gr[i]) + bg));
            }
    }
    if (seg == kScanSeg - 1) *st = s;
}

// ---------------------------------------------------------------------------------------------
// gated feed-forward activation
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) glu_kernel(const T *__restrict__ gu, T *__restrict__ out, int64_t total, int ff, int act) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = i / ff;
        const int j = static_cast<int>(i % ff);
        const float g = to_f(gu[t * 2 * ff + j]), u = to_f(gu[t * 2 * ff + ff + j]);
        out[i] = from_f<T>(glu_act(g, act) * u);
    }
}

// ---------------------------------------------------------------------------------------------
// plain GEMM: float32 FMA, k in ascending order, any shape; y = x w^T
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) gemm_plain_kernel(const T *__restrict__ x, const T *__restrict__ w, T *__restrict__ y, int M,
                                                         int N, int K) {
    __shared__ float xs[16][65], ws[16][65];
    pdl_launch_dependents();
    pdl_wait();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i / 16, k = i % 16;
            xs[k][r] = (m0 + r < M && k0 + k < K) ? to_f(x[static_cast<int64_t>(m0 + r) * K + k0 + k]) : 0.f;
            ws[k][r] = (n0 + r < N && k0 + k < K) ? to_f(w[static_cast<int64_t>(n0 + r) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                xv[i] = xs[k][ty * 4 + i];
                wv[i] = ws[k][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) y[static_cast<int64_t>(m) * N + n] = from_f<T>(acc[i][j]);
        }
}

// ---------------------------------------------------------------------------------------------
// logit scale + greedy choice (ties: the last index, as atoma_sample_greedy)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) scale_greedy_kernel(const T *__restrict__ logits, float *__restrict__ out,
                                                           uint32_t *__restrict__ token_out, int vocab, float scale,
                                                           float softcap) {
    __shared__ float bv[256];
    __shared__ int bi[256];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t base = static_cast<int64_t>(blockIdx.x) * vocab;
    float best = -INFINITY;
    int idx = -1;
    for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
        float v = to_f(logits[base + c]) * scale;
        if (softcap > 0.f) v = softcap * tanhf(v / softcap);
        if (out) out[base + c] = v;
        if (v >= best) {
            best = v;
            idx = c;
        }
    }
    bv[threadIdx.x] = best;
    bi[threadIdx.x] = idx;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = bv[threadIdx.x + s];
            const int oi = bi[threadIdx.x + s];
            if (oi >= 0 && (bi[threadIdx.x] < 0 || ov > bv[threadIdx.x] || (ov == bv[threadIdx.x] && oi > bi[threadIdx.x]))) {
                bv[threadIdx.x] = ov;
                bi[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0 && token_out) token_out[blockIdx.x] = static_cast<uint32_t>(bi[0] < 0 ? 0 : bi[0]);
}

bool finish(cudaError_t e, const char *what) {
    note_launch();
    if (e != cudaSuccess) {
        set_status(static_cast<int>(e), "%s: %s", what, cudaGetErrorString(e));
        return false;
    }
    return check_launch(what);
}

bool bad_dtype(uint32_t dtype, const char *what) {
    if (dtype == ATOMA_DTYPE_BF16 || dtype == ATOMA_DTYPE_F32) return false;
    set_status(kErrInvalidArg, "%s: dtype must be 1 (bfloat16) or 2 (float32), got %u", what, dtype);
    return true;
}

}  // namespace

#define HYB_DISPATCH(dtype, CALL)                      \
    ((dtype) == ATOMA_DTYPE_BF16 ? CALL(__nv_bfloat16) : CALL(float))

bool hyb_embed_sinusoid(const uint32_t *tokens, const int64_t *positions, const void *table, const double *inv_freq, float *out,
                        int64_t T, int64_t width, int64_t vocab, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (bad_dtype(dtype, "atoma_embed_sinusoid")) return false;
    if (!tokens || !positions || !table || !inv_freq || !out || width <= 0 || vocab <= 0) {
        set_status(kErrInvalidArg, "atoma_embed_sinusoid: null argument or empty table");
        return false;
    }
#define CALL(TT) launch_ex(embed_sinusoid_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(128), 0, stream, tokens, positions, \
                           static_cast<const TT *>(table), inv_freq, out, static_cast<int>(width), vocab)
    return finish(HYB_DISPATCH(dtype, CALL), "embed_sinusoid_kernel");
#undef CALL
}

bool hyb_rmsnorm_rows(const float *x, const int32_t *rows, const float *weight, float offset, void *out, int64_t R, int64_t width,
                      float eps, uint32_t dtype, cudaStream_t stream) {
    if (R <= 0) return true;
    if (bad_dtype(dtype, "atoma_rmsnorm_rows")) return false;
    if (!x || !weight || !out || width <= 0) {
        set_status(kErrInvalidArg, "atoma_rmsnorm_rows: null argument");
        return false;
    }
#define CALL(TT) launch_ex(rmsnorm_rows_kernel<TT>, dim3(static_cast<unsigned>(R)), dim3(kRowThreads), 0, stream, x, rows, weight, \
                           offset, static_cast<TT *>(out), static_cast<int>(width), eps)
    return finish(HYB_DISPATCH(dtype, CALL), "rmsnorm_rows_kernel");
#undef CALL
}

bool hyb_postnorm_add_prenorm(const void *y, float *x, const float *w_post, const float *w_pre, void *h, int64_t T, int64_t width,
                              float eps, float offset, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (bad_dtype(dtype, "atoma_postnorm_add_prenorm")) return false;
    if (!y || !x || !w_post || (w_pre && !h) || width <= 0 || width * 4 > 200 * 1024) {
        set_status(kErrInvalidArg, "atoma_postnorm_add_prenorm: null argument or width %lld", static_cast<long long>(width));
        return false;
    }
    const size_t smem = static_cast<size_t>(width) * 4;
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(postnorm_add_prenorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(postnorm_add_prenorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
#define CALL(TT) launch_ex(postnorm_add_prenorm_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(kRowThreads), smem, stream, \
                           static_cast<const TT *>(y), x, w_post, w_pre, static_cast<TT *>(h), static_cast<int>(width), eps, offset)
    return finish(HYB_DISPATCH(dtype, CALL), "postnorm_add_prenorm_kernel");
#undef CALL
}

bool hyb_qk_norm_cache(const void *qkv, const float *bias, const float *q_w, const float *k_w, const int64_t *positions,
                       const int64_t *slots, void *q_out, void *k_cache, void *v_cache, int64_t T, int64_t H, int64_t G, int64_t dim,
                       int64_t vdim, float eps, float temp_coef, int64_t temp_every, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (bad_dtype(dtype, "atoma_qk_norm_cache")) return false;
    if (!qkv || !q_w || !k_w || !positions || !q_out || H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 ||
        (slots && (!k_cache || !v_cache))) {
        set_status(kErrInvalidArg, "atoma_qk_norm_cache: null argument, or kv heads (%lld) do not divide heads (%lld)",
                   static_cast<long long>(G), static_cast<long long>(H));
        return false;
    }
#define CALL(TT) launch_ex(qk_norm_cache_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(kRowThreads), 0, stream, \
                           static_cast<const TT *>(qkv), bias, q_w, k_w, positions, slots, static_cast<TT *>(q_out), \
                           static_cast<TT *>(k_cache), static_cast<TT *>(v_cache), static_cast<int>(H * dim), \
                           static_cast<int>(G * dim), static_cast<int>(G * vdim), eps, temp_coef, temp_every)
    return finish(HYB_DISPATCH(dtype, CALL), "qk_norm_cache_kernel");
#undef CALL
}

bool hyb_attention_check(const atoma_sigmoid_attn_args &a) {
    if (bad_dtype(a.dtype, "atoma_sigmoid_attention_paged")) return false;
    if (!a.q || !a.k_cache || !a.v_cache || !a.out || !a.positions || !a.token_seq || !a.block_tables ||
        !a.head_bias || a.H <= 0 || a.G <= 0 || a.H % a.G || a.dim <= 0 || a.vdim <= 0 || a.block_size <= 0 || a.max_blocks <= 0) {
        set_status(kErrInvalidArg, "atoma_sigmoid_attention_paged: null argument or inconsistent head counts");
        return false;
    }
    return true;
}

bool hyb_attention_general(const atoma_sigmoid_attn_args &a, cudaStream_t stream) {
    if (a.H * a.vdim > kGenThreads * kGenMaxOut) {
        set_status(kErrUnsupported, "atoma_sigmoid_attention_paged: heads * vdim = %lld exceeds %d",
                   static_cast<long long>(a.H * a.vdim), kGenThreads * kGenMaxOut);
        return false;
    }
    const size_t smem = static_cast<size_t>(a.H * a.dim + 2 * a.H * kGenKeys + a.H * a.H) * 4;
    if (smem > 200 * 1024) {
        set_status(kErrUnsupported, "atoma_sigmoid_attention_paged: %zu bytes of shared memory", smem);
        return false;
    }
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(sigmoid_attn_general_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(sigmoid_attn_general_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
    // decode-only batches over long contexts: split the keys so that the few query tokens fill the device
    int splits = 1;
    if (a.max_query_len == 1 && a.max_seq_len >= 4 * kGenKeys && !(g_hybrid_debug & 2)) {
        const int64_t want = (2 * current_device_info().sm_count + a.T - 1) / a.T;
        splits = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>({want, (a.max_seq_len + 2 * kGenKeys - 1) / (2 * kGenKeys), 64})));
    }
    float *partial = nullptr;
    if (splits > 1) {
        partial = static_cast<float *>(get_workspace(stream, static_cast<size_t>(a.T) * splits * a.H * a.vdim * 4, kWorkspaceHybridAttn));
        if (!partial) return false;
    }
    const dim3 grid(static_cast<unsigned>(a.T), static_cast<unsigned>(splits));
#define CALL(TT) launch_ex(sigmoid_attn_general_kernel<TT>, grid, dim3(kGenThreads), smem, stream, a, splits, partial)
    if (!finish(HYB_DISPATCH(a.dtype, CALL), "sigmoid_attn_general_kernel")) return false;
#undef CALL
    if (splits == 1) return true;
    return hyb_attn_split_reduce(partial, a.out, a.T, splits, a.H * a.vdim, a.dtype, stream);
}

bool hyb_attn_split_reduce(const float *partial, void *out, int64_t T, int splits, int64_t n, uint32_t dtype, cudaStream_t stream) {
#define CALL(TT) launch_ex(attn_split_reduce_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(256), 0, stream, partial, \
                           static_cast<TT *>(out), splits, static_cast<int>(n))
    return finish(HYB_DISPATCH(dtype, CALL), "attn_split_reduce_kernel");
#undef CALL
}

bool hyb_attention_fast(const atoma_sigmoid_attn_args &a, cudaStream_t stream, bool *taken);   // hybrid_attention.cu
bool hyb_sigmoid_attention_tc(const atoma_sigmoid_attn_args &a, cudaStream_t stream, bool *taken);   // softmax_attention_tc.cu

bool hyb_attention(const atoma_sigmoid_attn_args &a, cudaStream_t stream) {
    if (a.T <= 0) return true;
    if (!hyb_attention_check(a)) return false;
    if (!(g_hybrid_debug & 2) && !a.slopes && !a.talk && a.softcap == 0.f) {
        // independent heads (no distance term, no cap, no talk): the warp-level tensor-core kernels that softmax attention uses
        bool taken = false;
        const bool ok = hyb_sigmoid_attention_tc(a, stream, &taken);
        if (taken || !ok) return ok;
    }
    if (!(g_hybrid_debug & 2)) {
        bool taken = false;
        const bool ok = hyb_attention_fast(a, stream, &taken);
        if (taken) return ok;
    }
    return hyb_attention_general(a, stream);
}

bool hyb_mingru_scan(const void *zxg, const float *bias, float *state, const int32_t *slots, const int32_t *query_start,
                     const int32_t *context_lens, void *out, int64_t T, int64_t B, int64_t S, int32_t max_query_len,
                     uint32_t dtype, cudaStream_t stream) {
    if (T <= 0 || B <= 0) return true;
    if (bad_dtype(dtype, "atoma_mingru_scan")) return false;
    if (!zxg || !state || !slots || !query_start || !context_lens || !out || S <= 0) {
        set_status(kErrInvalidArg, "atoma_mingru_scan: null argument");
        return false;
    }
    if (max_query_len >= 4 * kScanSeg && !(g_hybrid_debug & 4)) {
        const dim3 grid(static_cast<unsigned>((S + 31) / 32), static_cast<unsigned>(B));
#define CALL(TT) launch_ex(mingru_scan_kernel<TT>, grid, dim3(32, kScanSeg), 0, stream, static_cast<const TT *>(zxg), bias, state, \
                           slots, query_start, context_lens, static_cast<TT *>(out), static_cast<int>(S))
        return finish(HYB_DISPATCH(dtype, CALL), "mingru_scan_kernel");
#undef CALL
    }
    const dim3 grid(static_cast<unsigned>((S + 127) / 128), static_cast<unsigned>(B));
#define CALL(TT) launch_ex(mingru_seq_kernel<TT>, grid, dim3(128), 0, stream, static_cast<const TT *>(zxg), bias, state, slots, \
                           query_start, context_lens, static_cast<TT *>(out), static_cast<int>(S))
    return finish(HYB_DISPATCH(dtype, CALL), "mingru_seq_kernel");
#undef CALL
}

bool hyb_glu(const void *gu, void *out, int64_t T, int64_t ff, int32_t act, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0 || ff <= 0) return true;
    if (bad_dtype(dtype, "atoma_glu")) return false;
    if (!gu || !out || act < 0 || act > 2) {
        set_status(kErrInvalidArg, "atoma_glu: null argument or unknown activation %d", act);
        return false;
    }
    const int64_t total = T * ff;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148 * 8));
#define CALL(TT) launch_ex(glu_kernel<TT>, dim3(grid), dim3(256), 0, stream, static_cast<const TT *>(gu), static_cast<TT *>(out), total, \
                           static_cast<int>(ff), act)
    return finish(HYB_DISPATCH(dtype, CALL), "glu_kernel");
#undef CALL
}

bool hyb_linear(const void *x, const void *w, void *y, int64_t T, int64_t N, int64_t K, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return true;
    if (bad_dtype(dtype, "atoma_linear")) return false;
    if (!x || !w || !y || K <= 0) {
        set_status(kErrInvalidArg, "atoma_linear: null argument or K = %lld", static_cast<long long>(K));
        return false;
    }
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (dtype == ATOMA_DTYPE_BF16 && !(g_hybrid_debug & 1) && K % 8 == 0 && N % 8 == 0 && al(x) && al(w) && al(y) &&
        current_device_info().cc_major == 10) {
        atoma_gemm_tn(x, w, y, T, N, K, K, K, N, 1, stream);
        return atoma_last_status() == 0;
    }
    const dim3 grid(static_cast<unsigned>((N + 63) / 64), static_cast<unsigned>((T + 63) / 64));
#define CALL(TT) launch_ex(gemm_plain_kernel<TT>, grid, dim3(256), 0, stream, static_cast<const TT *>(x), static_cast<const TT *>(w), \
                           static_cast<TT *>(y), static_cast<int>(T), static_cast<int>(N), static_cast<int>(K))
    return finish(HYB_DISPATCH(dtype, CALL), "gemm_plain_kernel");
#undef CALL
}

// gate/up projection + gated activation: act_out[T, ff] = act(x Wg^T) * (x Wu^T), w_gate_up = [Wg; Wu].
bool hyb_gate_up_act(const void *x, const void *w_gate_up, void *proj, void *act_out, int64_t T, int64_t ff, int64_t K, int32_t act,
                     uint32_t dtype, cudaStream_t stream) {
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    // decode-sized steps in bfloat16: the activation runs in the projection's epilogue (the tile pairs gate row i with up row i)
    if (dtype == ATOMA_DTYPE_BF16 && !(g_hybrid_debug & 1) && T <= 128 && K % 64 == 0 && ff % 8 == 0 && al(x) && al(w_gate_up) &&
        al(act_out) && current_device_info().cc_major == 10) {
        atoma_gate_up_act(x, w_gate_up, act_out, T, ff, K, K, K, ff, act, 1, stream);
        return atoma_last_status() == 0;
    }
    if (!hyb_linear(x, w_gate_up, proj, T, 2 * ff, K, dtype, stream)) return false;
    return hyb_glu(proj, act_out, T, ff, act, dtype, stream);
}

bool hyb_glu_clamped_bias(const void *, int64_t, const float *, void *, int64_t, int64_t, float, float, float, uint32_t, cudaStream_t);

// gate/up projection + clamped gated activation with biases: act_out[T, ff] = g sigmoid(alpha g) (u + shift) on the clamped,
// biased projections; w_gate_up = [Wg; Wu], bias = [bg; bu] (may be null).
bool hyb_gate_up_clamped(const void *x, const void *w_gate_up, const float *bias, void *proj, void *act_out, int64_t T, int64_t ff, int64_t K,
                         float limit, float alpha, float shift, uint32_t dtype, cudaStream_t stream) {
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    // decode-sized steps in bfloat16: the activation runs in the projection's epilogue (the tile pairs gate row i with up row i)
    if (dtype == ATOMA_DTYPE_BF16 && !(g_hybrid_debug & 1) && T <= 128 && K % 64 == 0 && ff % 8 == 0 && al(x) && al(w_gate_up) &&
        al(act_out) && current_device_info().cc_major == 10) {
        atoma_gate_up_clamped(x, w_gate_up, bias, act_out, T, ff, K, K, K, ff, limit, alpha, shift, 1, stream);
        return atoma_last_status() == 0;
    }
    if (!hyb_linear(x, w_gate_up, proj, T, 2 * ff, K, dtype, stream)) return false;
    return hyb_glu_clamped_bias(proj, 2 * ff, bias, act_out, T, ff, limit, alpha, shift, dtype, stream);
}

bool hyb_scale_greedy(const void *logits, float *out, uint32_t *token_out, int64_t R, int64_t vocab, float scale, float softcap,
                      uint32_t dtype, cudaStream_t stream) {
    if (R <= 0) return true;
    if (bad_dtype(dtype, "atoma_scale_logits_greedy")) return false;
    if (!logits || vocab <= 0) {
        set_status(kErrInvalidArg, "atoma_scale_logits_greedy: null argument");
        return false;
    }
#define CALL(TT) launch_ex(scale_greedy_kernel<TT>, dim3(static_cast<unsigned>(R)), dim3(256), 0, stream, \
                           static_cast<const TT *>(logits), out, token_out, static_cast<int>(vocab), scale, softcap)
    return finish(HYB_DISPATCH(dtype, CALL), "scale_greedy_kernel");
#undef CALL
}

}  // namespace atoma

using namespace atoma;

extern "C" void atoma_embed_sinusoid(const uint32_t *tokens, const int64_t *positions, const void *table, const double *inv_freq,
                                     float *out, int64_t T, int64_t width, int64_t vocab, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_embed_sinusoid(tokens, positions, table, inv_freq, out, T, width, vocab, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_rmsnorm_rows(const float *x, const int32_t *rows, const float *weight, float weight_offset, void *out, int64_t R,
                                   int64_t width, float eps, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_rmsnorm_rows(x, rows, weight, weight_offset, out, R, width, eps, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_postnorm_add_prenorm(const void *y, float *x, const float *w_post, const float *w_pre, void *h, int64_t T,
                                           int64_t width, float eps, float weight_offset, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_postnorm_add_prenorm(y, x, w_post, w_pre, h, T, width, eps, weight_offset, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_qk_norm_cache(const void *qkv, const float *bias, const float *q_weight, const float *k_weight,
                                    const int64_t *positions, const int64_t *slot_mapping, void *q_out, void *k_cache, void *v_cache,
                                    int64_t T, int64_t H, int64_t G, int64_t dim, int64_t vdim, float eps, float temp_coef,
                                    int64_t temp_every, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_qk_norm_cache(qkv, bias, q_weight, k_weight, positions, slot_mapping, q_out, k_cache, v_cache, T, H, G, dim, vdim, eps,
                      temp_coef, temp_every, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_sigmoid_attention_paged(const atoma_sigmoid_attn_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_sigmoid_attention_paged: args is NULL");
        return;
    }
    hyb_attention(*args, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_mingru_scan(const void *zxg, const float *bias, float *state, const int32_t *state_slots,
                                  const int32_t *query_start, const int32_t *context_lens, void *out, int64_t T, int64_t B, int64_t S,
                                  int32_t max_query_len, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_mingru_scan(zxg, bias, state, state_slots, query_start, context_lens, out, T, B, S, max_query_len, dtype,
                    static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_glu(const void *gu, void *out, int64_t T, int64_t ff, int32_t act, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_glu(gu, out, T, ff, act, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_linear(const void *x, const void *w, void *y, int64_t T, int64_t N, int64_t K, uint32_t dtype,
                             atoma_stream_t stream) {
    clear_status();
    hyb_linear(x, w, y, T, N, K, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_scale_logits_greedy(const void *logits, float *logits_f32, uint32_t *token_out, int64_t R, int64_t vocab,
                                          float scale, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_scale_greedy(logits, logits_f32, token_out, R, vocab, scale, 0.f, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_finish_logits_greedy(const void *logits, float *logits_f32, uint32_t *token_out, int64_t R, int64_t vocab, float scale,
                                           float softcap, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_scale_greedy(logits, logits_f32, token_out, R, vocab, scale, softcap, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_debug_hybrid(int flags) { g_hybrid_debug = flags; }
extern "C" void atoma_linear_glu_clamped(const void *x, const void *w_gate_up, const float *bias, void *proj, void *act_out, int64_t T,
                                         int64_t ff, int64_t K, float limit, float alpha, float up_shift, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_gate_up_clamped(x, w_gate_up, bias, proj, act_out, T, ff, K, limit, alpha, up_shift, dtype, static_cast<cudaStream_t>(stream));
}
