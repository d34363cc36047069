// Latent attention over a paged cache of ONE shared latent per token — include/atoma_hybrid.h.
//
// Keys and values of every head are linear images of a cached latent c_j: k_h = Wk_h c_j, v_h = Wv_h c_j.  Nothing
// is expanded per key here: the query is moved into the latent space once (q_lat_h = Wk_h^T q_h, atoma_head_project),
// scores are q_lat_h . c_j, the weighted sum of latents is taken per head, and a head's values come from that sum
// (Wv_h sum_j w_j c_j, atoma_head_project again).  The cache is read once per token for all heads.
//
// Softmax with a sink: the running maximum starts at the sink and the running denominator at one (exp(sink - sink)),
// so the sink is one more term of the denominator that has no key and no value.  Sliding window: keys
// [max(0, p - window + 1), p].  Scores, weights and sums are float32; keys are visited in position order in
// tiles that start at the window's first key, so a query's result does not depend on the batch around it.
#include "common.cuh"
#include "hybrid_common.cuh"
#include "mha_params.h"
#include "tc_products.cuh"

#include "atoma_hybrid.h"

#include <algorithm>
#include <cstring>

namespace atoma {

extern int g_hybrid_debug;
int try_launch_prefill_tc(const MhaParams &p, bool is_bf16, cudaStream_t stream);   // prefill_attention.cu
bool hyb_linear(const void *, const void *, void *, int64_t, int64_t, int64_t, uint32_t, cudaStream_t);

namespace {

using namespace hybrid;

// ---------------------------------------------------------------------------------------------
// RMS norms of the two latents + cache write
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kRowThreads) latent_norm_cache_kernel(const T *__restrict__ proj, int64_t ld,
                                                                        const float *__restrict__ q_w, const float *__restrict__ kv_w,
                                                                        const int64_t *__restrict__ slots, T *__restrict__ cq_out,
                                                                        T *__restrict__ cache, int q_rank, int kv_rank, float eps) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const T *r = proj + t * ld;
    if (q_rank > 0) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
            const float v = to_f(r[c]);
            ss = fmaf(v, v, ss);
        }
        const float inv = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(q_rank) + eps);
        for (int c = threadIdx.x; c < q_rank; c += blockDim.x) cq_out[t * q_rank + c] = from_f<T>(to_f(r[c]) * inv * q_w[c]);
    }
    const int64_t slot = slots ? slots[t] : -1;
    if (slot < 0) return;
    float ss = 0.f;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) {
        const float v = to_f(r[q_rank + c]);
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(kv_rank) + eps);
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) cache[slot * kv_rank + c] = from_f<T>(to_f(r[q_rank + c]) * inv * kv_w[c]);
}

// ---------------------------------------------------------------------------------------------
// Per-head projection: out[t, h, n] = sum_k in[t, h, k] w(h, k, n); float32 FMA tiles, k ascending.
// ---------------------------------------------------------------------------------------------
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256) head_project_kernel(const TA *__restrict__ in, int64_t ld_in, int64_t in_hs,
                                                           const TW *__restrict__ w, int64_t w_hs, int64_t w_ks, int64_t w_ns,
                                                           TO *__restrict__ out, int64_t ld_out, int64_t out_hs, int M, int N, int K) {
    __shared__ float xs[16][65], ws[16][65];
    pdl_launch_dependents();
    pdl_wait();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int64_t h = blockIdx.z;
    in += h * in_hs;
    w += h * w_hs;
    out += h * out_hs;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i / 16, k = i % 16;
            xs[k][r] = (m0 + r < M && k0 + k < K) ? to_f(in[static_cast<int64_t>(m0 + r) * ld_in + k0 + k]) : 0.f;
        }
        if (w_ns == 1) {   // n contiguous: read along n
            for (int i = threadIdx.x; i < 64 * 16; i += 256) {
                const int k = i / 64, r = i % 64;
                ws[k][r] = (n0 + r < N && k0 + k < K) ? to_f(w[static_cast<int64_t>(k0 + k) * w_ks + (n0 + r)]) : 0.f;
            }
        } else {
            for (int i = threadIdx.x; i < 64 * 16; i += 256) {
                const int r = i / 16, k = i % 16;
                ws[k][r] = (n0 + r < N && k0 + k < K) ? to_f(w[static_cast<int64_t>(k0 + k) * w_ks + static_cast<int64_t>(n0 + r) * w_ns]) : 0.f;
            }
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
            if (m < M && n < N) out[static_cast<int64_t>(m) * ld_out + n] = from_f<TO>(acc[i][j]);
        }
}

// ---------------------------------------------------------------------------------------------
// Attention, general kernel: one CTA per (query token, key split).
// ---------------------------------------------------------------------------------------------
constexpr int kLatThreads = 256;
constexpr int kLatKeys = 32;
constexpr int kLatMaxOut = 32;   // outputs per thread: H * R <= 8192

template <typename T>
__global__ void __launch_bounds__(kLatThreads) latent_attn_general_kernel(const atoma_latent_attn_args a, int splits, int head_chunk,
                                                                          float *__restrict__ partial, float *__restrict__ partial_ml) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    // heads [h0, h0 + H) of the a.H heads: a CTA's outputs (H x R) are bounded by its registers, more heads take more CTAs
    const int h0 = static_cast<int>(blockIdx.z) * head_chunk, H = min(head_chunk, static_cast<int>(a.H) - h0), HT = static_cast<int>(a.H);
    const int R = static_cast<int>(a.R);
    const int cs = R + 1;                  // padded row of the staged latents
    float *q_s = sm;                       // [H][R]
    float *c_s = q_s + H * R;              // [kLatKeys][R + 1]
    float *w_s = c_s + kLatKeys * cs;      // [H][kLatKeys]
    float *m_s = w_s + H * kLatKeys;       // [H] running maximum
    float *l_s = m_s + H;                  // [H] running denominator
    float *f_s = l_s + H;                  // [H] rescale factor of the tile
    const int t = blockIdx.x;
    const int b = a.token_seq[t];
    if (a.skip_min_q > 0 && a.query_start[b + 1] - a.query_start[b] >= a.skip_min_q) return;   // served on expanded keys
    const int p = static_cast<int>(a.positions[t]);
    const int32_t *bt = a.block_tables + static_cast<int64_t>(b) * a.max_blocks;
    const T *cache = static_cast<const T *>(a.latent_cache);
    const int bs = static_cast<int>(a.block_size);
    const int lo = a.window > 0 ? max(0, p - static_cast<int>(a.window) + 1) : 0;
    int k_lo = lo, k_hi = p + 1;
    if (splits > 1) {
        const int n = p + 1 - lo;
        const int per = ((n + splits - 1) / splits + kLatKeys - 1) / kLatKeys * kLatKeys;
        k_lo = min(p + 1, lo + static_cast<int>(blockIdx.y) * per);
        k_hi = min(p + 1, k_lo + per);
    }
    const float *q = a.q_lat + (static_cast<int64_t>(t) * HT + h0) * R;
    for (int i = threadIdx.x; i < H * R; i += kLatThreads) q_s[i] = q[i];
    const bool first = blockIdx.y == 0;
    for (int h = threadIdx.x; h < H; h += kLatThreads) {
        const bool snk = first && a.sink != nullptr;
        m_s[h] = snk ? a.sink[h0 + h] : -INFINITY;
        l_s[h] = snk ? 1.f : 0.f;
    }
    float acc[kLatMaxOut];
#pragma unroll
    for (int r = 0; r < kLatMaxOut; ++r) acc[r] = 0.f;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int j0 = k_lo; j0 < k_hi; j0 += kLatKeys) {
        for (int i = threadIdx.x; i < kLatKeys * R; i += kLatThreads) {
            const int jj = i / R, r = i % R, j = j0 + jj;
            float v = 0.f;
            if (j < k_hi) v = to_f(cache[(static_cast<int64_t>(bt[j / bs]) * bs + j % bs) * R + r]);
            c_s[jj * cs + r] = v;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < H * kLatKeys; idx += kLatThreads) {
            const int h = idx / kLatKeys, jj = idx % kLatKeys;
            float s = -INFINITY;
            if (j0 + jj < k_hi) {
                const float *qh = q_s + h * R, *cr = c_s + jj * cs;
                float dot = 0.f;
                for (int r = 0; r < R; ++r) dot = fmaf(qh[r], cr[r], dot);
                s = dot * a.scale;
            }
            w_s[idx] = s;
        }
        __syncthreads();
        for (int h = warp; h < H; h += kLatThreads / 32) {
            const float s = w_s[h * kLatKeys + lane];
            float mx = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, mx);    // finite: the tile holds at least one key
            const float e = s == -INFINITY ? 0.f : expf(s - m_new);
            float sum = e;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const float f = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
            w_s[h * kLatKeys + lane] = e;
            __syncwarp();
            if (lane == 0) {
                m_s[h] = m_new;
                l_s[h] = l_s[h] * f + sum;
                f_s[h] = f;
            }
        }
        __syncthreads();
        const int nj = min(kLatKeys, k_hi - j0);
#pragma unroll
        for (int r = 0; r < kLatMaxOut; ++r) {
            const int od = threadIdx.x + r * kLatThreads;
            if (od < H * R) {
                const int h = od / R, d = od % R;
                float s = acc[r] * f_s[h];
                for (int jj = 0; jj < nj; ++jj) s = fmaf(w_s[h * kLatKeys + jj], c_s[jj * cs + d], s);
                acc[r] = s;
            }
        }
        __syncthreads();
    }
    if (partial) {
        float *o = partial + ((static_cast<int64_t>(t) * splits + blockIdx.y) * HT + h0) * R;
#pragma unroll
        for (int r = 0; r < kLatMaxOut; ++r) {
            const int od = threadIdx.x + r * kLatThreads;
            if (od < H * R) o[od] = acc[r];
        }
        float *ml = partial_ml + ((static_cast<int64_t>(t) * splits + blockIdx.y) * HT + h0) * 2;
        for (int h = threadIdx.x; h < H; h += kLatThreads) {
            ml[2 * h] = m_s[h];
            ml[2 * h + 1] = l_s[h];
        }
        return;
    }
    float *o = a.out + (static_cast<int64_t>(t) * HT + h0) * R;
#pragma unroll
    for (int r = 0; r < kLatMaxOut; ++r) {
        const int od = threadIdx.x + r * kLatThreads;
        if (od < H * R) {
            const float l = l_s[od / R];
            o[od] = l > 0.f ? acc[r] / l : 0.f;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Attention on tensor cores (bfloat16 cache): a CTA owns 16 * MT consecutive (query, head) rows of ONE sequence — for a
// decoded token its heads, for a prompt's portion several queries with all their heads — and walks the keys those rows can
// see in tiles of 32, staged once in shared memory (cp.async, double buffered) and used as BOTH operands: S = Q C^T reads
// the tile as stored (keys x latent), O += P C reads it transposed (ldmatrix.trans).  Per tile: the score product is split
// over the warps along the LATENT axis (a warp multiplies all rows by 32 or 16 keys over a quarter of the latent columns, so
// that every fragment it loads feeds several mma.sync m16n8k16), the four partial score tiles are summed while the rows'
// running maxima / denominators are updated in float32 with the window mask per row, P is rounded to bfloat16, and each
// warp accumulates its share of the latent columns for all rows.  Why mma.sync and not tcgen05: the rows of a tile are H heads
// of a few queries (16 to 64), far below a 128-row tensor-memory tile, and every row has its own window, so a larger tile
// would multiply mostly masked pairs.
// ---------------------------------------------------------------------------------------------
constexpr int kTcKeys = 32;
constexpr int kSpLd = 40;         // row stride of the partial score tiles (floats)
constexpr int kTcMaxNT = 8;      // n8 tiles of a warp's share of the latent columns: R <= 64 * warps

template <int MT, int NW>   // row tiles of 16; warps (4 or 8)
__global__ void __launch_bounds__(32 * NW) latent_attn_tc_kernel(const atoma_latent_attn_args a, int splits, float *__restrict__ partial,
                                                                 float *__restrict__ partial_ml) {
    extern __shared__ __align__(16) unsigned char smraw[];
    constexpr int ROWS = 16 * MT, NTHR = 32 * NW;
    constexpr int KEYS_W = NW == 8 ? 16 : 32;      // keys a warp multiplies in the score product
    constexpr int NKT = KEYS_W / 8;
    pdl_launch_dependents();
    pdl_wait();
    const int H = static_cast<int>(a.H), R = static_cast<int>(a.R), bs = static_cast<int>(a.block_size);
    const int b = blockIdx.y;
    const int q0 = a.query_start[b], nq = a.query_start[b + 1] - q0;
    const int row0 = blockIdx.x * ROWS, nrows = nq * H;
    if (row0 >= nrows) return;
    if (a.skip_min_q > 0 && nq >= a.skip_min_q) return;   // served on expanded keys
    const int ldc = R + 8;
    __nv_bfloat16 *Qs = reinterpret_cast<__nv_bfloat16 *>(smraw);                 // [ROWS][R + 8]
    __nv_bfloat16 *Cs = Qs + ROWS * ldc;                                          // [2][32][R + 8]
    float *Sp = reinterpret_cast<float *>(Cs + 2 * kTcKeys * ldc);                // [4][ROWS][40] partial scores per latent quarter
    __nv_bfloat16 *Pb = reinterpret_cast<__nv_bfloat16 *>(Sp + 4 * ROWS * kSpLd);  // [ROWS][40]
    float *m_s = reinterpret_cast<float *>(Pb + ROWS * 40);
    float *l_s = m_s + ROWS, *f_s = l_s + ROWS;
    int *p_s = reinterpret_cast<int *>(f_s + ROWS), *lo_s = p_s + ROWS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int32_t *bt = a.block_tables + static_cast<int64_t>(b) * a.max_blocks;
    const __nv_bfloat16 *cache = static_cast<const __nv_bfloat16 *>(a.latent_cache);
    const int split = blockIdx.z;
    for (int r = tid; r < ROWS; r += NTHR) {
        const int gr = row0 + r;
        int p = -1, lo = 0;
        float m = -INFINITY, l = 0.f;
        if (gr < nrows) {
            p = static_cast<int>(a.positions[q0 + gr / H]);
            lo = a.window > 0 ? max(0, p - static_cast<int>(a.window) + 1) : 0;
            if (split == 0 && a.sink) {
                m = a.sink[gr % H];
                l = 1.f;
            }
        }
        p_s[r] = p;
        lo_s[r] = lo;
        m_s[r] = m;
        l_s[r] = l;
    }
    // queries -> bfloat16 rows (rows of one sequence are contiguous in q_lat: (token, head) flattened)
    const float *q = a.q_lat + (static_cast<int64_t>(q0) * H + row0) * R;
    for (int i = tid; i < ROWS * (R / 4); i += NTHR) {
        const int r = i / (R / 4), c = (i % (R / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < nrows) v = *reinterpret_cast<const float4 *>(q + static_cast<int64_t>(r) * R + c);
        uint2 w;
        w.x = pack2<__nv_bfloat16>(v.x, v.y);
        w.y = pack2<__nv_bfloat16>(v.z, v.w);
        *reinterpret_cast<uint2 *>(Qs + r * ldc + c) = w;
    }
    // keys of the CTA: from the first row's window start to the last valid row's position
    const int first_p = static_cast<int>(a.positions[q0 + row0 / H]);
    const int last_p = static_cast<int>(a.positions[q0 + (min(row0 + ROWS, nrows) - 1) / H]);
    int k_lo = a.window > 0 ? max(0, first_p - static_cast<int>(a.window) + 1) : 0, k_hi = last_p + 1;
    if (splits > 1) {
        const int n = k_hi - k_lo;
        const int per = ((n + splits - 1) / splits + kTcKeys - 1) / kTcKeys * kTcKeys;
        k_lo = min(k_hi, k_lo + split * per);
        k_hi = min(k_hi, k_lo + per);
    }
    const int chunks = R / 8;   // 16-byte pieces of a latent row
    auto stage = [&](int j0, int buf) {
        __nv_bfloat16 *dst = Cs + buf * kTcKeys * ldc;
        for (int i = tid; i < kTcKeys * chunks; i += NTHR) {
            const int jj = i / chunks, c = (i % chunks) * 8, j = j0 + jj;
            const bool in = j < k_hi;
            const __nv_bfloat16 *src = in ? cache + (static_cast<int64_t>(bt[j / bs]) * bs + j % bs) * R + c : cache;
            cp_async_16(smem_u32(dst + jj * ldc + c), src, in ? 16 : 0);
        }
        cp_async_commit();
    };
    const int Rv = a.out_cols > 0 ? static_cast<int>(a.out_cols) : R;   // columns of the weighted sum that anyone reads
    const int NT = Rv / (8 * NW);              // n8 tiles of this warp's output columns (even)
    float acc[MT][kTcMaxNT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < kTcMaxNT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mt][nt][e] = 0.f;
    const int g = lane >> 2, t4 = lane & 3;
    const int kq = warp & 3, key0 = NW == 8 ? (warp >> 2) * 16 : 0;
    const int col0 = warp * (Rv / NW);
    if (k_lo < k_hi) stage(k_lo, 0);
    int it = 0;
    for (int j0 = k_lo; j0 < k_hi; j0 += kTcKeys, ++it) {
        const int buf = it & 1;
        cp_async_wait_all();
        __syncthreads();
        if (j0 + kTcKeys < k_hi) stage(j0 + kTcKeys, buf ^ 1);
        const __nv_bfloat16 *C = Cs + buf * kTcKeys * ldc;
        // ---- partial scores: all rows x this warp's keys over its quarter of the latent columns ----
        {
            float sc[MT][NKT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int n = 0; n < NKT; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) sc[mt][n][e] = 0.f;
            const int kend = (kq + 1) * (R / 4);
#pragma unroll 2
            for (int kk = kq * (R / 4); kk < kend; kk += 16) {
                uint32_t af[MT][4];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(af[mt], smem_u32(Qs + (mt * 16 + (lane & 15)) * ldc + kk + (lane >> 4) * 8));
#pragma unroll
                for (int nb = 0; nb < NKT / 2; ++nb) {
                    uint32_t bf[4];
                    ldmatrix_x4(bf, smem_u32(C + (key0 + nb * 16 + (lane & 7) + (lane >> 4) * 8) * ldc + kk + ((lane >> 3) & 1) * 8));
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        Mma16816<__nv_bfloat16>::run(sc[mt][2 * nb], af[mt], bf[0], bf[1]);
                        Mma16816<__nv_bfloat16>::run(sc[mt][2 * nb + 1], af[mt], bf[2], bf[3]);
                    }
                }
            }
            float *sp = Sp + kq * ROWS * kSpLd;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int n = 0; n < NKT; ++n) {   // 8-byte stores, row stride 40 floats: a half-warp's stores fall on distinct banks
                    float *s0 = sp + (mt * 16 + g) * kSpLd + key0 + n * 8 + 2 * t4;
                    *reinterpret_cast<float2 *>(s0) = make_float2(sc[mt][n][0], sc[mt][n][1]);
                    *reinterpret_cast<float2 *>(s0 + 8 * kSpLd) = make_float2(sc[mt][n][2], sc[mt][n][3]);
                }
        }
        __syncthreads();
        // ---- running softmax of the rows (lane = key); the four partial tiles are summed in a fixed order ----
#pragma unroll
        for (int r = warp; r < ROWS; r += NW) {      // independent rows: their shuffles and exponentials interleave
            const int j = j0 + lane;
            const bool vis = j < k_hi && j >= lo_s[r] && j <= p_s[r];
            const float raw = (Sp[r * kSpLd + lane] + Sp[(ROWS + r) * kSpLd + lane]) + (Sp[(2 * ROWS + r) * kSpLd + lane] + Sp[(3 * ROWS + r) * kSpLd + lane]);
            const float s = vis ? raw * a.scale : -INFINITY;
            float mx = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_old = m_s[r];
            const float m_new = fmaxf(m_old, mx);
            const float e = vis ? __expf(s - m_new) : 0.f;
            float sum = e;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const float f = m_old == -INFINITY ? 0.f : __expf(m_old - m_new);
            Pb[r * 40 + lane] = __float2bfloat16_rn(e);
            __syncwarp();
            if (lane == 0) {
                m_s[r] = m_new;
                l_s[r] = l_s[r] * f + sum;
                f_s[r] = f;
            }
        }
        __syncthreads();
        // ---- this warp's share of the latent columns for all rows ----
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const float f0 = f_s[mt * 16 + g], f1 = f_s[mt * 16 + g + 8];
#pragma unroll
            for (int nt = 0; nt < kTcMaxNT; ++nt)
                if (nt < NT) {
                    acc[mt][nt][0] *= f0;
                    acc[mt][nt][1] *= f0;
                    acc[mt][nt][2] *= f1;
                    acc[mt][nt][3] *= f1;
                }
        }
#pragma unroll
        for (int kk = 0; kk < kTcKeys; kk += 16) {
            uint32_t pf[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(pf[mt], smem_u32(Pb + (mt * 16 + (lane & 15)) * 40 + kk + (lane >> 4) * 8));
#pragma unroll
            for (int nj = 0; nj < kTcMaxNT / 2; ++nj)
                if (2 * nj < NT) {
                    uint32_t bf[4];
                    ldmatrix_x4_trans(bf, smem_u32(C + (kk + (lane & 7) + ((lane >> 3) & 1) * 8) * ldc + col0 + nj * 16 + (lane >> 4) * 8));
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        Mma16816<__nv_bfloat16>::run(acc[mt][2 * nj], pf[mt], bf[0], bf[1]);
                        Mma16816<__nv_bfloat16>::run(acc[mt][2 * nj + 1], pf[mt], bf[2], bf[3]);
                    }
                }
        }
    }
    __syncthreads();
    // ---- results: row (token, head) -> out[(token * H + head) * R + col] ----
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = mt * 16 + g + half * 8, gr = row0 + r;
            if (gr >= nrows) continue;
            const int64_t flat = static_cast<int64_t>(q0) * H + gr;    // token * H + head
            if (partial) {
                float *o = partial + ((flat / H) * splits + split) * H * R + (flat % H) * R;
#pragma unroll
                for (int nt = 0; nt < kTcMaxNT; ++nt)
                    if (nt < NT) {
                        o[col0 + nt * 8 + 2 * t4] = acc[mt][nt][half * 2];
                        o[col0 + nt * 8 + 2 * t4 + 1] = acc[mt][nt][half * 2 + 1];
                    }
                if (warp == 0 && t4 == 0) {
                    float *ml = partial_ml + (((flat / H) * splits + split) * H + flat % H) * 2;
                    ml[0] = m_s[r];
                    ml[1] = l_s[r];
                }
            } else {
                const float l = l_s[r], inv = l > 0.f ? 1.f / l : 0.f;
                float *o = a.out + flat * R;
#pragma unroll
                for (int nt = 0; nt < kTcMaxNT; ++nt)
                    if (nt < NT) {
                        o[col0 + nt * 8 + 2 * t4] = acc[mt][nt][half * 2] * inv;
                        o[col0 + nt * 8 + 2 * t4 + 1] = acc[mt][nt][half * 2 + 1] * inv;
                    }
            }
        }
}

size_t tc_attn_smem(int mt, int64_t R) {
    const size_t rows = 16 * mt, ldc = R + 8;
    return rows * ldc * 2 + 2 * kTcKeys * ldc * 2 + 4 * rows * kSpLd * 4 + rows * 40 * 2 + rows * 5 * 4;
}

// Splits of one (query, head) are merged in split order: M = max m_k, out = sum_k acc_k e^(m_k - M) / sum_k l_k e^(m_k - M).
// One CTA per (token, head); the factors are formed once per CTA.
__global__ void __launch_bounds__(128) latent_split_reduce_kernel(const float *__restrict__ partial, const float *__restrict__ partial_ml,
                                                                  float *__restrict__ out, int splits, int H, int R) {
    __shared__ float f_s[64];
    __shared__ float den_s;
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x / H;
    const int h = blockIdx.x % H;
    if (threadIdx.x == 0) {
        float M = -INFINITY;
        for (int k = 0; k < splits; ++k) M = fmaxf(M, partial_ml[((t * splits + k) * H + h) * 2]);
        float den = 0.f;
        for (int k = 0; k < splits; ++k) {
            const float m = partial_ml[((t * splits + k) * H + h) * 2];
            const float f = m == -INFINITY ? 0.f : expf(m - M);
            f_s[k] = f;
            den = fmaf(partial_ml[((t * splits + k) * H + h) * 2 + 1], f, den);
        }
        den_s = den;
    }
    __syncthreads();
    const float inv = den_s > 0.f ? 1.f / den_s : 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        float num = 0.f;
        for (int k = 0; k < splits; ++k) num = fmaf(partial[((t * splits + k) * H + h) * R + i], f_s[k], num);
        out[(t * H + h) * R + i] = num * inv;
    }
}

// ---------------------------------------------------------------------------------------------
// Long prompt portions on expanded keys and values: plan (which sequences, which keys), gather of their latents.
// ---------------------------------------------------------------------------------------------
__global__ void latent_expand_plan_kernel(const int32_t *__restrict__ query_start, const int32_t *__restrict__ context_lens, int B,
                                          int window, int min_q, int32_t *__restrict__ cu_k, int32_t *__restrict__ key_lo) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int acc = 0;
    for (int b = 0; b < B; ++b) {
        const int nq = query_start[b + 1] - query_start[b], ctx = context_lens[b];
        int lo = 0, n = 0;
        if (nq >= min_q) {
            lo = window > 0 ? max(0, ctx - window + 1) : 0;   // the first key the portion's first query sees
            n = ctx + nq - lo;
        }
        cu_k[b] = acc;
        key_lo[b] = lo;
        acc += n;
    }
    cu_k[B] = acc;
}

// One warp per gathered row: C[cu_k[b] + i, :] = cache[page(key_lo[b] + i), :]
__global__ void __launch_bounds__(256) latent_gather_kernel(const __nv_bfloat16 *__restrict__ cache, const int32_t *__restrict__ block_tables,
                                                            int64_t max_blocks, const int32_t *__restrict__ cu_k,
                                                            const int32_t *__restrict__ key_lo, __nv_bfloat16 *__restrict__ out, int R,
                                                            int bs) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int n = cu_k[b + 1] - cu_k[b];
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= n) return;
    const int j = key_lo[b] + i;
    const int32_t *bt = block_tables + static_cast<int64_t>(b) * max_blocks;
    const uint4 *src = reinterpret_cast<const uint4 *>(cache + (static_cast<int64_t>(bt[j / bs]) * bs + j % bs) * R);
    uint4 *dst = reinterpret_cast<uint4 *>(out + static_cast<int64_t>(cu_k[b] + i) * R);
    for (int c = threadIdx.x & 31; c < R / 8; c += 32) dst[c] = src[c];
}

}  // namespace

#define HYB_DISPATCH(dtype, CALL) ((dtype) == ATOMA_DTYPE_BF16 ? CALL(__nv_bfloat16) : CALL(float))

bool hyb_latent_norm_cache(const void *proj, int64_t ld, const float *q_w, const float *kv_w, const int64_t *slots, void *cq_out,
                           void *cache, int64_t T, int64_t q_rank, int64_t kv_rank, float eps, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_latent_norm_cache")) return false;
    if (!proj || kv_rank <= 0 || q_rank < 0 || ld < q_rank + kv_rank || !kv_w || (q_rank > 0 && (!q_w || !cq_out)) || (slots && !cache)) {
        set_status(kErrInvalidArg, "atoma_latent_norm_cache: null argument or a row stride below q_rank + kv_rank");
        return false;
    }
#define CALL(TT) launch_ex(latent_norm_cache_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(kRowThreads), 0, stream, \
                           static_cast<const TT *>(proj), ld, q_w, kv_w, slots, static_cast<TT *>(cq_out), static_cast<TT *>(cache), \
                           static_cast<int>(q_rank), static_cast<int>(kv_rank), eps)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "latent_norm_cache_kernel");
#undef CALL
}

// Per-head projection with explicit strides: head h of `in` starts in_hs elements into a row of ld_in, head h of `out`
// out_hs elements into a row of ld_out (so heads that carry more than the projected part, or an output row that keeps
// room for more, need no copies).  w [H n, R] as in atoma_head_project.
bool hyb_head_project_ld(const void *in, int64_t ld_in, int64_t in_hs, const void *w, void *out, int64_t ld_out, int64_t out_hs, int64_t T,
                         int64_t H, int64_t n, int64_t R, int32_t absorb, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_head_project")) return false;
    if (!in || !w || !out || H <= 0 || n <= 0 || R <= 0) {
        set_status(kErrInvalidArg, "atoma_head_project: null argument or empty head");
        return false;
    }
    const int M = static_cast<int>(T);
    cudaError_t e;
    if (dtype == ATOMA_DTYPE_BF16 && !(g_hybrid_debug & 1)) {   // tensor cores: operands rounded to bfloat16, float32 accumulation
        tc::GemmArgs p{};
        p.a = in;
        p.b = static_cast<const __nv_bfloat16 *>(w);
        p.o = out;
        p.b_zs = n * R;
        p.M = M;
        p.lda = ld_in, p.a_zs = in_hs, p.ldo = ld_out, p.o_zs = out_hs;
        if (absorb) {
            p.b_ks = R, p.b_ns = 1, p.N = static_cast<int>(R), p.K = static_cast<int>(n);
            const dim3 grid(static_cast<unsigned>((R + 63) / 64), static_cast<unsigned>((T + 63) / 64), static_cast<unsigned>(H));
            e = launch_ex(tc::gemm_kernel<__nv_bfloat16, float, false>, grid, dim3(128), 0, stream, p);
        } else {
            p.b_ks = 1, p.b_ns = R, p.N = static_cast<int>(n), p.K = static_cast<int>(R);
            const dim3 grid(static_cast<unsigned>((n + 63) / 64), static_cast<unsigned>((T + 63) / 64), static_cast<unsigned>(H));
            e = launch_ex(tc::gemm_kernel<float, __nv_bfloat16, false>, grid, dim3(128), 0, stream, p);
        }
        return hybrid::launched(e, "tc::gemm_kernel<head>");
    }
    if (absorb) {
        const dim3 grid(static_cast<unsigned>((R + 63) / 64), static_cast<unsigned>((T + 63) / 64), static_cast<unsigned>(H));
#define CALL(TT) launch_ex(head_project_kernel<TT, TT, float>, grid, dim3(256), 0, stream, static_cast<const TT *>(in), ld_in, in_hs, \
                           static_cast<const TT *>(w), n * R, R, static_cast<int64_t>(1), static_cast<float *>(out), ld_out, out_hs, M, \
                           static_cast<int>(R), static_cast<int>(n))
        e = HYB_DISPATCH(dtype, CALL);
#undef CALL
    } else {
        const dim3 grid(static_cast<unsigned>((n + 63) / 64), static_cast<unsigned>((T + 63) / 64), static_cast<unsigned>(H));
#define CALL(TT) launch_ex(head_project_kernel<float, TT, TT>, grid, dim3(256), 0, stream, static_cast<const float *>(in), ld_in, in_hs, \
                           static_cast<const TT *>(w), n * R, static_cast<int64_t>(1), R, static_cast<TT *>(out), ld_out, out_hs, M, \
                           static_cast<int>(n), static_cast<int>(R))
        e = HYB_DISPATCH(dtype, CALL);
#undef CALL
    }
    return hybrid::launched(e, "head_project_kernel");
}

bool hyb_head_project(const void *in, const void *w, void *out, int64_t T, int64_t H, int64_t n, int64_t R, int32_t absorb, uint32_t dtype,
                      cudaStream_t stream) {
    if (absorb) return hyb_head_project_ld(in, H * n, n, w, out, H * R, R, T, H, n, R, 1, dtype, stream);
    return hyb_head_project_ld(in, H * R, R, w, out, H * n, n, T, H, n, R, 0, dtype, stream);
}

// The tensor-core kernel takes bfloat16 caches whose rows are a multiple of 64 entries (16-byte rows for cp.async, whole ldmatrix
// tiles per quarter of the row in the score product) and whose summed columns (all of the row, or its first out_cols) are a
// multiple of 64 up to 256 (four warps) or a multiple of 128 up to 512 (eight warps): at most 8 accumulator tiles per warp and row
// tile.  Rows of up to 576 entries fit shared memory.  Everything else runs the general kernel.
bool hyb_latent_attention_tc(const atoma_latent_attn_args &a, cudaStream_t stream, bool *taken) {
    *taken = false;
    const int64_t rv = a.out_cols > 0 ? a.out_cols : a.R;
    const bool four = a.R % 64 == 0 && a.R <= 256 && rv % 64 == 0, eight = a.R % 64 == 0 && a.R > 256 && a.R <= 576 && rv % 128 == 0 && rv <= 512;
    if (a.dtype != ATOMA_DTYPE_BF16 || (g_hybrid_debug & 2) || !(four || eight) || !a.query_start || a.max_query_len <= 0 ||
        (reinterpret_cast<uintptr_t>(a.latent_cache) & 15) || (reinterpret_cast<uintptr_t>(a.q_lat) & 15) ||
        current_device_info().cc_major < 8)
        return true;
    *taken = true;
    const int64_t need_rows = static_cast<int64_t>(a.max_query_len) * a.H;
    int mt = 4;                                                    // measured: 64 rows per CTA beat 32 by 1.3x (per-tile barriers and staging amortise)
    while (mt > 1 && 16 * (mt / 2) >= need_rows) mt /= 2;          // no more rows than the longest portion has
    const int rows = 16 * mt;
    const unsigned gx = static_cast<unsigned>((need_rows + rows - 1) / rows);
    // few CTAs over many keys (decode steps): split the keys
    int64_t span = a.max_seq_len > 0 ? a.max_seq_len : 0;
    if (a.window > 0) span = std::min<int64_t>(span, a.window + a.max_query_len);
    int splits = 1;
    const int64_t ctas = static_cast<int64_t>(gx) * a.B;
    if (span >= 8 * kTcKeys && ctas < current_device_info().sm_count)
        splits = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>({(2 * current_device_info().sm_count + ctas - 1) / ctas,
                                                                         (span + 4 * kTcKeys - 1) / (4 * kTcKeys), 64})));
    float *partial = nullptr, *partial_ml = nullptr;
    if (splits > 1) {
        const size_t n_acc = static_cast<size_t>(a.T) * splits * a.H * a.R, n_ml = static_cast<size_t>(a.T) * splits * a.H * 2;
        partial = static_cast<float *>(get_workspace(stream, (n_acc + n_ml) * 4, kWorkspaceHybridAttn));
        if (!partial) return false;
        partial_ml = partial + n_acc;
    }
    const size_t smem = tc_attn_smem(mt, a.R);
    const dim3 grid(gx, static_cast<unsigned>(a.B), static_cast<unsigned>(splits));
    cudaError_t e;
#define LAUNCH_TC(M, N)                                                                                                          \
    {                                                                                                                            \
        if (smem > 48 * 1024) cudaFuncSetAttribute(latent_attn_tc_kernel<M, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
        e = launch_ex(latent_attn_tc_kernel<M, N>, grid, dim3(32 * N), smem, stream, a, splits, partial, partial_ml);            \
    }
    if (four) {
        if (mt == 4) LAUNCH_TC(4, 4) else if (mt == 2) LAUNCH_TC(2, 4) else LAUNCH_TC(1, 4)
    } else {
        if (mt == 4) LAUNCH_TC(4, 8) else if (mt == 2) LAUNCH_TC(2, 8) else LAUNCH_TC(1, 8)
    }
#undef LAUNCH_TC
    if (!hybrid::launched(e, "latent_attn_tc_kernel")) return false;
    if (splits == 1) return true;
    return hybrid::launched(launch_ex(latent_split_reduce_kernel, dim3(static_cast<unsigned>(a.T * a.H)), dim3(128), 0, stream,
                                      static_cast<const float *>(partial), static_cast<const float *>(partial_ml), a.out, splits,
                                      static_cast<int>(a.H), static_cast<int>(a.R)),
                            "latent_split_reduce_kernel");
}

bool hyb_latent_attention(const atoma_latent_attn_args &a, cudaStream_t stream) {
    if (a.T <= 0) return true;
    if (!hybrid::known_dtype(a.dtype, "atoma_latent_attention_paged")) return false;
    if (!a.q_lat || !a.latent_cache || !a.out || !a.positions || !a.token_seq || !a.block_tables || a.H <= 0 || a.R <= 0 ||
        a.block_size <= 0 || a.max_blocks <= 0 || a.out_cols < 0 || a.out_cols > a.R) {
        set_status(kErrInvalidArg, "atoma_latent_attention_paged: null argument or empty shape");
        return false;
    }
    bool taken = false;
    const bool ok = hyb_latent_attention_tc(a, stream, &taken);
    if (taken || !ok) return ok;
    if (a.R > kLatThreads * kLatMaxOut) {
        set_status(kErrUnsupported, "atoma_latent_attention_paged: a latent size of %lld exceeds %d", static_cast<long long>(a.R),
                   kLatThreads * kLatMaxOut);
        return false;
    }
    const int head_chunk = static_cast<int>(std::min<int64_t>(a.H, kLatThreads * kLatMaxOut / a.R));
    const unsigned head_chunks = static_cast<unsigned>((a.H + head_chunk - 1) / head_chunk);
    const size_t smem = static_cast<size_t>(head_chunk * a.R + kLatKeys * (a.R + 1) + head_chunk * kLatKeys + 3 * head_chunk) * 4;
    if (smem > 200 * 1024) {
        set_status(kErrUnsupported, "atoma_latent_attention_paged: %zu bytes of shared memory", smem);
        return false;
    }
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(latent_attn_general_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(latent_attn_general_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
    // few query tokens over many keys (decode steps): split the keys so that the device is filled
    int64_t span = a.max_seq_len > 0 ? a.max_seq_len : 0;
    if (a.window > 0) span = std::min<int64_t>(span, a.window);
    int splits = 1;
    if (span >= 4 * kLatKeys && !(g_hybrid_debug & 2)) {
        const int64_t want = (2 * current_device_info().sm_count + a.T - 1) / a.T;
        splits = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>({want, (span + 2 * kLatKeys - 1) / (2 * kLatKeys), 64})));
    }
    float *partial = nullptr, *partial_ml = nullptr;
    if (splits > 1) {
        const size_t n_acc = static_cast<size_t>(a.T) * splits * a.H * a.R, n_ml = static_cast<size_t>(a.T) * splits * a.H * 2;
        partial = static_cast<float *>(get_workspace(stream, (n_acc + n_ml) * 4, kWorkspaceHybridAttn));
        if (!partial) return false;
        partial_ml = partial + n_acc;
    }
    const dim3 grid(static_cast<unsigned>(a.T), static_cast<unsigned>(splits), head_chunks);
#define CALL(TT) launch_ex(latent_attn_general_kernel<TT>, grid, dim3(kLatThreads), smem, stream, a, splits, head_chunk, partial, partial_ml)
    if (!hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "latent_attn_general_kernel")) return false;
#undef CALL
    if (splits == 1) return true;
    return hybrid::launched(launch_ex(latent_split_reduce_kernel, dim3(static_cast<unsigned>(a.T * a.H)), dim3(128), 0, stream,
                                      static_cast<const float *>(partial), static_cast<const float *>(partial_ml), a.out, splits,
                                      static_cast<int>(a.H), static_cast<int>(a.R)),
                            "latent_split_reduce_kernel");
}


// Shapes the expanded path takes: bfloat16, equal key and value head sizes of 64 or 128, 16-byte latent rows, sm_100.
bool hyb_latent_expanded_ok(int64_t dim, int64_t vdim, int64_t R, uint32_t dtype) {
    return dtype == ATOMA_DTYPE_BF16 && dim == vdim && (dim == 64 || dim == 128) && R % 8 == 0 && current_device_info().cc_major == 10 &&
           !(g_hybrid_debug & 2);
}

bool hyb_latent_attention_expanded(const atoma_latent_expanded_args &a, cudaStream_t stream) {
    if (a.T <= 0 || a.B <= 0 || a.max_keys <= 0) return true;
    if (!a.q || !a.latent_cache || !a.w_uk || !a.w_uv || !a.out || !a.query_start || !a.context_lens || !a.block_tables || a.H <= 0 ||
        a.min_q < 32 || !hyb_latent_expanded_ok(a.dim, a.dim, a.R, ATOMA_DTYPE_BF16)) {
        set_status(kErrInvalidArg, "atoma_latent_attention_expanded: null argument, or a shape outside bfloat16 heads of 64 / 128 with min_q >= 32");
        return false;
    }
    const int64_t HD = a.H * a.dim;
    auto up = [](int64_t x) { return (x + 255) / 256 * 256; };
    const int64_t rows = a.max_keys + 128;   // the attention kernel's TMA boxes may start up to a tile before the end
    const int64_t b_int = up((2 * a.B + 2) * 4), b_c = up(rows * a.R * 2), b_kv = up(rows * HD * 2);
    char *ws = static_cast<char *>(get_workspace(stream, static_cast<size_t>(b_int + b_c + 2 * b_kv), kWorkspaceLatentExpand));
    if (!ws) return false;
    int32_t *cu_k = reinterpret_cast<int32_t *>(ws), *key_lo = cu_k + a.B + 1;
    __nv_bfloat16 *C = reinterpret_cast<__nv_bfloat16 *>(ws + b_int);
    __nv_bfloat16 *K = reinterpret_cast<__nv_bfloat16 *>(ws + b_int + b_c), *V = reinterpret_cast<__nv_bfloat16 *>(ws + b_int + b_c + b_kv);
    if (!hybrid::launched(launch_ex(latent_expand_plan_kernel, dim3(1), dim3(32), 0, stream, a.query_start, a.context_lens,
                                    static_cast<int>(a.B), static_cast<int>(a.window), static_cast<int>(a.min_q), cu_k, key_lo),
                          "latent_expand_plan_kernel"))
        return false;
    const int64_t span = a.window > 0 ? std::min<int64_t>(a.max_seq_len, a.window - 1 + a.max_query_len) : a.max_seq_len;
    const dim3 gg(static_cast<unsigned>((span + 7) / 8), static_cast<unsigned>(a.B));
    if (!hybrid::launched(launch_ex(latent_gather_kernel, gg, dim3(256), 0, stream, static_cast<const __nv_bfloat16 *>(a.latent_cache),
                                    a.block_tables, a.max_blocks, static_cast<const int32_t *>(cu_k), static_cast<const int32_t *>(key_lo), C,
                                    static_cast<int>(a.R), static_cast<int>(a.block_size)),
                          "latent_gather_kernel"))
        return false;
    if (!hyb_linear(C, a.w_uk, K, a.max_keys, HD, a.R, ATOMA_DTYPE_BF16, stream)) return false;
    if (!hyb_linear(C, a.w_uv, V, a.max_keys, HD, a.R, ATOMA_DTYPE_BF16, stream)) return false;
    MhaParams p;
    std::memset(&p, 0, sizeof(p));
    p.q = a.q, p.k = K, p.v = V, p.o = a.out;
    p.cu_q = a.query_start, p.cu_k = cu_k;
    p.q_rs = p.k_rs = p.v_rs = p.o_rs = HD;
    p.q_hs = p.k_hs = p.v_hs = p.o_hs = a.dim;
    p.b = static_cast<int>(a.B), p.h = p.h_k = static_cast<int>(a.H), p.d = static_cast<int>(a.dim);
    p.seqlen_q = a.max_query_len, p.seqlen_k = static_cast<int>(span);
    p.page = 1;
    p.scale = a.scale, p.scale_log2 = a.scale * 1.4426950408889634f;
    p.is_causal = 1, p.k_cumulative = 1;
    p.window_left = static_cast<int>(a.window), p.min_len_q = a.min_q, p.sink = a.sink;
    const int r = try_launch_prefill_tc(p, true, stream);
    if (r == 1) return true;
    if (r == 0) set_status(kErrUnsupported, "atoma_latent_attention_expanded: the step is outside the tensor-memory attention kernel's envelope");
    return false;
}

}  // namespace atoma

using namespace atoma;

extern "C" void atoma_latent_norm_cache(const void *proj, int64_t ld, const float *q_weight, const float *kv_weight,
                                        const int64_t *slot_mapping, void *cq_out, void *latent_cache, int64_t T, int64_t q_rank,
                                        int64_t kv_rank, float eps, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_latent_norm_cache(proj, ld, q_weight, kv_weight, slot_mapping, cq_out, latent_cache, T, q_rank, kv_rank, eps, dtype,
                          static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_head_project(const void *in, const void *w, void *out, int64_t T, int64_t H, int64_t n, int64_t R, int32_t absorb,
                                   uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_head_project(in, w, out, T, H, n, R, absorb, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_latent_attention_expanded(const atoma_latent_expanded_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_latent_attention_expanded: args is NULL");
        return;
    }
    hyb_latent_attention_expanded(*args, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_latent_attention_paged(const atoma_latent_attn_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_latent_attention_paged: args is NULL");
        return;
    }
    hyb_latent_attention(*args, static_cast<cudaStream_t>(stream));
}
