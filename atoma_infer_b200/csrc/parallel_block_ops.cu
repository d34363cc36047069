// Operators of PARALLEL decoder blocks and their mixers — include/atoma_hybrid.h.
//
// A parallel block norms the residual stream once; the mixer and the feed-forward both read that row, each through a
// causal tap filter over time, and both results join the stream in one update (fused here with whatever precedes the next
// layer and with its input norm).  The mixers that need more than attention kernels:
//   - tap filters whose inputs before a portion come from a per-sequence history (the portion's last inputs replace it),
//   - matrix-state recurrences (gated linear attention, gated delta rule): every head keeps S [dim, vdim] in float32; the
//     columns of S are independent in both recurrences, so a CTA owns 32 columns of one head of one sequence, the rows
//     of a column are spread over `parts` threads (registers), and the tokens are visited strictly in order,
//   - rotary positions on queries, keys and values with the cache write, the turn-back of a head's sum, and the
//     latent-attention variants that keep one rotated key part beside the latent.
// Statistics, angles, decays, gates of the recurrences and the state are float32 whatever the activation format; every
// result is reduced in an order that depends on the token alone, never on the batch around it.
#include "common.cuh"
#include "hybrid_common.cuh"

#include "atoma_hybrid.h"

#include <algorithm>

namespace atoma {

extern int g_hybrid_debug;   // bit 1: general kernels only; bit 4: scans with many rows per lane
bool hyb_head_project_ld(const void *, int64_t, int64_t, const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int32_t,
                         uint32_t, cudaStream_t);   // latent_attention.cu

namespace {

using namespace hybrid;

constexpr int kMaxTaps = 16;

// ---------------------------------------------------------------------------------------------
// residual update of a parallel block + what precedes the next layer + its input norm
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kRowThreads) parallel_residual_norm_kernel(const atoma_parallel_residual_args a) {
    extern __shared__ float row[];
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int W = static_cast<int>(a.width);
    const T *ya = a.y_a ? static_cast<const T *>(a.y_a) + t * W : nullptr;
    const T *yb = a.y_b ? static_cast<const T *>(a.y_b) + t * W : nullptr;
    const T *yf = a.y_ff ? static_cast<const T *>(a.y_ff) + t * W : nullptr;
    float inv_a = 1.f, inv_b = 1.f;
    if (ya && a.norm_a) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < W; c += blockDim.x) {
            const float v = to_f(ya[c]);
            ss = fmaf(v, v, ss);
        }
        inv_a = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(W) + a.eps);
    }
    if (yb && a.norm_b) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < W; c += blockDim.x) {
            const float v = to_f(yb[c]);
            ss = fmaf(v, v, ss);
        }
        inv_b = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(W) + a.eps);
    }
    float *x = a.x + t * W;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float m = 0.f;
        if (ya) m += a.norm_a ? to_f(ya[c]) * inv_a * a.norm_a[c] : to_f(ya[c]);
        if (yb) m += a.norm_b ? to_f(yb[c]) * inv_b * a.norm_b[c] : to_f(yb[c]);
        float v = x[c] + a.mix_scale * m;
        if (yf) v += to_f(yf[c]);
        if (a.trace) a.trace[t * W + c] = v;
        if (a.add_rows) v += a.add_rows[t * W + c];
        if (a.add_vec) v += a.add_vec[c];
        x[c] = v;
        row[c] = v;
        ss = fmaf(v, v, ss);
    }
    if (!a.w_next) return;
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(W) + a.eps);
    T *h = static_cast<T *>(a.h) + t * W;
    for (int c = threadIdx.x; c < W; c += blockDim.x) h[c] = from_f<T>(row[c] * inv * (a.weight_offset + a.w_next[c]));
}

// ---------------------------------------------------------------------------------------------
// tap filters with carried inputs
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) tap_filter_kernel(const atoma_tap_filter_args a) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int C = static_cast<int>(a.channels), taps = static_cast<int>(a.taps);
    if (c >= C) return;
    const int b = a.token_seq[t];
    const int i = static_cast<int>(t) - a.query_start[b];     // index inside the portion
    const int ctx = a.context_lens[b];
    const T *in = static_cast<const T *>(a.in);
    const float *hist = a.history ? a.history + static_cast<int64_t>(a.state_slots[b]) * a.history_stride : nullptr;
    const float cur = to_f(in[t * a.ld_in + c]);
    float f1 = 0.f, f2 = 0.f;
    for (int j = 0; j + 1 < taps; ++j) {
        const int back = taps - 1 - j;
        float v = 0.f;
        if (i - back >= 0) v = to_f(in[(t - back) * a.ld_in + c]);
        else if (ctx + i - back >= 0 && hist) v = hist[static_cast<int64_t>(taps - 1 + i - back) * C + c];
        f1 = fmaf(a.w1[c * taps + j], v, f1);
        if (a.w2) f2 = fmaf(a.w2[c * taps + j], v, f2);
    }
    f1 = fmaf(a.w1[c * taps + taps - 1], cur, f1);
    if (a.residual) f1 += cur;
    if (a.act == 1) f1 = silu(f1);
    static_cast<T *>(a.out1)[t * a.ld_out + c] = from_f<T>(f1);
    if (a.w2) {
        f2 = fmaf(a.w2[c * taps + taps - 1], cur, f2);
        if (a.residual) f2 += cur;
        if (a.act == 1) f2 = silu(f2);
        static_cast<T *>(a.out2)[t * a.ld_out + c] = from_f<T>(f2);
    }
}

// The same filter for bfloat16 rows of 16-byte pieces: a thread owns 8 neighbouring channels and `run` consecutive tokens, keeps
// the filters' weights and the last TAPS - 1 inputs in registers, and slides that window from token to token; it is filled anew
// at the run's first token and wherever a portion starts (from the rows before, the sequence's carried inputs, or zeros).
// Per element the products are added in the order of the kernel above, so both give the same bits.
template <int TAPS>
__global__ void __launch_bounds__(128) tap_filter_vec_kernel(const atoma_tap_filter_args a, int run) {
    pdl_launch_dependents();
    pdl_wait();
    const int C = static_cast<int>(a.channels), T = static_cast<int>(a.T);
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c0 >= C) return;
    const int t_first = blockIdx.y * run, t_end = min(T, t_first + run);
    const __nv_bfloat16 *in = static_cast<const __nv_bfloat16 *>(a.in);
    float w1[8][TAPS], w2[8][TAPS];
    {
        const float4 *p1 = reinterpret_cast<const float4 *>(a.w1 + static_cast<int64_t>(c0) * TAPS);
        const float4 *p2 = a.w2 ? reinterpret_cast<const float4 *>(a.w2 + static_cast<int64_t>(c0) * TAPS) : p1;
#pragma unroll
        for (int i = 0; i < 2 * TAPS; ++i) {
            const float4 x = p1[i], y = p2[i];
            const float xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                w1[(4 * i + e) / TAPS][(4 * i + e) % TAPS] = xs[e];
                w2[(4 * i + e) / TAPS][(4 * i + e) % TAPS] = ys[e];
            }
        }
    }
    auto row8 = [&](int64_t t, float *v) {
        const uint4 r = *reinterpret_cast<const uint4 *>(in + t * a.ld_in + c0);
        const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            v[2 * e] = __uint_as_float(u[e] << 16);
            v[2 * e + 1] = __uint_as_float(u[e] & 0xffff0000u);
        }
    };
    float win[TAPS > 1 ? TAPS - 1 : 1][8];                     // win[k]: the input TAPS - 1 - k tokens back
    for (int t = t_first; t < t_end; ++t) {
        const int b = a.token_seq[t];
        const int i = t - a.query_start[b];
        if (TAPS > 1 && (t == t_first || i == 0)) {
            const int ctx = a.context_lens[b];
            const float *hist = a.history ? a.history + static_cast<int64_t>(a.state_slots[b]) * a.history_stride : nullptr;
#pragma unroll
            for (int k = 0; k < TAPS - 1; ++k) {
                const int back = TAPS - 1 - k;
                if (i - back >= 0) {
                    row8(t - back, win[k]);
                } else if (ctx + i - back >= 0 && hist) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) win[k][e] = hist[static_cast<int64_t>(TAPS - 1 + i - back) * C + c0 + e];
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) win[k][e] = 0.f;
                }
            }
        }
        float cur[8], f1[8], f2[8];
        row8(t, cur);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float x = 0.f, y = 0.f;
#pragma unroll
            for (int k = 0; k < TAPS - 1; ++k) {
                x = fmaf(w1[e][k], win[k][e], x);
                y = fmaf(w2[e][k], win[k][e], y);
            }
            x = fmaf(w1[e][TAPS - 1], cur[e], x);
            y = fmaf(w2[e][TAPS - 1], cur[e], y);
            if (a.residual) {
                x += cur[e];
                y += cur[e];
            }
            if (a.act == 1) {
                x = silu(x);
                y = silu(y);
            }
            f1[e] = x;
            f2[e] = y;
        }
        uint4 o;
        o.x = pack2<__nv_bfloat16>(f1[0], f1[1]);
        o.y = pack2<__nv_bfloat16>(f1[2], f1[3]);
        o.z = pack2<__nv_bfloat16>(f1[4], f1[5]);
        o.w = pack2<__nv_bfloat16>(f1[6], f1[7]);
        *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(a.out1) + static_cast<int64_t>(t) * a.ld_out + c0) = o;
        if (a.w2) {
            o.x = pack2<__nv_bfloat16>(f2[0], f2[1]);
            o.y = pack2<__nv_bfloat16>(f2[2], f2[3]);
            o.z = pack2<__nv_bfloat16>(f2[4], f2[5]);
            o.w = pack2<__nv_bfloat16>(f2[6], f2[7]);
            *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(a.out2) + static_cast<int64_t>(t) * a.ld_out + c0) = o;
        }
#pragma unroll
        for (int k = 0; k + 1 < TAPS - 1; ++k)
#pragma unroll
            for (int e = 0; e < 8; ++e) win[k][e] = win[k + 1][e];
        if (TAPS > 1) {
#pragma unroll
            for (int e = 0; e < 8; ++e) win[TAPS - 2][e] = cur[e];
        }
    }
}

// history[k] <- the sequence's input at position (context + n) - (taps - 1) + k, from the portion or from the old history
template <typename T>
__global__ void __launch_bounds__(256) tap_history_kernel(const atoma_tap_filter_args a) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int C = static_cast<int>(a.channels), keep = static_cast<int>(a.taps) - 1;
    if (c >= C) return;
    const int q0 = a.query_start[b], n = a.query_start[b + 1] - q0, ctx = a.context_lens[b];
    if (n <= 0) return;
    float *hist = a.history + static_cast<int64_t>(a.state_slots[b]) * a.history_stride;
    const T *in = static_cast<const T *>(a.in);
    float old[kMaxTaps];
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) old[k] = (k < keep && k + n < keep && ctx - keep + k + n >= 0) ? hist[static_cast<int64_t>(k + n) * C + c] : 0.f;
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) {
        if (k >= keep) break;
        const int rel = n - keep + k;
        hist[static_cast<int64_t>(k) * C + c] = rel >= 0 ? to_f(in[static_cast<int64_t>(q0 + rel) * a.ld_in + c]) : old[k];
    }
}

// ---------------------------------------------------------------------------------------------
// matrix-state recurrences
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// One CTA = kScanWarps compute warps + kScanWarps staging warps for 32 * kScanWarps / PW columns of one head of one sequence.
// A compute warp owns 32 / PW columns; the dim rows of a column are spread over PW lanes (RPT registers each), so the sums over
// the rows are PW-lane shuffles in a fixed order and the token loop has no CTA-wide barrier.  While the compute warps walk through
// one chunk of staged tokens, the staging warps load the next one (number-format conversion, the decays' exponentials, the unit
// norms of q and k) into the other buffer; one barrier per chunk.
// Staged row of a token: element i of q / k / decay at (i / RPT) * (RPT + 4) + i % RPT — a lane's RPT values are contiguous and
// 16-byte aligned (float4 loads), and the PW lanes of a column read distinct banks.
// Two splits per key size: many rows per lane (few instructions per state entry: steps with many CTAs) and 8 rows per lane (a
// short chain per token and four times the warps: steps with few).  Both add in the same order, so they give the same bits.
constexpr int kScanWarps = 4;

template <int PW>
__device__ __forceinline__ float parts_sum(float v) {
#pragma unroll
    for (int o = 32 / PW; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T, int KIND, int RPT, int PW>
__global__ void __launch_bounds__(64 * kScanWarps, 2) state_scan_kernel(const atoma_state_scan_args a, int chunk) {
    extern __shared__ __align__(16) float sm[];
    constexpr int CW = 32 / PW, COLS = CW * kScanWarps, DS = PW * (RPT + 4);
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, b = blockIdx.z;
    const int D = static_cast<int>(a.dim), V = static_cast<int>(a.vdim), H = static_cast<int>(a.H);
    const int q0 = a.query_start[b], n = a.query_start[b + 1] - q0;
    if (n <= 0) return;
    const int per_tok = (KIND == 0 ? 3 : 2) * DS + COLS + 4;     // q, k, (decay per channel), v of the CTA's columns, beta and decay
    for (int i = threadIdx.x; i < 2 * chunk * per_tok; i += blockDim.x) sm[i] = 0.f;   // what lies beyond dim stays zero
    const int kvh = KIND == 1 ? h / (H / static_cast<int>(a.G)) : h;
    const T *qp = static_cast<const T *>(a.q), *kp = static_cast<const T *>(a.k), *vp = static_cast<const T *>(a.v);
    const int jb = blockIdx.x * COLS;
    const bool loader = warp >= kScanWarps;
    // ---- staging (all warps for the first chunk, the staging warps afterwards) ----
    // A warp takes TU tokens at a time: every load of the TU tokens is issued before the first value is used, so a chunk costs a
    // few round trips to memory, not one per token.  Lane l holds elements l, l + 32, ... of a token's q / k / decay rows; the sums
    // of squares run over a lane's elements in index order, then over the lanes by xor-shuffles: the same order for every token,
    // wherever it falls in a chunk or a batch.
    constexpr int EPL = RPT * PW / 32;                           // elements of a row per lane
    constexpr int TU = EPL <= 4 ? 4 : (EPL == 8 ? 2 : 1);
    const int vcol = (lane < COLS && jb + lane < V) ? jb + lane : -1;
    float zb[EPL];                                               // what does not change from token to token
    float neg_rate = 0.f, dtb = 0.f;
    if (KIND == 0) {
#pragma unroll
        for (int e = 0; e < EPL; ++e) zb[e] = lane + 32 * e < D ? a.z_bias[h * D + lane + 32 * e] : 0.f;
    } else {
        neg_rate = -expf(a.a_log[h]);
        dtb = a.dt_bias[h];
    }
    const float inv_tau = 1.0f / a.tau;
    auto stage = [&](int t0, float *buf, int w, int nw) {
        const int nt = min(chunk, n - t0);
        for (int tk0 = w * TU; tk0 < nt; tk0 += nw * TU) {
            // every address is valid (a token beyond the chunk reads the chunk's last, an element beyond dim reads element 0), so
            // the loads carry no branches and all of them are in flight together
            T qr[TU][EPL], kr[TU][EPL], zr[KIND == 0 ? TU : 1][KIND == 0 ? EPL : 1], vr[TU], br[TU], ar[TU];
#pragma unroll
            for (int u = 0; u < TU; ++u) {
                const int64_t t = q0 + t0 + min(tk0 + u, nt - 1);
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    const int i = lane + 32 * e < D ? lane + 32 * e : 0;
                    qr[u][e] = qp[t * a.ld_q + kvh * D + i];
                    kr[u][e] = kp[t * a.ld_k + kvh * D + i];
                    if (KIND == 0) zr[u][e] = static_cast<const T *>(a.z)[t * a.ld_z + h * D + i];
                }
                vr[u] = vp[t * a.ld_v + h * V + max(vcol, 0)];
                if (KIND == 1) {
                    br[u] = static_cast<const T *>(a.b_pre)[t * a.ld_b + h];
                    ar[u] = static_cast<const T *>(a.a_pre)[t * a.ld_a + h];
                }
            }
#pragma unroll
            for (int u = 0; u < TU; ++u) {
                if (tk0 + u >= nt) break;
                float *row = buf + (tk0 + u) * per_tok;
                float qv[EPL], kv[EPL];
                float sq = 0.f, sk = 0.f, dot = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    const bool in = lane + 32 * e < D;
                    qv[e] = in ? to_f(qr[u][e]) : 0.f;
                    kv[e] = in ? to_f(kr[u][e]) : 0.f;
                    sq = fmaf(qv[e], qv[e], sq);
                    sk = fmaf(kv[e], kv[e], sk);
                    dot = fmaf(qv[e], kv[e], dot);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    if (KIND == 1) {
                        sq += __shfl_xor_sync(0xffffffffu, sq, o);
                        sk += __shfl_xor_sync(0xffffffffu, sk, o);
                    }
                    dot += __shfl_xor_sync(0xffffffffu, dot, o);
                }
                float fq = a.q_scale, fk = 1.f;
                if (KIND == 1) {
                    fq = a.q_scale / sqrtf(sq + a.unit_eps);     // unit length per head, the query scaled
                    fk = 1.0f / sqrtf(sk + a.unit_eps);
                }
                if (lane == 0) {
                    if (KIND == 1) {
                        row[per_tok - 4] = sigmoidf_(to_f(br[u]));
                        row[per_tok - 3] = expf(neg_rate * softplusf_(to_f(ar[u]) + dtb));
                    }
                    row[per_tok - 2] = dot * fq * fk;            // q . k of the token as the recurrence sees them
                }
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    const int i = lane + 32 * e;
                    if (i < D) {
                        const int o = (i / RPT) * (RPT + 4) + i % RPT;
                        if (KIND == 0) {
                            const float decay = expf(log_sigmoid(to_f(zr[u][e]) + zb[e]) * inv_tau);
                            row[o] = qv[e] * fq * decay;         // the read-out of the updated state, written on the old one (see below)
                            row[2 * DS + o] = decay;
                        } else {
                            row[o] = qv[e] * fq;
                        }
                        row[DS + o] = kv[e] * fk;
                    }
                }
                if (lane < COLS) row[(KIND == 0 ? 3 : 2) * DS + lane] = vcol >= 0 ? to_f(vr[u]) : 0.f;
            }
        }
    };
    // ---- the state of this lane: rows part * RPT + r of column j ----
    const int part = lane / CW, j = jb + (warp % kScanWarps) * CW + lane % CW;
    float *S_g = a.state + static_cast<int64_t>(a.state_slots[b]) * a.state_stride + static_cast<int64_t>(h) * D * V;
    float S[RPT];
    const bool fresh = a.context_lens[b] == 0;
    if (!loader) {
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
            const int i = part * RPT + r;
            S[r] = (!fresh && i < D && j < V) ? S_g[static_cast<int64_t>(i) * V + j] : 0.f;
        }
    }
    __syncthreads();                                         // the zero fill is done
    stage(0, sm, warp, 2 * kScanWarps);
    __syncthreads();
    int it = 0;
    for (int t0 = 0; t0 < n; t0 += chunk, ++it) {
        const float *buf = sm + (it & 1) * chunk * per_tok;
        if (loader) {
            if (t0 + chunk < n) stage(t0 + chunk, sm + ((it + 1) & 1) * chunk * per_tok, warp - kScanWarps, kScanWarps);
        } else {
            const int nt = min(chunk, n - t0);
            for (int tk = 0; tk < nt; ++tk) {
                const float *row = buf + tk * per_tok;
                const float4 *qr = reinterpret_cast<const float4 *>(row + part * (RPT + 4));
                const float4 *kr = reinterpret_cast<const float4 *>(row + DS + part * (RPT + 4));
                const float vj = row[(KIND == 0 ? 3 : 2) * DS + (warp % kScanWarps) * CW + lane % CW];
                float o;
                // Both recurrences read the state AFTER the token's write.  With S' = A S + k w^T (A the decay, w the written row):
                // S'^T q = S^T (A q) + (k . q) w, so the sums over the rows run on the state as the previous token left it and the
                // write is the only step between two tokens.
                // Order of a sum over the rows, the same for every split of the rows over lanes: groups of 8 rows (four partial sums
                // over rows m, m + 4, added as (0 + 1) + (2 + 3)), then a binary tree over the groups — inside a lane first, then by
                // xor-shuffles over the lanes of the column.
                constexpr int G8 = RPT / 8;
                const float kq = row[per_tok - 2];
                if (KIND == 0) {
                    const float4 *ar = reinterpret_cast<const float4 *>(row + 2 * DS + part * (RPT + 4));
                    float gs[G8];
#pragma unroll
                    for (int g8 = 0; g8 < G8; ++g8) {
                        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int r4 = 2 * g8; r4 < 2 * g8 + 2; ++r4) {
                            const float4 a4 = ar[r4], k4 = kr[r4], q4 = qr[r4];     // q4: the query times the decay
                            c[0] = fmaf(S[4 * r4], q4.x, c[0]);
                            S[4 * r4] = fmaf(a4.x, S[4 * r4], k4.x * vj);
                            c[1] = fmaf(S[4 * r4 + 1], q4.y, c[1]);
                            S[4 * r4 + 1] = fmaf(a4.y, S[4 * r4 + 1], k4.y * vj);
                            c[2] = fmaf(S[4 * r4 + 2], q4.z, c[2]);
                            S[4 * r4 + 2] = fmaf(a4.z, S[4 * r4 + 2], k4.z * vj);
                            c[3] = fmaf(S[4 * r4 + 3], q4.w, c[3]);
                            S[4 * r4 + 3] = fmaf(a4.w, S[4 * r4 + 3], k4.w * vj);
                        }
                        gs[g8] = (c[0] + c[1]) + (c[2] + c[3]);
                    }
#pragma unroll
                    for (int w = 1; w < G8; w <<= 1)
#pragma unroll
                        for (int g8 = 0; g8 < G8; g8 += 2 * w) gs[g8] += gs[g8 + w];
                    o = fmaf(kq, vj, parts_sum<PW>(gs[0]));
                } else {
                    const float beta = row[per_tok - 4], g = row[per_tok - 3];
                    float gk[G8], gq[G8];
#pragma unroll
                    for (int g8 = 0; g8 < G8; ++g8) {
                        float c[4] = {0.f, 0.f, 0.f, 0.f}, d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int r4 = 2 * g8; r4 < 2 * g8 + 2; ++r4) {
                            const float4 k4 = kr[r4], q4 = qr[r4];
                            c[0] = fmaf(S[4 * r4], k4.x, c[0]);
                            d[0] = fmaf(S[4 * r4], q4.x, d[0]);
                            c[1] = fmaf(S[4 * r4 + 1], k4.y, c[1]);
                            d[1] = fmaf(S[4 * r4 + 1], q4.y, d[1]);
                            c[2] = fmaf(S[4 * r4 + 2], k4.z, c[2]);
                            d[2] = fmaf(S[4 * r4 + 2], q4.z, d[2]);
                            c[3] = fmaf(S[4 * r4 + 3], k4.w, c[3]);
                            d[3] = fmaf(S[4 * r4 + 3], q4.w, d[3]);
                        }
                        gk[g8] = (c[0] + c[1]) + (c[2] + c[3]);
                        gq[g8] = (d[0] + d[1]) + (d[2] + d[3]);
                    }
#pragma unroll
                    for (int w = 1; w < G8; w <<= 1)
#pragma unroll
                        for (int g8 = 0; g8 < G8; g8 += 2 * w) {
                            gk[g8] += gk[g8 + w];
                            gq[g8] += gq[g8 + w];
                        }
                    float sk = gk[0], sq = gq[0];
#pragma unroll
                    for (int x = 32 / PW; x < 32; x <<= 1) {
                        sk += __shfl_xor_sync(0xffffffffu, sk, x);
                        sq += __shfl_xor_sync(0xffffffffu, sq, x);
                    }
                    const float u = beta * (vj - g * sk);        // the decayed state's answer to k
                    o = fmaf(g, sq, u * kq);
#pragma unroll
                    for (int r4 = 0; r4 < RPT / 4; ++r4) {
                        const float4 k4 = kr[r4];
                        S[4 * r4] = fmaf(g, S[4 * r4], k4.x * u);
                        S[4 * r4 + 1] = fmaf(g, S[4 * r4 + 1], k4.y * u);
                        S[4 * r4 + 2] = fmaf(g, S[4 * r4 + 2], k4.z * u);
                        S[4 * r4 + 3] = fmaf(g, S[4 * r4 + 3], k4.w * u);
                    }
                }
                if (part == 0 && j < V) a.out[static_cast<int64_t>(q0 + t0 + tk) * H * V + h * V + j] = o;
            }
        }
        __syncthreads();
    }
    if (!loader) {
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
            const int i = part * RPT + r;
            if (i < D && j < V) S_g[static_cast<int64_t>(i) * V + j] = S[r];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// per-head RMS norm of a float32 read-out, times a gate
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) headnorm_gate_kernel(const float *__restrict__ o, const float *__restrict__ weight,
                                                            const T *__restrict__ gate, int64_t ld_gate, T *__restrict__ out, int H, int V,
                                                            float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int h = warp; h < H; h += nwarp) {
        const float *r = o + (t * H + h) * V;
        float ss = 0.f;
        for (int c = lane; c < V; c += 32) ss = fmaf(r[c], r[c], ss);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
        const float inv = 1.0f / sqrtf(ss / static_cast<float>(V) + eps);
        for (int c = lane; c < V; c += 32) {
            float v = r[c] * inv * weight[c];
            if (gate) v *= silu(to_f(gate[t * ld_gate + h * V + c]));
            out[(t * H + h) * V + c] = from_f<T>(v);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// rotary positions
// ---------------------------------------------------------------------------------------------
// buf [n] float32 (one warp's): the first 2 pairs entries turned by sign * pos * freq, written to dst as T.
template <typename T>
__device__ __forceinline__ void rotate_store(const float *buf, int n, const float *__restrict__ freq, int pairs, int interleaved, float pos,
                                             float sign, T *__restrict__ dst, int lane) {
    for (int i = lane; i < pairs; i += 32) {
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + pairs;
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        sn *= sign;
        const float u = buf[ia], v = buf[ib];
        dst[ia] = from_f<T>(u * cs - v * sn);
        dst[ib] = from_f<T>(v * cs + u * sn);
    }
    for (int i = 2 * pairs + lane; i < n; i += 32) dst[i] = from_f<T>(buf[i]);
}

template <typename T>
__global__ void __launch_bounds__(256) qkv_headnorm_rope_cache_kernel(const atoma_qkv_rope_args a) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int H = static_cast<int>(a.H), G = static_cast<int>(a.G), D = static_cast<int>(a.dim), V = static_cast<int>(a.vdim);
    const int wide = max(D, V);
    float *buf = sm + warp * wide;
    const T *row = static_cast<const T *>(a.proj) + t * a.ld;
    const float pos = static_cast<float>(a.positions[t]);
    const int64_t slot = a.slot_mapping ? a.slot_mapping[t] : -1;
    for (int u = warp; u < H + 2 * G; u += nwarp) {
        const bool is_q = u < H, is_k = !is_q && u < H + G;
        const int hd = is_q ? u : (is_k ? u - H : u - H - G);
        if (!is_q && slot < 0) continue;
        const int n = (is_q || is_k) ? D : V;
        const T *src = row + (is_q ? a.q_off + hd * D : (is_k ? a.k_off + hd * D : a.v_off + hd * V));
        const float *w = is_q ? a.q_weight : (is_k ? a.k_weight : nullptr);
        float ss = 0.f;
        for (int c = lane; c < n; c += 32) {
            const float v = to_f(src[c]);
            buf[c] = v;
            ss = fmaf(v, v, ss);
        }
        if (w) {
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
            const float inv = 1.0f / sqrtf(ss / static_cast<float>(n) + a.eps);
            for (int c = lane; c < n; c += 32) buf[c] = buf[c] * inv * w[c];
        }
        __syncwarp();
        T *dst = is_q ? static_cast<T *>(a.q_out) + (t * H + hd) * D
                      : (is_k ? static_cast<T *>(a.k_cache) + (slot * G + hd) * D : static_cast<T *>(a.v_cache) + (slot * G + hd) * V);
        const bool vpart = !is_q && !is_k;
        const float *freq = vpart ? a.v_freq : a.qk_freq;
        const int pairs = freq ? static_cast<int>(vpart ? a.v_pairs : a.rot_pairs) : 0;
        rotate_store<T>(buf, n, freq, pairs, a.interleaved, pos, 1.f, dst, lane);
        __syncwarp();
    }
}

template <typename T>
__global__ void __launch_bounds__(256) rotate_heads_kernel(T *__restrict__ x, const int64_t *__restrict__ positions,
                                                           const float *__restrict__ freq, int H, int n, int pairs, int interleaved,
                                                           float sign) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const float pos = static_cast<float>(positions[t]);
    T *row = x + t * H * n;
    for (int idx = threadIdx.x; idx < H * pairs; idx += blockDim.x) {
        const int h = idx / pairs, i = idx % pairs;
        const int ia = h * n + (interleaved ? 2 * i : i), ib = h * n + (interleaved ? 2 * i + 1 : i + pairs);
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        sn *= sign;
        const float u = to_f(row[ia]), v = to_f(row[ib]);
        row[ia] = from_f<T>(u * cs - v * sn);
        row[ib] = from_f<T>(v * cs + u * sn);
    }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads) latent_norm_rope_cache_kernel(const T *__restrict__ proj, int64_t ld,
                                                                             const float *__restrict__ q_w, const float *__restrict__ kv_w,
                                                                             const float *__restrict__ freq, int pairs, int interleaved,
                                                                             const int64_t *__restrict__ positions,
                                                                             const int64_t *__restrict__ slots, T *__restrict__ cq_out,
                                                                             T *__restrict__ cache, int q_rank, int kv_rank, int rot_dim,
                                                                             float eps) {
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
    T *dst = cache + slot * (kv_rank + rot_dim);
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) dst[c] = from_f<T>(to_f(r[q_rank + c]) * inv * kv_w[c]);
    const T *kr = r + q_rank + kv_rank;
    const float pos = static_cast<float>(positions[t]);
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + pairs;
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        const float u = to_f(kr[ia]), v = to_f(kr[ib]);
        dst[kv_rank + ia] = from_f<T>(u * cs - v * sn);
        dst[kv_rank + ib] = from_f<T>(v * cs + u * sn);
    }
    for (int c = 2 * pairs + threadIdx.x; c < rot_dim; c += blockDim.x) dst[kv_rank + c] = kr[c];
}

// q_lat[t, h, kv_rank + c] = the rotated part of query head h, float32
template <typename T>
__global__ void __launch_bounds__(256) latent_query_rope_kernel(const T *__restrict__ q, const float *__restrict__ freq, int pairs,
                                                                int interleaved, const int64_t *__restrict__ positions,
                                                                float *__restrict__ q_lat, int H, int dim, int rot_dim, int kv_rank) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const float pos = static_cast<float>(positions[t]);
    const int hs = dim + rot_dim, row = kv_rank + rot_dim;
    for (int idx = threadIdx.x; idx < H * pairs; idx += blockDim.x) {
        const int h = idx / pairs, i = idx % pairs;
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + pairs;
        const T *src = q + (t * H + h) * hs + dim;
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        const float u = to_f(src[ia]), v = to_f(src[ib]);
        float *dst = q_lat + (t * H + h) * row + kv_rank;
        dst[ia] = u * cs - v * sn;
        dst[ib] = v * cs + u * sn;
    }
    const int rest = rot_dim - 2 * pairs;
    for (int idx = threadIdx.x; idx < H * rest; idx += blockDim.x) {
        const int h = idx / rest, c = 2 * pairs + idx % rest;
        q_lat[(t * H + h) * row + kv_rank + c] = to_f(q[(t * H + h) * hs + dim + c]);
    }
}

}  // namespace

#define HYB_DISPATCH(dtype, CALL) ((dtype) == ATOMA_DTYPE_BF16 ? CALL(__nv_bfloat16) : CALL(float))

bool hyb_parallel_residual_norm(const atoma_parallel_residual_args &a, cudaStream_t stream) {
    if (a.T <= 0) return true;
    if (!hybrid::known_dtype(a.dtype, "atoma_parallel_residual_norm")) return false;
    if (!a.x || a.width <= 0 || (a.w_next && !a.h) || (a.norm_a && !a.y_a) || (a.norm_b && !a.y_b)) {
        set_status(kErrInvalidArg, "atoma_parallel_residual_norm: null argument");
        return false;
    }
    const size_t smem = static_cast<size_t>(a.width) * 4;
    if (smem > 200 * 1024) {
        set_status(kErrUnsupported, "atoma_parallel_residual_norm: a width of %lld exceeds shared memory", static_cast<long long>(a.width));
        return false;
    }
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(parallel_residual_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(parallel_residual_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    }
#define CALL(TT) launch_ex(parallel_residual_norm_kernel<TT>, dim3(static_cast<unsigned>(a.T)), dim3(kRowThreads), smem, stream, a)
    return hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "parallel_residual_norm_kernel");
#undef CALL
}

bool hyb_tap_filter(const atoma_tap_filter_args &a, cudaStream_t stream) {
    if (a.T <= 0 || a.channels <= 0) return true;
    if (!hybrid::known_dtype(a.dtype, "atoma_tap_filter")) return false;
    if (!a.in || !a.w1 || !a.out1 || (a.w2 && !a.out2) || a.taps < 1 || a.taps > kMaxTaps || a.ld_in < a.channels || a.ld_out < a.channels ||
        !a.token_seq || !a.query_start || !a.context_lens || a.B <= 0 ||
        (a.taps > 1 && (!a.history || !a.state_slots || a.history_stride < (a.taps - 1) * a.channels))) {
        set_status(kErrInvalidArg, "atoma_tap_filter: null argument, more than %d taps, or a history row shorter than (taps - 1) channels", kMaxTaps);
        return false;
    }
    const unsigned cb = static_cast<unsigned>((a.channels + 255) / 256);
    auto piece16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = a.dtype == ATOMA_DTYPE_BF16 && a.taps >= 2 && a.taps <= 4 && a.channels % 8 == 0 && a.ld_in % 8 == 0 && a.ld_out % 8 == 0 &&
                     piece16(a.in) && piece16(a.out1) && piece16(a.out2) && piece16(a.w1) && piece16(a.w2) && !(g_hybrid_debug & 2);
    if (vec) {
        // tokens per thread: long steps amortise the window's refill, short ones keep the device filled
        const int run = a.T >= 4096 ? 16 : (a.T >= 1024 ? 8 : (a.T >= 256 ? 4 : 1));
        const dim3 grid(static_cast<unsigned>((a.channels / 8 + 127) / 128), static_cast<unsigned>((a.T + run - 1) / run));
        cudaError_t e;
        if (a.taps == 2) e = launch_ex(tap_filter_vec_kernel<2>, grid, dim3(128), 0, stream, a, run);
        else if (a.taps == 3) e = launch_ex(tap_filter_vec_kernel<3>, grid, dim3(128), 0, stream, a, run);
        else e = launch_ex(tap_filter_vec_kernel<4>, grid, dim3(128), 0, stream, a, run);
        if (!hybrid::launched(e, "tap_filter_vec_kernel")) return false;
    } else {
#define CALL(TT) launch_ex(tap_filter_kernel<TT>, dim3(cb, static_cast<unsigned>(a.T)), dim3(256), 0, stream, a)
        if (!hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "tap_filter_kernel")) return false;
#undef CALL
    }
    if (a.taps == 1) return true;
#define CALL(TT) launch_ex(tap_history_kernel<TT>, dim3(cb, static_cast<unsigned>(a.B)), dim3(256), 0, stream, a)
    return hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "tap_history_kernel");
#undef CALL
}

bool hyb_state_scan(const atoma_state_scan_args &a, cudaStream_t stream) {
    if (a.T <= 0 || a.B <= 0) return true;
    if (!hybrid::known_dtype(a.dtype, "atoma_state_scan")) return false;
    const bool gla = a.kind == 0, delta = a.kind == 1;
    if ((!gla && !delta) || !a.q || !a.k || !a.v || !a.state || !a.state_slots || !a.query_start || !a.context_lens || !a.out || a.H <= 0 ||
        a.dim <= 0 || a.vdim <= 0 || a.state_stride < a.H * a.dim * a.vdim || (gla && (!a.z || !a.z_bias || !(a.tau > 0.f))) ||
        (delta && (!a.b_pre || !a.a_pre || !a.a_log || !a.dt_bias || a.G <= 0 || a.H % a.G))) {
        set_status(kErrInvalidArg, "atoma_state_scan: null argument, unknown kind %d, or a state row shorter than heads * dim * vdim", a.kind);
        return false;
    }
    // rows of a column per lane (RPT) and lanes per column (PW): dim <= RPT * PW
    int rpt = a.dim <= 64 ? 16 : 32;
    int pw = a.dim <= 128 ? 4 : (a.dim <= 256 ? 8 : 16);
    if (a.dim > 512) {
        set_status(kErrUnsupported, "atoma_state_scan: a key size of %lld exceeds 512", static_cast<long long>(a.dim));
        return false;
    }
    // few CTAs (one long prompt, a handful of decoded tokens): 8 rows per lane, so that a token is a short chain and the state's
    // entries are spread over more warps — as long as all CTAs are resident at once (two per SM): a second wave would walk the
    // tokens a second time
    const int64_t ctas_many = (a.vdim + 32 / pw * kScanWarps - 1) / (32 / pw * kScanWarps) * a.H * a.B;
    if (a.dim <= 256 && !(g_hybrid_debug & 16) && ctas_many * (rpt / 8) <= 2 * current_device_info().sm_count) {
        pw = pw * rpt / 8;
        rpt = 8;
    }
    const int cols = 32 / pw * kScanWarps;
    const int per_tok = (gla ? 3 : 2) * pw * (rpt + 4) + cols + 4;
    int64_t longest = a.T;                                   // a bound of the longest portion: T tokens over B sequences, each has one at least
    longest = std::max<int64_t>(1, a.T - (a.B - 1));
    // staged tokens per buffer: at most 32, no more than the longest portion, and two CTAs' buffers fit one SM
    const int chunk = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>({32, longest, 96 * 1024 / (8 * per_tok)})));
    const size_t smem = static_cast<size_t>(2 * chunk * per_tok) * 4;
    const dim3 grid(static_cast<unsigned>((a.vdim + cols - 1) / cols), static_cast<unsigned>(a.H), static_cast<unsigned>(a.B));
    const dim3 block(64 * kScanWarps);
    cudaError_t e;
#define SCAN(TT, KIND, RPT, PW)                                                                                                    \
    do {                                                                                                                            \
        if (smem > 48 * 1024) cudaFuncSetAttribute(state_scan_kernel<TT, KIND, RPT, PW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
        e = launch_ex(state_scan_kernel<TT, KIND, RPT, PW>, grid, block, smem, stream, a, chunk);                                   \
    } while (0)
#define SCAN_K(TT, KIND)                                \
    do {                                                \
        if (rpt == 8 && pw == 8) SCAN(TT, KIND, 8, 8);  \
        else if (rpt == 8 && pw == 16) SCAN(TT, KIND, 8, 16); \
        else if (rpt == 8) SCAN(TT, KIND, 8, 32);       \
        else if (rpt == 16) SCAN(TT, KIND, 16, 4);      \
        else if (pw == 4) SCAN(TT, KIND, 32, 4);        \
        else if (pw == 8) SCAN(TT, KIND, 32, 8);        \
        else SCAN(TT, KIND, 32, 16);                    \
    } while (0)
#define SCAN_T(TT)                                      \
    do {                                                \
        if (gla) SCAN_K(TT, 0);                         \
        else SCAN_K(TT, 1);                             \
    } while (0)
    if (a.dtype == ATOMA_DTYPE_BF16) SCAN_T(__nv_bfloat16);
    else SCAN_T(float);
#undef SCAN_T
#undef SCAN_K
#undef SCAN
    return hybrid::launched(e, "state_scan_kernel");
}

bool hyb_headnorm_gate(const float *o, const float *weight, const void *gate, int64_t ld_gate, void *out, int64_t T, int64_t H, int64_t vdim,
                       float eps, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_headnorm_gate")) return false;
    if (!o || !weight || !out || H <= 0 || vdim <= 0 || (gate && ld_gate < H * vdim)) {
        set_status(kErrInvalidArg, "atoma_headnorm_gate: null argument or a gate row shorter than heads * vdim");
        return false;
    }
    const unsigned threads = static_cast<unsigned>(std::min<int64_t>(8, H) * 32);
#define CALL(TT) launch_ex(headnorm_gate_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(threads), 0, stream, o, weight, \
                           static_cast<const TT *>(gate), ld_gate, static_cast<TT *>(out), static_cast<int>(H), static_cast<int>(vdim), eps)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "headnorm_gate_kernel");
#undef CALL
}

bool hyb_qkv_headnorm_rope_cache(const atoma_qkv_rope_args &a, cudaStream_t stream) {
    if (a.T <= 0) return true;
    if (!hybrid::known_dtype(a.dtype, "atoma_qkv_headnorm_rope_cache")) return false;
    if (!a.proj || !a.q_out || !a.positions || a.H <= 0 || a.G <= 0 || a.H % a.G || a.dim <= 0 || a.vdim <= 0 ||
        (a.slot_mapping && (!a.k_cache || !a.v_cache)) || a.q_off < 0 || a.k_off < 0 || a.v_off < 0 || a.q_off + a.H * a.dim > a.ld ||
        a.k_off + a.G * a.dim > a.ld || a.v_off + a.G * a.vdim > a.ld || a.rot_pairs < 0 || 2 * a.rot_pairs > a.dim || a.v_pairs < 0 ||
        2 * a.v_pairs > a.vdim || (a.rot_pairs > 0 && !a.qk_freq)) {
        set_status(kErrInvalidArg, "atoma_qkv_headnorm_rope_cache: null argument, columns outside the row, or more rotated entries than a head has");
        return false;
    }
    const unsigned warps = static_cast<unsigned>(std::min<int64_t>(8, a.H + 2 * a.G));
    const size_t smem = static_cast<size_t>(warps) * std::max(a.dim, a.vdim) * 4;
    if (smem > 48 * 1024) {
        set_status(kErrUnsupported, "atoma_qkv_headnorm_rope_cache: heads of %lld entries", static_cast<long long>(std::max(a.dim, a.vdim)));
        return false;
    }
#define CALL(TT) launch_ex(qkv_headnorm_rope_cache_kernel<TT>, dim3(static_cast<unsigned>(a.T)), dim3(warps * 32), smem, stream, a)
    return hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "qkv_headnorm_rope_cache_kernel");
#undef CALL
}

bool hyb_rotate_heads(void *x, const int64_t *positions, const float *freq, int64_t T, int64_t H, int64_t n, int64_t pairs, int32_t interleaved,
                      float sign, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0 || pairs <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_rotate_heads")) return false;
    if (!x || !positions || !freq || H <= 0 || 2 * pairs > n) {
        set_status(kErrInvalidArg, "atoma_rotate_heads: null argument or more rotated entries than a head has");
        return false;
    }
#define CALL(TT) launch_ex(rotate_heads_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(256), 0, stream, static_cast<TT *>(x), positions, freq, \
                           static_cast<int>(H), static_cast<int>(n), static_cast<int>(pairs), interleaved, sign)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "rotate_heads_kernel");
#undef CALL
}

bool hyb_latent_norm_rope_cache(const void *proj, int64_t ld, const float *q_w, const float *kv_w, const float *freq, int64_t pairs,
                                int32_t interleaved, const int64_t *positions, const int64_t *slots, void *cq_out, void *cache, int64_t T,
                                int64_t q_rank, int64_t kv_rank, int64_t rot_dim, float eps, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_latent_norm_rope_cache")) return false;
    if (!proj || kv_rank <= 0 || q_rank < 0 || rot_dim < 0 || ld < q_rank + kv_rank + rot_dim || !kv_w || (q_rank > 0 && (!q_w || !cq_out)) ||
        (slots && !cache) || !positions || pairs < 0 || 2 * pairs > rot_dim || (pairs > 0 && !freq)) {
        set_status(kErrInvalidArg, "atoma_latent_norm_rope_cache: null argument or a row shorter than q_rank + kv_rank + rot_dim");
        return false;
    }
#define CALL(TT) launch_ex(latent_norm_rope_cache_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(kRowThreads), 0, stream, \
                           static_cast<const TT *>(proj), ld, q_w, kv_w, freq, static_cast<int>(pairs), interleaved, positions, slots, \
                           static_cast<TT *>(cq_out), static_cast<TT *>(cache), static_cast<int>(q_rank), static_cast<int>(kv_rank), \
                           static_cast<int>(rot_dim), eps)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "latent_norm_rope_cache_kernel");
#undef CALL
}

bool hyb_latent_query_absorb_rope(const void *q, const void *w_uk, const float *freq, int64_t pairs, int32_t interleaved,
                                  const int64_t *positions, float *q_lat, int64_t T, int64_t H, int64_t dim, int64_t rot_dim, int64_t kv_rank,
                                  uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_latent_query_absorb_rope")) return false;
    if (!q || !w_uk || !q_lat || !positions || H <= 0 || dim <= 0 || rot_dim < 0 || kv_rank <= 0 || pairs < 0 || 2 * pairs > rot_dim ||
        (pairs > 0 && !freq)) {
        set_status(kErrInvalidArg, "atoma_latent_query_absorb_rope: null argument or more rotated entries than the rotated part has");
        return false;
    }
    const int64_t hs = dim + rot_dim, row = kv_rank + rot_dim;
    if (!hyb_head_project_ld(q, H * hs, hs, w_uk, q_lat, H * row, row, T, H, dim, kv_rank, 1, dtype, stream)) return false;
    if (rot_dim == 0) return true;
#define CALL(TT) launch_ex(latent_query_rope_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(256), 0, stream, static_cast<const TT *>(q), freq, \
                           static_cast<int>(pairs), interleaved, positions, q_lat, static_cast<int>(H), static_cast<int>(dim), \
                           static_cast<int>(rot_dim), static_cast<int>(kv_rank))
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "latent_query_rope_kernel");
#undef CALL
}

bool hyb_latent_expand_values(const float *o_lat, const void *w_uv, void *out, int64_t T, int64_t H, int64_t vdim, int64_t kv_rank, int64_t row,
                              uint32_t dtype, cudaStream_t stream) {
    if (row < kv_rank) {
        set_status(kErrInvalidArg, "atoma_latent_expand_values: rows of %lld entries for a latent of %lld", static_cast<long long>(row),
                   static_cast<long long>(kv_rank));
        return false;
    }
    return hyb_head_project_ld(o_lat, H * row, row, w_uv, out, H * vdim, vdim, T, H, vdim, kv_rank, 0, dtype, stream);
}

}  // namespace atoma

using namespace atoma;

extern "C" void atoma_parallel_residual_norm(const atoma_parallel_residual_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_parallel_residual_norm: args is NULL");
        return;
    }
    hyb_parallel_residual_norm(*args, static_cast<cudaStream_t>(stream));
}

extern "C" void atoma_tap_filter(const atoma_tap_filter_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_tap_filter: args is NULL");
        return;
    }
    hyb_tap_filter(*args, static_cast<cudaStream_t>(stream));
}

extern "C" void atoma_state_scan(const atoma_state_scan_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_state_scan: args is NULL");
        return;
    }
    hyb_state_scan(*args, static_cast<cudaStream_t>(stream));
}

extern "C" void atoma_headnorm_gate(const float *o, const float *weight, const void *gate, int64_t ld_gate, void *out, int64_t T, int64_t H,
                                    int64_t vdim, float eps, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_headnorm_gate(o, weight, gate, ld_gate, out, T, H, vdim, eps, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" void atoma_qkv_headnorm_rope_cache(const atoma_qkv_rope_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_qkv_headnorm_rope_cache: args is NULL");
        return;
    }
    hyb_qkv_headnorm_rope_cache(*args, static_cast<cudaStream_t>(stream));
}

extern "C" void atoma_rotate_heads(void *x, const int64_t *positions, const float *freq, int64_t T, int64_t H, int64_t n, int64_t pairs,
                                   int32_t interleaved, float sign, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_rotate_heads(x, positions, freq, T, H, n, pairs, interleaved, sign, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" void atoma_latent_norm_rope_cache(const void *proj, int64_t ld, const float *q_weight, const float *kv_weight, const float *freq,
                                             int64_t pairs, int32_t interleaved, const int64_t *positions, const int64_t *slot_mapping,
                                             void *cq_out, void *cache, int64_t T, int64_t q_rank, int64_t kv_rank, int64_t rot_dim, float eps,
                                             uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_latent_norm_rope_cache(proj, ld, q_weight, kv_weight, freq, pairs, interleaved, positions, slot_mapping, cq_out, cache, T, q_rank, kv_rank,
                               rot_dim, eps, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" void atoma_latent_query_absorb_rope(const void *q, const void *w_uk, const float *freq, int64_t pairs, int32_t interleaved,
                                               const int64_t *positions, float *q_lat, int64_t T, int64_t H, int64_t dim, int64_t rot_dim,
                                               int64_t kv_rank, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_latent_query_absorb_rope(q, w_uk, freq, pairs, interleaved, positions, q_lat, T, H, dim, rot_dim, kv_rank, dtype,
                                 static_cast<cudaStream_t>(stream));
}

extern "C" void atoma_latent_expand_values(const float *o_lat, const void *w_uv, void *out, int64_t T, int64_t H, int64_t vdim, int64_t kv_rank,
                                           int64_t row, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_latent_expand_values(o_lat, w_uv, out, T, H, vdim, kv_rank, row, dtype, static_cast<cudaStream_t>(stream));
}
