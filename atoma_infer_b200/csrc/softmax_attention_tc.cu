// Softmax attention over a paged bfloat16 cache on tensor cores (include/atoma_hybrid.h, atoma_softmax_attention_paged):
// grouped key/value heads, a sliding window that also keeps the first tokens, a bias looked up by query-key distance and a
// sigmoid gate on the output.
//
// One kernel, two row mappings (four warps per CTA, key tiles of 64 at absolute positions 64 i .. 64 i + 63):
//  * portions (ROWS_ARE_HEADS = false): a CTA owns 64 consecutive query tokens of one sequence and one head, a warp 16 of
//    them; every warp multiplies its rows with all 64 keys of a tile.
//  * single tokens (ROWS_ARE_HEADS = true): a CTA owns one token and one key/value head; the rows of the tile are the query
//    heads that share it (the keys and values are streamed once for all of them), and the four warps take 16 keys each of
//    every tile; their running (maximum, sum, output) triples are merged in warp order at the end.  `splits` > 1 cuts a
//    token's tile list into contiguous ranges (one CTA each) whose triples a second kernel merges in range order.
// The tiles a CTA visits are the ones that hold a visible key of any of its rows: the kept first tokens (below the window's
// start), then the window up to the diagonal.  Keys and values are staged with cp.async through the block table (double
// buffered), S = Q K^T and O += P V run on mma.sync m16n8k16 (bf16 in, float32 out); scale, bias, mask, running maximum
// and sum are float32 in the exp2 domain; P is rounded to bfloat16 for the second product.  A row's arithmetic depends on
// its position and the layer's constants only.
//
// Why mma.sync and not tcgen05: the single-token mapping has at most 16 useful rows (a 128-row tensor-memory tile would be
// 7/8 padding) and is bound by the cache stream; portions of 128 tokens and more in the shapes the tensor-memory prefill
// kernel takes run there (softmax_attention_long.cu), so this file's portion mapping serves the short ones and the other shapes.
#include "common.cuh"
#include "hybrid_common.cuh"

#include "atoma_hybrid.h"

#include <algorithm>

namespace atoma {
namespace {

using namespace hybrid;

constexpr int kKeys = 64;          // keys per tile
constexpr int kRowsCta = 64;       // query rows per CTA (portions)
constexpr int kBiasSmem = 2048;    // distances whose bias is kept in shared memory (portions)
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {   // 2^x, flushing; ex2(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct TcLayout {
    int k_off, v_off, bias_off, total;
};
__host__ __device__ inline TcLayout tc_layout(int D, int DV, int bias_n) {
    TcLayout l;
    l.k_off = 0;
    l.v_off = 2 * kKeys * (D + 8) * 2;
    l.bias_off = l.v_off + 2 * kKeys * (DV + 8) * 2;
    l.total = l.bias_off + bias_n * 4;
    return l;
}

// EXACT: dim = vdim = DMAX (the usual case): strides and loop bounds are compile-time constants.
// SIG: the weight of a visible key is sigmoid(score * scale + head_bias[h]) and nothing is normalised (no running maximum, no
// denominator, no rescaling: the outputs are plain sums) — the same tiles, staging and products serve both kinds of attention.
template <int DMAX, bool ROWS_ARE_HEADS, bool EXACT, bool SIG>
__global__ void __launch_bounds__(128, 3) softmax_attn_tc_kernel(const atoma_softmax_attn_args a, int bias_n, int splits, float *__restrict__ partial,
                                                                 const float *__restrict__ head_bias) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    pdl_wait();
    constexpr int NT = ROWS_ARE_HEADS ? 2 : kKeys / 8;   // 8-key score tiles per warp and key tile
    const int H = static_cast<int>(a.H), G = static_cast<int>(a.G);
    const int D = EXACT ? DMAX : static_cast<int>(a.dim), DV = EXACT ? DMAX : static_cast<int>(a.vdim);
    const int rep = H / G;
    const int b = blockIdx.y;
    const int t_begin = a.query_start[b], n_q = a.query_start[b + 1] - t_begin;
    if (ROWS_ARE_HEADS ? n_q != 1 : n_q <= 1) return;   // single tokens are served by the rows-are-heads mapping
    if (a.skip_min_q > 0 && n_q >= a.skip_min_q) return;   // long portions are served elsewhere
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t4 = lane & 3, rq = lane >> 2;
    const int ctx = static_cast<int>(a.positions[t_begin]);
    // rows of this CTA / warp
    int h0, g, tok0, rows_w, p_first, p_last, split = 0;
    if constexpr (ROWS_ARE_HEADS) {
        const int chunks = (rep + 15) / 16;
        split = blockIdx.x;
        g = blockIdx.z / chunks;
        h0 = g * rep + (blockIdx.z % chunks) * 16;
        rows_w = min(16, g * rep + rep - h0);
        tok0 = t_begin;
        p_first = p_last = ctx;
    } else {
        const int r0 = blockIdx.x * kRowsCta;
        if (r0 >= n_q) return;
        h0 = blockIdx.z;
        g = h0 / rep;
        tok0 = t_begin + r0 + warp * 16;
        rows_w = max(0, min(16, n_q - r0 - warp * 16));
        p_first = ctx + r0;
        p_last = ctx + min(n_q, r0 + kRowsCta) - 1;
    }
    const int pw0 = ROWS_ARE_HEADS ? ctx : p_first + warp * 16;   // position of the warp's row 0
    const int window = (a.window > 0 && a.window < 0x3fffffff) ? static_cast<int>(a.window) : 0x3fffffff;
    const int keep = a.keep_first <= 0 ? 0 : (a.keep_first < 0x3fffffff ? static_cast<int>(a.keep_first) : 0x3fffffff);
    const int bs = static_cast<int>(a.block_size);
    const int32_t *bt = a.block_tables + static_cast<int64_t>(b) * a.max_blocks;
    const TcLayout L = tc_layout(D, DV, ROWS_ARE_HEADS ? 0 : bias_n);
    __nv_bfloat16 *Ks0 = reinterpret_cast<__nv_bfloat16 *>(smem + L.k_off);
    __nv_bfloat16 *Vs0 = reinterpret_cast<__nv_bfloat16 *>(smem + L.v_off);
    float *bias_s = reinterpret_cast<float *>(smem + L.bias_off);
    const int k_stage = kKeys * (D + 8), v_stage = kKeys * (DV + 8);
    const __nv_bfloat16 *kc = static_cast<const __nv_bfloat16 *>(a.k_cache);
    const __nv_bfloat16 *vc = static_cast<const __nv_bfloat16 *>(a.v_cache);
    const int last_row = static_cast<int>(a.dist_rows) - 1;
    if constexpr (!ROWS_ARE_HEADS) {
        for (int i = threadIdx.x; i < bias_n; i += blockDim.x) bias_s[i] = a.dist_bias[static_cast<int64_t>(i) * H + h0] * kLog2e;
    }

    // the CTA's tiles: kept first tokens below the window's start, then the window up to the diagonal
    const int lo_cta = max(0, p_first - window + 1);
    const int kt_lo = lo_cta / kKeys, kt_hi = p_last / kKeys;
    const int ka = min((min(keep, lo_cta) + kKeys - 1) / kKeys, kt_lo);
    const int n_tiles = ka + (kt_hi - kt_lo + 1);
    int i_begin = 0, i_end = n_tiles;
    if (ROWS_ARE_HEADS && splits > 1) {
        const int per = (n_tiles + splits - 1) / splits;
        i_begin = min(n_tiles, split * per);
        i_end = min(n_tiles, i_begin + per);
    }
    auto tile_of = [&](int i) { return i < ka ? i : kt_lo + (i - ka); };

    // query fragments (A operand: rows rq / rq + 8, k = 2 t4 .. + 1 and + 8)
    uint32_t qf[DMAX / 16][4];
    {
        const __nv_bfloat16 *q = static_cast<const __nv_bfloat16 *>(a.q);
        const int64_t row_stride = ROWS_ARE_HEADS ? D : static_cast<int64_t>(H) * D;
        const __nv_bfloat16 *q0 = q + (static_cast<int64_t>(tok0) * H + h0) * D;
#pragma unroll
        for (int kk = 0; kk < DMAX / 16; ++kk) {
            qf[kk][0] = qf[kk][1] = qf[kk][2] = qf[kk][3] = 0u;
            if (kk * 16 < D) {
                const int col = kk * 16 + 2 * t4;
                if (rq < rows_w) {
                    qf[kk][0] = *reinterpret_cast<const uint32_t *>(q0 + rq * row_stride + col);
                    qf[kk][2] = *reinterpret_cast<const uint32_t *>(q0 + rq * row_stride + col + 8);
                }
                if (rq + 8 < rows_w) {
                    qf[kk][1] = *reinterpret_cast<const uint32_t *>(q0 + (rq + 8) * row_stride + col);
                    qf[kk][3] = *reinterpret_cast<const uint32_t *>(q0 + (rq + 8) * row_stride + col + 8);
                }
            }
        }
    }
    float o[DMAX / 8][4];
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float scale2 = a.scale * kLog2e;
    float hb[2] = {0.f, 0.f};                                  // SIG: the bias of the head of rows rq and rq + 8, in log2 units
    if constexpr (SIG) {
        if (head_bias) {
            if constexpr (ROWS_ARE_HEADS) {
                hb[0] = rq < rows_w ? head_bias[h0 + rq] * kLog2e : 0.f;
                hb[1] = rq + 8 < rows_w ? head_bias[h0 + rq + 8] * kLog2e : 0.f;
            } else {
                hb[0] = hb[1] = head_bias[h0] * kLog2e;
            }
        }
    }

    // cache rows (of the CTA's key/value head) of a tile's keys, looked up once per key one tile ahead of the copies that use
    // them (-1: past the last key)
    __shared__ int64_t slot_s[2][kKeys];
    auto slot_of = [&](int i) -> int64_t {     // thread t < 64: the cache row of key t of tile i, (slot * G + g)
        if (threadIdx.x >= kKeys) return -1;
        const int j = tile_of(i) * kKeys + threadIdx.x;
        return j <= p_last ? (static_cast<int64_t>(bt[j / bs]) * bs + j % bs) * G + g : -1;
    };
    auto fill_slots = [&](int i, int buf) {
        const int64_t v = slot_of(i);
        if (threadIdx.x < kKeys) slot_s[buf][threadIdx.x] = v;
    };
    const int ck = D / 8, cv = DV / 8;   // 16-byte pieces per cache row of one kv head
    const int k_jj0 = threadIdx.x / ck, k_e0 = threadIdx.x % ck, k_djj = 128 / ck, k_de = 128 % ck;
    const int v_jj0 = threadIdx.x / cv, v_e0 = threadIdx.x % cv, v_djj = 128 / cv, v_de = 128 % cv;
    auto stage_tile = [&](int buf, int st) {
        __nv_bfloat16 *Kd = Ks0 + st * k_stage, *Vd = Vs0 + st * v_stage;
        const int64_t *slots = slot_s[buf];
        for (int jj = k_jj0, e = k_e0; jj < kKeys;) {     // thread -> pieces threadIdx.x, + 128, ... of the tile, (row, piece) kept incrementally
            const int64_t slot = slots[jj];
            cp_async_16(smem_u32(Kd + jj * (D + 8) + e * 8), kc + (slot < 0 ? 0 : slot) * D + e * 8, slot < 0 ? 0 : 16);
            jj += k_djj, e += k_de;
            if (e >= ck) e -= ck, ++jj;
        }
        for (int jj = v_jj0, e = v_e0; jj < kKeys;) {
            const int64_t slot = slots[jj];
            cp_async_16(smem_u32(Vd + jj * (DV + 8) + e * 8), vc + (slot < 0 ? 0 : slot) * DV + e * 8, slot < 0 ? 0 : 16);
            jj += v_djj, e += v_de;
            if (e >= cv) e -= cv, ++jj;
        }
        cp_async_commit();
    };
    if (i_begin < i_end) fill_slots(i_begin, 0);
    if (i_begin + 1 < i_end) fill_slots(i_begin + 1, 1);
    __syncthreads();   // bias_s, slot_s
    if (i_begin < i_end) stage_tile(0, 0);

    const int key_off = ROWS_ARE_HEADS ? warp * 16 : 0;   // the warp's keys inside a tile
    const int pw_last = ROWS_ARE_HEADS ? ctx : pw0 + 15;
    const int lo_w = max(0, pw0 - window + 1);
    for (int i = i_begin; i < i_end; ++i) {
        const int st = (i - i_begin) & 1;
        const int64_t slot_ahead = i + 2 < i_end ? slot_of(i + 2) : -1;   // the block-table read flies during this tile's math
        if (i + 1 < i_end) {
            stage_tile(st ^ 1, st ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            cp_async_wait_all();
        }
        __syncthreads();
        const int kt = tile_of(i);
        const int j0 = kt * kKeys + key_off, j1 = j0 + NT * 8 - 1;   // this warp's keys of the tile
        // nothing of the warp's rows sees these keys: above the diagonal, or behind the window and not kept
        const bool dead = rows_w <= 0 || j0 > pw_last || (j1 < lo_w && j0 >= keep);
        if (!dead) {
            const __nv_bfloat16 *Ks = Ks0 + st * k_stage, *Vs = Vs0 + st * v_stage;
            float sacc[NT][4];
#pragma unroll
            for (int n = 0; n < NT; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < DMAX / 16; ++kk) {
                if (kk * 16 < D) {
#pragma unroll
                    for (int np = 0; np < NT / 2; ++np) {
                        uint32_t r[4];
                        const __nv_bfloat16 *src = Ks + (key_off + (np * 2 + (lane >> 4)) * 8 + (lane & 7)) * (D + 8) + kk * 16 + ((lane >> 3) & 1) * 8;
                        ldmatrix_x4(r, smem_u32(src));
                        Mma16816<__nv_bfloat16>::run(sacc[np * 2], qf[kk], r[0], r[1]);
                        Mma16816<__nv_bfloat16>::run(sacc[np * 2 + 1], qf[kk], r[2], r[3]);
                    }
                }
            }
            // every pair of the warp's rows and keys is visible: below the diagonal for the first row, inside the window of the
            // last row (or all kept)
            const bool all_visible = rows_w == 16 && j1 <= pw0 && (pw_last - j0 < window || j1 < keep);
            const int dist0 = pw0 + rq - j0 - 2 * t4;   // distance of (row rq, key j0 + 2 t4)
            if constexpr (SIG) {
                // weights: sigmoid(score * scale + bias) = 1 / (1 + 2^-(x log2 e)); zero where the key is not visible
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int half = e >> 1, row = rq + half * 8;
                        const int dist = ROWS_ARE_HEADS ? ctx - (j0 + n * 8 + 2 * t4 + (e & 1)) : dist0 + half * 8 - n * 8 - (e & 1);
                        float pv = __frcp_rn(1.f + ex2(-fmaf(sacc[n][e], scale2, hb[half])));
                        if (!all_visible) {
                            const int j = (ROWS_ARE_HEADS ? ctx : pw0 + row) - dist;
                            if (!(row < rows_w && dist >= 0 && (dist < window || j < keep))) pv = 0.f;
                        }
                        sacc[n][e] = pv;
                    }
            } else {
                // scale, bias, mask; running maximum per row (rows rq and rq + 8)
                float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int half = e >> 1, row = rq + half * 8;
                        const int dist = ROWS_ARE_HEADS ? ctx - (j0 + n * 8 + 2 * t4 + (e & 1)) : dist0 + half * 8 - n * 8 - (e & 1);
                        float s = sacc[n][e] * scale2;
                        if (a.dist_bias) {
                            if constexpr (ROWS_ARE_HEADS) {
                                if (row < rows_w && dist >= 0) s += __ldg(a.dist_bias + static_cast<int64_t>(min(dist, last_row)) * H + h0 + row) * kLog2e;
                            } else if (bias_n > last_row) {   // the whole table is in shared memory
                                s += bias_s[min(max(dist, 0), last_row)];
                            } else if (dist >= 0) {
                                s += dist < bias_n ? bias_s[dist] : __ldg(a.dist_bias + static_cast<int64_t>(min(dist, last_row)) * H + h0) * kLog2e;
                            }
                        }
                        if (!all_visible) {
                            const int j = (ROWS_ARE_HEADS ? ctx : pw0 + row) - dist;
                            if (!(row < rows_w && dist >= 0 && (dist < window || j < keep))) s = -INFINITY;
                        }
                        sacc[n][e] = s;
                        tmax[half] = fmaxf(tmax[half], s);
                    }
                float corr[2], msub[2];
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    tmax[hf] = fmaxf(tmax[hf], __shfl_xor_sync(0xffffffffu, tmax[hf], 1));
                    tmax[hf] = fmaxf(tmax[hf], __shfl_xor_sync(0xffffffffu, tmax[hf], 2));
                    const float m_new = fmaxf(m_run[hf], tmax[hf]);
                    msub[hf] = m_new == -INFINITY ? 0.f : m_new;          // a row that has seen nothing yet: exp2(-inf - 0) = 0
                    corr[hf] = m_run[hf] == -INFINITY ? 0.f : ex2(m_run[hf] - msub[hf]);
                    m_run[hf] = m_new;
                    l_run[hf] *= corr[hf];
                }
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float pv = ex2(sacc[n][e] - msub[e >> 1]);
                        sacc[n][e] = pv;
                        l_run[e >> 1] += pv;
                    }
                if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {   // no row's maximum moved: nothing to rescale
#pragma unroll
                    for (int n = 0; n < DMAX / 8; ++n) {
                        o[n][0] *= corr[0];
                        o[n][1] *= corr[0];
                        o[n][2] *= corr[1];
                        o[n][3] *= corr[1];
                    }
                }
            }
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk) {
                uint32_t af[4];
                af[0] = pack2<__nv_bfloat16>(sacc[2 * kk][0], sacc[2 * kk][1]);
                af[1] = pack2<__nv_bfloat16>(sacc[2 * kk][2], sacc[2 * kk][3]);
                af[2] = pack2<__nv_bfloat16>(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
                af[3] = pack2<__nv_bfloat16>(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < DMAX / 16; ++n2) {
                    if (n2 * 16 < DV) {
                        uint32_t r[4];
                        const __nv_bfloat16 *src = Vs + (key_off + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * (DV + 8) + n2 * 16 + (lane >> 4) * 8;
                        ldmatrix_x4_trans(r, smem_u32(src));
                        Mma16816<__nv_bfloat16>::run(o[n2 * 2], af, r[0], r[1]);
                        Mma16816<__nv_bfloat16>::run(o[n2 * 2 + 1], af, r[2], r[3]);
                    }
                }
            }
        }
        if (i + 2 < i_end && threadIdx.x < kKeys) slot_s[st][threadIdx.x] = slot_ahead;   // this tile's copies, which read slot_s[st], were issued before the barrier above
        __syncthreads();   // the stage is free for the tile after next
    }
    // row sums: the four lanes of a quad hold disjoint columns
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        l_run[hf] += __shfl_xor_sync(0xffffffffu, l_run[hf], 1);
        l_run[hf] += __shfl_xor_sync(0xffffffffu, l_run[hf], 2);
    }

    if constexpr (!ROWS_ARE_HEADS) {
        __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(a.out) + (static_cast<int64_t>(tok0) * H + h0) * DV;
        const __nv_bfloat16 *gate = a.gate ? static_cast<const __nv_bfloat16 *>(a.gate) + static_cast<int64_t>(tok0) * a.ld_gate + h0 * DV : nullptr;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int row = rq + hf * 8;
            if (row >= rows_w) continue;
            const float inv = SIG ? 1.f : 1.f / l_run[hf];
#pragma unroll
            for (int n = 0; n < DMAX / 8; ++n) {
                if (n * 8 < DV) {
                    const int col = n * 8 + 2 * t4;
                    float v0 = o[n][2 * hf] * inv, v1 = o[n][2 * hf + 1] * inv;
                    if (gate) {
                        const float2 gv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(gate + static_cast<int64_t>(row) * a.ld_gate + col));
                        v0 *= sigmoidf_(gv.x);
                        v1 *= sigmoidf_(gv.y);
                    }
                    *reinterpret_cast<uint32_t *>(out + static_cast<int64_t>(row) * H * DV + col) = pack2<__nv_bfloat16>(v0, v1);
                }
            }
        }
        return;
    } else {
        // merge the four warps' (maximum, sum, output) per head row, in warp order; the staging buffers are free now
        float *m_s = reinterpret_cast<float *>(smem);          // [4][16]
        float *l_s = m_s + 64;                                   // [4][16]
        float *o_s = l_s + 64;                                   // [4][16][DV]
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const int row = rq + hf * 8;
            if (t4 == 0) {
                m_s[warp * 16 + row] = SIG ? 0.f : m_run[hf];
                l_s[warp * 16 + row] = l_run[hf];
            }
#pragma unroll
            for (int n = 0; n < DMAX / 8; ++n)
                if (n * 8 < DV) {
                    float *dst = o_s + (warp * 16 + row) * DV + n * 8 + 2 * t4;
                    dst[0] = o[n][2 * hf];
                    dst[1] = o[n][2 * hf + 1];
                }
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < rows_w * DV; idx += blockDim.x) {
            const int row = idx / DV, d = idx % DV;
            float M = -INFINITY;
            for (int w = 0; w < 4; ++w) M = fmaxf(M, m_s[w * 16 + row]);
            float Lsum = 0.f, acc = 0.f;
            for (int w = 0; w < 4; ++w) {
                const float mw = m_s[w * 16 + row];
                const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
                Lsum = fmaf(l_s[w * 16 + row], f, Lsum);
                acc = fmaf(o_s[(w * 16 + row) * DV + d], f, acc);
            }
            const int h = h0 + row;
            if (partial) {   // this split's triple: [token][head][split] -> maximum, sum, then the un-normalised output
                float *pm = partial + ((static_cast<int64_t>(b) * H + h) * splits + split) * (DV + 2);
                if (d == 0) {
                    pm[0] = M;
                    pm[1] = SIG ? (split == 0 ? 1.f : 0.f) : Lsum;   // SIG: the merge divides the plain sum of the splits by one
                }
                pm[2 + d] = acc;
            } else {
                float v = SIG ? acc : acc / Lsum;
                if (a.gate) v *= sigmoidf_(__bfloat162float(static_cast<const __nv_bfloat16 *>(a.gate)[static_cast<int64_t>(tok0) * a.ld_gate + h * DV + d]));
                static_cast<__nv_bfloat16 *>(a.out)[(static_cast<int64_t>(tok0) * H + h) * DV + d] = __float2bfloat16_rn(v);
            }
        }
    }
}

// One CTA per (sequence with a single token, head): the splits' triples in split order.
__global__ void __launch_bounds__(128) softmax_split_merge_kernel(const atoma_softmax_attn_args a, int splits, const float *__restrict__ partial) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int t = a.query_start[b];
    if (a.query_start[b + 1] - t != 1) return;
    const int H = static_cast<int>(a.H), DV = static_cast<int>(a.vdim);
    const float *pm = partial + (static_cast<int64_t>(b) * H + h) * splits * (DV + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, pm[s * (DV + 2)]);
    float Lsum = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = pm[s * (DV + 2)];
        Lsum = fmaf(pm[s * (DV + 2) + 1], ms == -INFINITY ? 0.f : exp2f(ms - M), Lsum);
    }
    for (int d = threadIdx.x; d < DV; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = pm[s * (DV + 2)];
            acc = fmaf(pm[s * (DV + 2) + 2 + d], ms == -INFINITY ? 0.f : exp2f(ms - M), acc);
        }
        float v = acc / Lsum;
        if (a.gate) v *= sigmoidf_(__bfloat162float(static_cast<const __nv_bfloat16 *>(a.gate)[static_cast<int64_t>(t) * a.ld_gate + h * DV + d]));
        static_cast<__nv_bfloat16 *>(a.out)[(static_cast<int64_t>(t) * H + h) * DV + d] = __float2bfloat16_rn(v);
    }
}

template <int DMAX, bool ROWS_ARE_HEADS, bool EXACT, bool SIG>
cudaError_t launch_tc_exact(const atoma_softmax_attn_args &a, dim3 grid, size_t smem, int bias_n, int splits, float *partial, const float *head_bias,
                            cudaStream_t stream) {
    static int attr_dev = -1;
    const int dev = current_device_info().ordinal;
    if (attr_dev != dev) {
        cudaFuncSetAttribute(softmax_attn_tc_kernel<DMAX, ROWS_ARE_HEADS, EXACT, SIG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
        attr_dev = dev;
    }
    return launch_ex(softmax_attn_tc_kernel<DMAX, ROWS_ARE_HEADS, EXACT, SIG>, grid, dim3(128), smem, stream, a, bias_n, splits, partial, head_bias);
}
template <int DMAX, bool ROWS_ARE_HEADS, bool SIG>
cudaError_t launch_tc(const atoma_softmax_attn_args &a, dim3 grid, size_t smem, int bias_n, int splits, float *partial, const float *head_bias,
                      cudaStream_t stream) {
    return (a.dim == DMAX && a.vdim == DMAX) ? launch_tc_exact<DMAX, ROWS_ARE_HEADS, true, SIG>(a, grid, smem, bias_n, splits, partial, head_bias, stream)
                                             : launch_tc_exact<DMAX, ROWS_ARE_HEADS, false, SIG>(a, grid, smem, bias_n, splits, partial, head_bias, stream);
}

}  // namespace

// Takes bfloat16 batches whose head sizes are multiples of 16 up to 128.  Sequences with one token in the step (decoded
// tokens) run with the heads of a key/value group as the tile's rows, the others by query tile; a mixed batch launches both.
template <bool SIG>
bool attention_tc(const atoma_softmax_attn_args &a, const float *head_bias, cudaStream_t stream, bool *taken) {
    *taken = false;
    const int64_t kmax = std::max(a.dim, a.vdim);
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (a.dtype != ATOMA_DTYPE_BF16 || a.max_query_len < 1 || !a.query_start || a.dim % 16 || a.vdim % 16 || kmax > 128 || !al(a.q) ||
        !al(a.k_cache) || !al(a.v_cache) || !al(a.out) || (a.gate && (!al(a.gate) || a.ld_gate % 8)) || current_device_info().cc_major < 9)
        return true;
    *taken = true;
    const int D = static_cast<int>(a.dim), DV = static_cast<int>(a.vdim);
    const int rep = static_cast<int>(a.H / a.G), chunks = (rep + 15) / 16;
    // single tokens
    {
        const TcLayout L = tc_layout(D, DV, 0);
        const size_t smem = std::max<size_t>(L.total, static_cast<size_t>(128 + 64 * DV) * 4);
        // a token's visible keys: the window and the kept first tokens, at most its whole sequence
        int64_t keys = a.max_seq_len > 0 ? a.max_seq_len : 0;
        if (a.window > 0) keys = std::min<int64_t>(keys, a.window + std::max<int64_t>(a.keep_first, 0) + kKeys);
        const int64_t tiles = (keys + kKeys - 1) / kKeys;
        const int64_t ctas = a.B * a.G * chunks;
        // a few CTAs per SM and several waves of them, so that the last wave's idle SMs cost little; at least four tiles per split
        int splits = 1;
        if (tiles >= 8 && ctas < 8 * current_device_info().sm_count)
            splits = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>({(8 * current_device_info().sm_count + ctas - 1) / ctas, tiles / 4, 32})));
        float *partial = nullptr;
        if (splits > 1) {
            partial = static_cast<float *>(get_workspace(stream, static_cast<size_t>(a.B) * a.H * splits * (DV + 2) * 4, kWorkspaceHybridAttn));
            if (!partial) return false;
        }
        const dim3 grid(static_cast<unsigned>(splits), static_cast<unsigned>(a.B), static_cast<unsigned>(a.G * chunks));
        const cudaError_t e = kmax <= 64 ? launch_tc<64, true, SIG>(a, grid, smem, 0, splits, partial, head_bias, stream)
                                         : launch_tc<128, true, SIG>(a, grid, smem, 0, splits, partial, head_bias, stream);
        if (!hybrid::launched(e, "softmax_attn_tc_kernel<heads>")) return false;
        if (splits > 1 &&
            !hybrid::launched(launch_ex(softmax_split_merge_kernel, dim3(static_cast<unsigned>(a.B), static_cast<unsigned>(a.H)), dim3(128), 0, stream,
                                        a, splits, static_cast<const float *>(partial)),
                              "softmax_split_merge_kernel"))
            return false;
    }
    if (a.max_query_len <= 1) return true;
    // portions
    const int bias_n = a.dist_bias ? static_cast<int>(std::min<int64_t>(a.dist_rows, kBiasSmem)) : 0;
    const TcLayout L = tc_layout(D, DV, bias_n);
    const dim3 grid(static_cast<unsigned>((a.max_query_len + kRowsCta - 1) / kRowsCta), static_cast<unsigned>(a.B), static_cast<unsigned>(a.H));
    const cudaError_t e = kmax <= 64 ? launch_tc<64, false, SIG>(a, grid, L.total, bias_n, 1, nullptr, head_bias, stream)
                                     : launch_tc<128, false, SIG>(a, grid, L.total, bias_n, 1, nullptr, head_bias, stream);
    return hybrid::launched(e, "softmax_attn_tc_kernel<tokens>");
}

bool hyb_softmax_attention_tc(const atoma_softmax_attn_args &a, cudaStream_t stream, bool *taken) {
    return attention_tc<false>(a, nullptr, stream, taken);
}

// Sigmoid attention whose heads do not talk to each other (no slopes, no cap on the scores, no mixing of the heads' weights: the
// caller knows) on the same kernels: weights sigmoid(score * scale + head_bias[h]), outputs the plain weighted sums.
bool hyb_sigmoid_attention_tc(const atoma_sigmoid_attn_args &s, cudaStream_t stream, bool *taken) {
    *taken = false;
    if (s.talk || s.softcap != 0.f || !s.query_start) return true;
    atoma_softmax_attn_args a{};
    a.q = s.q;
    a.k_cache = s.k_cache;
    a.v_cache = s.v_cache;
    a.out = s.out;
    a.positions = s.positions;
    a.token_seq = s.token_seq;
    a.query_start = s.query_start;
    a.block_tables = s.block_tables;
    a.T = s.T;
    a.B = s.B;
    a.max_blocks = s.max_blocks;
    a.H = s.H;
    a.G = s.G;
    a.dim = s.dim;
    a.vdim = s.vdim;
    a.block_size = s.block_size;
    a.scale = s.scale;
    a.dtype = s.dtype;
    a.max_query_len = s.max_query_len;
    a.max_seq_len = s.max_seq_len;
    return attention_tc<true>(a, s.head_bias, stream, taken);
}

}  // namespace atoma
