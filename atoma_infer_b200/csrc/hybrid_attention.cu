// Sigmoid attention over a paged cache, tensor-core kernel for portions of prompts (include/atoma_hybrid.h).
//
// A CTA owns 16 consecutive query tokens of one sequence and ALL heads: warp h computes head h.  The talking-heads
// mix needs every head's weight of a (query, key) pair before any head can apply it, so the CTA walks the keys in
// tiles of 32 and, per tile,
//   1. stages the tile's keys and values of every kv head in shared memory (cp.async through the block table; rows
//      past the sequence's end are zero-filled so that a masked weight never multiplies stale page contents),
//   2. warp h: S_h = Q_h K^T on mma.sync m16n8k16 (bf16 in, float32 out), then scale, soft cap, distance bias, head
//      bias and sigmoid in float32, causal mask as an exact zero, weights to shared memory as float32,
//   3. warp h: a'_h = sum_g talk[h, g] a_g in float32 straight into the A fragments of the second product,
//      O_h += a'_h V (bf16 in, float32 accumulators in registers).
// There is no softmax, hence no running maximum and no rescaling: tiles simply add, in position order.
// More heads than one CTA can hold (registers: a warp keeps its head's 16 x vdim float32 outputs) are spread over the
// CTAs of a thread-block cluster, `hpc` heads each: a CTA stages only its own kv heads, keeps its own heads' weights, and
// reads the other CTAs' weights for the mix through distributed shared memory (ld.shared::cluster) between two cluster
// barriers per tile.
// Tiles entirely behind the causal frontier are never visited.  Single decoded tokens of a mixed batch ride along as
// one-row tiles; decode-only batches take the split kernel of hybrid_ops.cu instead.
//
// Why mma.sync and not tcgen05 here: the M extent a CTA can offer is 16 query rows per head before the per-head
// float32 weights of a tile (H x rows x keys) outgrow shared memory, and the weight mix between the two products
// runs on CUDA cores; a 128-row tcgen05 tile per head would need the weights of all heads resident in tensor memory
// at once (H x 32 columns per 32 keys) with a tcgen05.ld / st round trip for the mix.
#include "common.cuh"
#include "hybrid_common.cuh"

#include "atoma_hybrid.h"

#include <algorithm>

namespace atoma {
namespace {

using namespace hybrid;

constexpr int kPfRows = 16;
// keys per tile: 32 for portions (the weight buffer holds 16 rows of every head), 64 for decode-only batches (one row:
// half as many barrier rounds per key)
constexpr int kPfKeysPrompt = 32, kPfKeysDecode = 64;

struct PfLayout {
    int k_off, v_off, p_off, talk_off, bias_off, slope_off, total;
};

// hpc = heads per CTA, gl = kv heads a CTA stages, H = all heads (the talking-heads matrix rows are kept whole)
// prow = query rows the weight buffer holds (16; 1 for decode-only batches, which lets several CTAs share an SM)
__host__ __device__ inline PfLayout pf_layout(int hpc, int gl, int H, int D, int DV, int stages, int prow, int kPfKeys, int kPfPStride) {
    PfLayout l;
    int off = 0;
    l.k_off = off;
    off += stages * gl * kPfKeys * (D + 8) * 2;
    l.v_off = off;
    off += stages * gl * kPfKeys * (DV + 8) * 2;
    l.p_off = off;
    off += H * prow * kPfPStride * 4;   // every head's weights of the tile: own heads computed here, the rest copied in
    l.talk_off = off;
    off += hpc * H * 4;
    l.bias_off = off;
    off += hpc * 4;
    l.slope_off = off;
    off += hpc * 4;
    l.total = off;
    return l;
}

__device__ __forceinline__ float4 ld_cluster_f4(uint32_t cluster_addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(cluster_addr));
    return v;
}

// The weight of one visible key with fast exponentials (ex2.approx + one Newton-free reciprocal): tanh(x) = 1 - 2 / (e^2x + 1).
// Relative error ~1e-6 of the weight — three orders below the bfloat16 rounding the weight gets before the second product.
__device__ __forceinline__ float sigmoid_weight_fast(float dot, float scale, float softcap, float inv_cap, float slope, float dist,
                                                     float head_bias) {
    float s = dot * scale;
    if (softcap > 0.f) s = softcap * (1.f - __fdividef(2.f, __expf(2.f * s * inv_cap) + 1.f));
    s = s - slope * dist + head_bias;
    return __fdividef(1.f, 1.f + __expf(-s));
}

template <int KMAX, int MAXWARPS, int kPfKeys>
__global__ void __launch_bounds__(32 * MAXWARPS, (MAXWARPS == 8 && kPfKeys == 32) ? 2 : 1) sigmoid_attn_prefill_kernel(const atoma_sigmoid_attn_args a, int hpc, int gl, int cs, int splits,
                                                                             float *__restrict__ partial, int stages) {
    constexpr int kPfPStride = kPfKeys + ((MAXWARPS == 8 && kPfKeys == 32) ? 4 : 8);   // +4: two such CTAs fit an SM at 32 heads
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int H = static_cast<int>(a.H), G = static_cast<int>(a.G), D = static_cast<int>(a.dim), DV = static_cast<int>(a.vdim);
    const int b = blockIdx.y;
    const int t_begin = a.query_start[b], n_q = a.query_start[b + 1] - t_begin;
    // splits > 1 (decode-only batches: one query row per sequence): blockIdx.x is the key split, not the query tile
    const int r0 = splits > 1 ? 0 : blockIdx.x * kPfRows;
    if (r0 >= n_q) return;
    const int rows = min(kPfRows, n_q - r0);
    const int tok0 = t_begin + r0;
    const int ctx = static_cast<int>(a.positions[t_begin]);
    const int p0 = ctx + r0, p_last = p0 + rows - 1, total = ctx + n_q;
    const int bs = static_cast<int>(a.block_size);
    const int32_t *bt = a.block_tables + static_cast<int64_t>(b) * a.max_blocks;
    const int hl = threadIdx.x >> 5, lane = threadIdx.x & 31, t4 = lane & 3, rq = lane >> 2;
    const int rank = cs > 1 ? static_cast<int>(cluster_ctarank()) : 0;
    const int h = rank * hpc + hl;                       // this warp's head
    const int c_lo = (rank * hpc) / (H / G);             // first kv head this CTA stages
    const int c = h / (H / G) - c_lo;                    // this warp's kv head among the staged ones
    const int nthreads = blockDim.x;
    const int prow = splits > 1 ? 1 : kPfRows;
    const PfLayout L = pf_layout(hpc, gl, H, D, DV, stages, prow, kPfKeys, kPfPStride);
    __nv_bfloat16 *Ks0 = reinterpret_cast<__nv_bfloat16 *>(smem + L.k_off);
    __nv_bfloat16 *Vs0 = reinterpret_cast<__nv_bfloat16 *>(smem + L.v_off);
    const int k_stage = gl * kPfKeys * (D + 8), v_stage = gl * kPfKeys * (DV + 8);   // elements per stage
    float *Ps = reinterpret_cast<float *>(smem + L.p_off);
    float *talk_s = reinterpret_cast<float *>(smem + L.talk_off);
    float *bias_s = reinterpret_cast<float *>(smem + L.bias_off);
    float *slope_s = reinterpret_cast<float *>(smem + L.slope_off);
    for (int i = threadIdx.x; i < hpc * H; i += nthreads) {
        const int row = rank * hpc + i / H, col = i % H;
        talk_s[i] = a.talk ? a.talk[row * H + col] : (row == col ? 1.f : 0.f);
    }
    for (int i = threadIdx.x; i < hpc; i += nthreads) {
        bias_s[i] = a.head_bias[rank * hpc + i];
        slope_s[i] = a.slopes ? a.slopes[rank * hpc + i] : 0.f;
    }
    const __nv_bfloat16 *kc = static_cast<const __nv_bfloat16 *>(a.k_cache);
    const __nv_bfloat16 *vc = static_cast<const __nv_bfloat16 *>(a.v_cache);

    // this warp's query fragments (A operand of m16n8k16: rows rq / rq + 8, k = 2 t4 .. + 1 and + 8)
    uint32_t qf[KMAX / 16][4];
    {
        const __nv_bfloat16 *q = static_cast<const __nv_bfloat16 *>(a.q) + static_cast<int64_t>(tok0) * H * D + h * D;
#pragma unroll
        for (int kk = 0; kk < KMAX / 16; ++kk) {
            qf[kk][0] = qf[kk][1] = qf[kk][2] = qf[kk][3] = 0u;
            if (kk * 16 < D) {
                const int col = kk * 16 + 2 * t4;
                if (rq < rows) {
                    qf[kk][0] = *reinterpret_cast<const uint32_t *>(q + static_cast<int64_t>(rq) * H * D + col);
                    qf[kk][2] = *reinterpret_cast<const uint32_t *>(q + static_cast<int64_t>(rq) * H * D + col + 8);
                }
                if (rq + 8 < rows) {
                    qf[kk][1] = *reinterpret_cast<const uint32_t *>(q + static_cast<int64_t>(rq + 8) * H * D + col);
                    qf[kk][3] = *reinterpret_cast<const uint32_t *>(q + static_cast<int64_t>(rq + 8) * H * D + col + 8);
                }
            }
        }
    }
    float o[KMAX / 8][4];
#pragma unroll
    for (int i = 0; i < KMAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const int ck = gl * D / 8, cv = gl * DV / 8;   // 16-byte pieces per staged cache row (this CTA's kv heads)
    __syncthreads();
    const float slope = slope_s[hl], hb = bias_s[hl];
    const float inv_cap = a.softcap > 0.f ? 1.f / a.softcap : 0.f;
    const uint32_t ps_base = smem_u32(Ps);
    int j_begin = 0, j_end = p_last + 1;
    if (splits > 1) {
        const int tiles = (p_last + kPfKeys) / kPfKeys, per = (tiles + splits - 1) / splits;
        j_begin = min(j_end, static_cast<int>(blockIdx.x) * per * kPfKeys);
        j_end = min(j_end, j_begin + per * kPfKeys);
    }

    // keys and values of one tile -> shared memory stage `st` (cp.async; rows past the sequence's end are zero-filled)
    auto stage_tile = [&](int j0, int st) {
        __nv_bfloat16 *Kd = Ks0 + st * k_stage, *Vd = Vs0 + st * v_stage;
        // warp w takes keys w, w + warps, ...; lane l the 16-byte pieces l, l + 32, ... of a row (their kv head and offset
        // do not depend on the key, so the divisions are hoisted out of the key loop)
        const int wid = threadIdx.x >> 5, nw = nthreads >> 5;
        for (int e = lane; e < ck; e += 32) {
            const int g = (e * 8) / D, d = (e * 8) % D;
            for (int jj = wid; jj < kPfKeys; jj += nw) {
                const int j = j0 + jj;
                const bool ok = j < total;
                const int64_t slot = ok ? static_cast<int64_t>(bt[j / bs]) * bs + j % bs : 0;
                cp_async_16(smem_u32(Kd + (g * kPfKeys + jj) * (D + 8) + d), kc + (slot * G + c_lo) * D + e * 8, ok ? 16 : 0);
            }
        }
        for (int e = lane; e < cv; e += 32) {
            const int g = (e * 8) / DV, d = (e * 8) % DV;
            for (int jj = wid; jj < kPfKeys; jj += nw) {
                const int j = j0 + jj;
                const bool ok = j < total;
                const int64_t slot = ok ? static_cast<int64_t>(bt[j / bs]) * bs + j % bs : 0;
                cp_async_16(smem_u32(Vd + (g * kPfKeys + jj) * (DV + 8) + d), vc + (slot * G + c_lo) * DV + e * 8, ok ? 16 : 0);
            }
        }
        cp_async_commit();
    };
    if (stages > 1 && j_begin < j_end) stage_tile(j_begin, 0);

    int it = 0;
    for (int j0 = j_begin; j0 < j_end; j0 += kPfKeys, ++it) {
        // 1. this tile's keys and values (with two stages: the next tile's copies are issued first and fly during the math)
        int st = 0;
        if (stages > 1) {
            st = it & 1;
            if (j0 + kPfKeys < j_end) {
                stage_tile(j0 + kPfKeys, st ^ 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                cp_async_wait_all();
            }
        } else {
            stage_tile(j0, 0);
            cp_async_wait_all();
        }
        const __nv_bfloat16 *Ks = Ks0 + st * k_stage, *Vs = Vs0 + st * v_stage;
        __syncthreads();

        // 2. scores and weights of this warp's head
        float sacc[kPfKeys / 8][4];
#pragma unroll
        for (int i = 0; i < kPfKeys / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KMAX / 16; ++kk) {
            if (kk * 16 < D) {
#pragma unroll
                for (int np = 0; np < kPfKeys / 16; ++np) {
                    uint32_t r[4];
                    const __nv_bfloat16 *src = Ks + (c * kPfKeys + (np * 2 + (lane >> 4)) * 8 + (lane & 7)) * (D + 8) + kk * 16 +
                                               ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(r, smem_u32(src));
                    Mma16816<__nv_bfloat16>::run(sacc[np * 2], qf[kk], r[0], r[1]);
                    Mma16816<__nv_bfloat16>::run(sacc[np * 2 + 1], qf[kk], r[2], r[3]);
                }
            }
        }
        if (prow == 1) {
            // decode-only batch: the one query row's raw scores sit in lanes 0..3; spread them over the warp (lane = key) through
            // the weight buffer so that every lane evaluates its own keys' weights instead of four lanes evaluating all of them
            float *prow_s = Ps + h * kPfPStride;
            if (rq == 0) {
#pragma unroll
                for (int nt = 0; nt < kPfKeys / 8; ++nt)
                    *reinterpret_cast<float2 *>(prow_s + nt * 8 + 2 * t4) = make_float2(sacc[nt][0], sacc[nt][1]);
            }
            __syncwarp();
#pragma unroll
            for (int u = 0; u < kPfKeys / 32; ++u) {
                const int j = j0 + u * 32 + lane;
                const float raw = prow_s[u * 32 + lane];
                prow_s[u * 32 + lane] = j <= p0 ? sigmoid_weight_fast(raw, a.scale, a.softcap, inv_cap, slope, static_cast<float>(p0 - j), hb) : 0.f;
            }
        } else {
#pragma unroll
        for (int nt = 0; nt < kPfKeys / 8; ++nt) {
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = rq + (e >> 1) * 8, j = j0 + nt * 8 + 2 * t4 + (e & 1), p = p0 + row;
                w[e] = (row < rows && j <= p)
                           ? sigmoid_weight_fast(sacc[nt][e], a.scale, a.softcap, inv_cap, slope, static_cast<float>(p - j), hb) : 0.f;
            }
            float *dst = Ps + (h * prow + rq) * kPfPStride + nt * 8 + 2 * t4;
            *reinterpret_cast<float2 *>(dst) = make_float2(w[0], w[1]);
            *reinterpret_cast<float2 *>(dst + 8 * kPfPStride) = make_float2(w[2], w[3]);
        }
        }
        if (cs > 1) {
            // the other CTAs' heads: copy their slices of the tile's weights into this CTA's buffer (16-byte loads through
            // distributed shared memory, all in flight at once), between two cluster barriers
            cluster_arrive_release();
            cluster_wait_acquire();
            const int row_f4 = kPfPStride / 4, per_head = rows * row_f4;   // float4 of a head's rows in use (contiguous)
            for (int idx = threadIdx.x; idx < per_head; idx += nthreads)
            for (int hd0 = 0; hd0 < H; hd0 += 4) {
                float4 v[4];
                int off[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int hd = hd0 + u, src_rank = hd / hpc;
                    off[u] = -1;
                    if (hd < H && src_rank != rank) {
                        off[u] = (hd * prow * row_f4 + idx) * 16;
                        v[u] = ld_cluster_f4(mapa_shared(ps_base + off[u], static_cast<uint32_t>(src_rank)));
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (off[u] >= 0) *reinterpret_cast<float4 *>(reinterpret_cast<unsigned char *>(Ps) + off[u]) = v[u];
            }
            cluster_arrive_release();
            cluster_wait_acquire();
        } else {
            __syncthreads();
        }

        // 3. mix the heads' weights and apply them to this warp's values
        float mk[kPfKeys / 32];   // one query row: lane = keys lane, lane + 32, ... of the tile
#pragma unroll
        for (int u = 0; u < kPfKeys / 32; ++u) mk[u] = 0.f;
        if (rows == 1)
#pragma unroll 4
            for (int g = 0; g < H; ++g) {
                const float tg = talk_s[hl * H + g];
#pragma unroll
                for (int u = 0; u < kPfKeys / 32; ++u) mk[u] = fmaf(tg, Ps[g * prow * kPfPStride + u * 32 + lane], mk[u]);
            }
#pragma unroll
        for (int kk = 0; kk < kPfKeys / 16; ++kk) {
            float m[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) m[i] = 0.f;
            if (rows == 1) {
                // the A fragment's row 0 is gathered with shuffles
                const int k0 = (kk * 16) % 32 + 2 * t4;
                const float mv = mk[(kk * 16) / 32];
                const float v0 = __shfl_sync(0xffffffffu, mv, k0), v1 = __shfl_sync(0xffffffffu, mv, k0 + 1);
                const float v4 = __shfl_sync(0xffffffffu, mv, k0 + 8), v5 = __shfl_sync(0xffffffffu, mv, k0 + 9);
                if (rq == 0) {
                    m[0] = v0;
                    m[1] = v1;
                    m[4] = v4;
                    m[5] = v5;
                }
            } else {
                const bool lower = rows > 8;     // rows 8 .. 15 exist
#pragma unroll 4
                for (int g = 0; g < H; ++g) {
                    const float tg = talk_s[hl * H + g];
                    const float *src = Ps + (g * prow + rq) * kPfPStride + kk * 16 + 2 * t4;
                    const float2 x0 = *reinterpret_cast<const float2 *>(src);
                    const float2 x2 = *reinterpret_cast<const float2 *>(src + 8);
                    m[0] = fmaf(tg, x0.x, m[0]);
                    m[1] = fmaf(tg, x0.y, m[1]);
                    m[4] = fmaf(tg, x2.x, m[4]);
                    m[5] = fmaf(tg, x2.y, m[5]);
                    if (lower) {
                        const float2 x1 = *reinterpret_cast<const float2 *>(src + 8 * kPfPStride);
                        const float2 x3 = *reinterpret_cast<const float2 *>(src + 8 * kPfPStride + 8);
                        m[2] = fmaf(tg, x1.x, m[2]);
                        m[3] = fmaf(tg, x1.y, m[3]);
                        m[6] = fmaf(tg, x3.x, m[6]);
                        m[7] = fmaf(tg, x3.y, m[7]);
                    }
                }
            }
            uint32_t af[4];
            af[0] = pack2<__nv_bfloat16>(m[0], m[1]);
            af[1] = pack2<__nv_bfloat16>(m[2], m[3]);
            af[2] = pack2<__nv_bfloat16>(m[4], m[5]);
            af[3] = pack2<__nv_bfloat16>(m[6], m[7]);
#pragma unroll
            for (int n2 = 0; n2 < KMAX / 16; ++n2) {
                if (n2 * 16 < DV) {
                    uint32_t r[4];
                    const __nv_bfloat16 *src = Vs + (c * kPfKeys + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * (DV + 8) + n2 * 16 +
                                               (lane >> 4) * 8;
                    ldmatrix_x4_trans(r, smem_u32(src));
                    Mma16816<__nv_bfloat16>::run(o[n2 * 2], af, r[0], r[1]);
                    Mma16816<__nv_bfloat16>::run(o[n2 * 2 + 1], af, r[2], r[3]);
                }
            }
        }
        __syncthreads();   // this tile's keys, values and weights are done with (remote readers finished before the mix)
    }

    if (partial) {   // this key split's float32 sums (one query row per sequence)
        if (rq == 0) {
            float *po = partial + (static_cast<int64_t>(tok0) * splits + blockIdx.x) * H * DV + h * DV;
#pragma unroll
            for (int nt = 0; nt < KMAX / 8; ++nt)
                if (nt * 8 < DV) *reinterpret_cast<float2 *>(po + nt * 8 + 2 * t4) = make_float2(o[nt][0], o[nt][1]);
        }
        return;
    }
    __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(a.out) + static_cast<int64_t>(tok0) * H * DV + h * DV;
#pragma unroll
    for (int nt = 0; nt < KMAX / 8; ++nt) {
        if (nt * 8 < DV) {
            const int col = nt * 8 + 2 * t4;
            if (rq < rows) *reinterpret_cast<uint32_t *>(out + static_cast<int64_t>(rq) * H * DV + col) = pack2<__nv_bfloat16>(o[nt][0], o[nt][1]);
            if (rq + 8 < rows)
                *reinterpret_cast<uint32_t *>(out + static_cast<int64_t>(rq + 8) * H * DV + col) = pack2<__nv_bfloat16>(o[nt][2], o[nt][3]);
        }
    }
}

template <int KMAX, int MAXWARPS, int KEYS>
cudaError_t launch_prefill(const atoma_sigmoid_attn_args &a, int hpc, int gl, int cs, int splits, float *partial, int stages,
                           size_t smem_bytes, cudaStream_t stream) {
    static int attr_dev = -1;
    const int dev = current_device_info().ordinal;
    if (attr_dev != dev) {
        cudaFuncSetAttribute(sigmoid_attn_prefill_kernel<KMAX, MAXWARPS, KEYS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_dev = dev;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(splits > 1 ? splits : (a.max_query_len + kPfRows - 1) / kPfRows), static_cast<unsigned>(a.B),
                       static_cast<unsigned>(cs));
    cfg.blockDim = dim3(static_cast<unsigned>(32 * hpc));
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cs > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = static_cast<unsigned>(cs);
        ++n;
    }
    if (launch_flags() & kLaunchPdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, sigmoid_attn_prefill_kernel<KMAX, MAXWARPS, KEYS>, a, hpc, gl, cs, splits, partial, stages);
}

}  // namespace

bool hyb_attn_split_reduce(const float *partial, void *out, int64_t T, int splits, int64_t n, uint32_t dtype, cudaStream_t stream);

// Takes bfloat16 batches with head sizes the tiles cover: mixed batches and prompt portions by query tile, decode-only
// batches by key split.
bool hyb_attention_fast(const atoma_sigmoid_attn_args &a, cudaStream_t stream, bool *taken) {
    *taken = false;
    const int64_t kmax = std::max(a.dim, a.vdim);
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (a.dtype != ATOMA_DTYPE_BF16 || a.max_query_len < 1 || !a.query_start || a.dim % 16 || a.vdim % 16 || kmax > 128 ||
        !al(a.q) || !al(a.k_cache) || !al(a.v_cache) || !al(a.out) || current_device_info().cc_major < 9)
        return true;
    // heads per CTA: the largest divisor of H that the register budget allows, with at most 8 CTAs per cluster and whole
    // kv-head groups per CTA (or several CTAs inside one group)
    const int H = static_cast<int>(a.H), G = static_cast<int>(a.G), rep = H / G;
    const int maxw = kmax <= 64 ? 16 : 8;
    int hpc = 0, gl = 0;
    for (int cand = std::min(H, maxw); cand >= 1; --cand) {
        if (H % cand || H / cand > 8) continue;
        if (cand % rep != 0 && rep % cand != 0) continue;
        const int g = cand % rep == 0 ? cand / rep : 1;
        if (pf_layout(cand, g, H, static_cast<int>(a.dim), static_cast<int>(a.vdim), 1, kPfRows, kPfKeysPrompt, kPfKeysPrompt + 8).total > 200 * 1024) continue;
        hpc = cand;
        gl = g;
        break;
    }
    if (!hpc) return true;
    const int cs = H / hpc;
    *taken = true;
    // decode-only batches: every sequence has ONE query row, so the keys are split over CTAs until the device is full;
    // the splits' float32 sums are added in split order by a second kernel (no softmax: partial results simply add)
    int splits = 1;
    float *partial = nullptr;
    if (a.max_query_len == 1 && a.max_seq_len > 2 * kPfKeysDecode) {
        const int64_t ctas = a.B * cs, tiles = (a.max_seq_len + kPfKeysDecode - 1) / kPfKeysDecode;
        // (measured: the time does not depend on this factor between 2 and 24 — the kernel is bound by its per-tile work)
        const int64_t want = (6 * current_device_info().sm_count + ctas - 1) / ctas;
        splits = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>({want, tiles / 2, 64})));
        if (splits > 1) {
            partial = static_cast<float *>(get_workspace(stream, static_cast<size_t>(a.T) * splits * a.H * a.vdim * 4, kWorkspaceHybridAttn));
            if (!partial) return false;
        }
    }
    // two staging buffers (the next tile's copies fly during the math) whenever they fit
    // (measured at 32 heads of 128: one double-buffered CTA per SM beats two single-buffered ones, 8.1 vs 9.1 ms at 4k tokens)
    const int prow = splits > 1 ? 1 : kPfRows, keys = splits > 1 ? kPfKeysDecode : kPfKeysPrompt;
    const int pstride = keys + ((kmax > 64 && keys == kPfKeysPrompt) ? 4 : 8);
    int stages = pf_layout(hpc, gl, H, static_cast<int>(a.dim), static_cast<int>(a.vdim), 2, prow, keys, pstride).total <= 200 * 1024 ? 2 : 1;
    if (splits == 1 && kmax > 64 && stages == 2) {   // 8-warp CTAs of 128 registers: two per SM when one staging buffer lets them fit
        const int one = pf_layout(hpc, gl, H, static_cast<int>(a.dim), static_cast<int>(a.vdim), 1, prow, keys, pstride).total + 1024;
        const int two = pf_layout(hpc, gl, H, static_cast<int>(a.dim), static_cast<int>(a.vdim), 2, prow, keys, pstride).total + 1024;
        if (2 * one <= 227 * 1024 && 2 * two > 227 * 1024) stages = 1;
    }
    PfLayout L = pf_layout(hpc, gl, H, static_cast<int>(a.dim), static_cast<int>(a.vdim), stages, prow, keys, pstride);
    if (L.total > 200 * 1024) {   // many kv heads per CTA at 64 keys: the decode-only batch runs as one-row tiles of 32 keys, unsplit
        splits = 1;
        partial = nullptr;
        stages = pf_layout(hpc, gl, H, static_cast<int>(a.dim), static_cast<int>(a.vdim), 2, kPfRows, kPfKeysPrompt, kPfKeysPrompt + ((kmax > 64) ? 4 : 8)).total <= 200 * 1024 ? 2 : 1;
        L = pf_layout(hpc, gl, H, static_cast<int>(a.dim), static_cast<int>(a.vdim), stages, kPfRows, kPfKeysPrompt, kPfKeysPrompt + ((kmax > 64) ? 4 : 8));
    }
    cudaError_t e;
    if (splits > 1)
        e = kmax <= 64 ? launch_prefill<64, 16, kPfKeysDecode>(a, hpc, gl, cs, splits, partial, stages, L.total, stream)
                       : launch_prefill<128, 8, kPfKeysDecode>(a, hpc, gl, cs, splits, partial, stages, L.total, stream);
    else
        e = kmax <= 64 ? launch_prefill<64, 16, kPfKeysPrompt>(a, hpc, gl, cs, splits, partial, stages, L.total, stream)
                       : launch_prefill<128, 8, kPfKeysPrompt>(a, hpc, gl, cs, splits, partial, stages, L.total, stream);
    note_launch();
    if (e != cudaSuccess) {
        set_status(static_cast<int>(e), "sigmoid_attn_prefill_kernel: %s", cudaGetErrorString(e));
        return false;
    }
    if (!check_launch("sigmoid_attn_prefill_kernel")) return false;
    if (splits > 1) return hyb_attn_split_reduce(partial, a.out, a.T, splits, a.H * a.vdim, a.dtype, stream);
    return true;
}

}  // namespace atoma
