// Softmax attention for LONG prompt portions on the tensor-memory prefill kernel (include/atoma_hybrid.h,
// atoma_softmax_attention_paged with long_seqs > 0): bfloat16 heads of 64 or 128, dim = vdim.
//
// For every sequence with at least long_min_q query tokens in the step:
//   1. softmax_long_plan_kernel fixes, on the device, the first key the portion's first query sees through the window and the
//      cumulative key offsets of the sequences;
//   2. paged_kv_gather_kernel copies those keys (normed) and values out of the pages into contiguous buffers;
//   3. prefill_attn_kernel (prefill_attention.cu: tcgen05, accumulators in tensor memory) runs causal attention with the window
//      and the distance term (the head's column of the table in shared memory, added to the scaled scores before the running
//      maximum), and writes the outputs and their log-sum-exp;
//   4. softmax_kept_merge_gate_kernel adds what the window hides but the kept first tokens show — at most keep_first keys per
//      row, read from the pages, merged through the log-sum-exp — and applies the output gate.
// Sequences below the threshold are served by the other kernels of the operator in the same step (they skip the long ones).
#include "common.cuh"
#include "hybrid_common.cuh"
#include "mha_params.h"

#include "atoma_hybrid.h"

#include <algorithm>
#include <cstring>

namespace atoma {

extern int g_hybrid_debug;
int try_launch_prefill_tc(const MhaParams &p, bool is_bf16, cudaStream_t stream);   // prefill_attention.cu

namespace {

using namespace hybrid;

__global__ void softmax_long_plan_kernel(const int32_t *__restrict__ query_start, const int64_t *__restrict__ positions, int B, int window,
                                         int min_q, int32_t *__restrict__ cu_k, int32_t *__restrict__ key_lo) {
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int acc = 0;
    for (int b = 0; b < B; ++b) {
        const int nq = query_start[b + 1] - query_start[b];
        int lo = 0, n = 0;
        if (nq >= min_q) {
            const int ctx = static_cast<int>(positions[query_start[b]]);
            lo = window > 0 ? max(0, ctx - window + 1) : 0;   // the first key the portion's first query sees
            n = ctx + nq - lo;
        }
        cu_k[b] = acc;
        key_lo[b] = lo;
        acc += n;
    }
    cu_k[B] = acc;
}

// One warp per gathered key: its row of the key cache and of the value cache (all key/value heads, `row` elements each).
__global__ void __launch_bounds__(256) paged_kv_gather_kernel(const __nv_bfloat16 *__restrict__ k_cache, const __nv_bfloat16 *__restrict__ v_cache,
                                                              const int32_t *__restrict__ block_tables, int64_t max_blocks,
                                                              const int32_t *__restrict__ cu_k, const int32_t *__restrict__ key_lo,
                                                              __nv_bfloat16 *__restrict__ k_out, __nv_bfloat16 *__restrict__ v_out, int row, int bs) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int n = cu_k[b + 1] - cu_k[b];
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= n) return;
    const int j = key_lo[b] + i;
    const int32_t *bt = block_tables + static_cast<int64_t>(b) * max_blocks;
    const int64_t slot = static_cast<int64_t>(bt[j / bs]) * bs + j % bs, dst = static_cast<int64_t>(cu_k[b] + i) * row;
    const uint4 *ks = reinterpret_cast<const uint4 *>(k_cache + slot * row), *vs = reinterpret_cast<const uint4 *>(v_cache + slot * row);
    uint4 *kd = reinterpret_cast<uint4 *>(k_out + dst), *vd = reinterpret_cast<uint4 *>(v_out + dst);
    for (int c = threadIdx.x & 31; c < row / 8; c += 32) {
        kd[c] = ks[c];
        vd[c] = vs[c];
    }
}

// One warp per (token of a long sequence, head): out <- merge(out, kept keys behind the window) * sigmoid(gate).
// PER = dim / 32 consecutive channels per lane (2 or 4: one 4- or 8-byte access).
template <int PER>
__device__ __forceinline__ void load_row(const __nv_bfloat16 *p, float (&v)[PER]) {
    if constexpr (PER == 4) {
        const uint2 r = *reinterpret_cast<const uint2 *>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.y));
        v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
    } else {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
        v[0] = a.x, v[1] = a.y;
    }
}
template <int PER>
__global__ void __launch_bounds__(128) softmax_kept_merge_gate_kernel(const atoma_softmax_attn_args a, const float *__restrict__ lse) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    constexpr int D = 32 * PER;
    const int H = static_cast<int>(a.H), G = static_cast<int>(a.G);
    const int64_t wid = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    const int64_t t = wid / H;
    const int h = static_cast<int>(wid % H);
    if (t >= a.T) return;
    const int b = a.token_seq[t];
    if (a.query_start[b + 1] - a.query_start[b] < a.long_min_q) return;
    const int p = static_cast<int>(a.positions[t]);
    const int lo = a.window > 0 ? max(0, p - static_cast<int>(a.window) + 1) : 0;
    const int kept = a.keep_first <= 0 ? 0 : (a.keep_first < lo ? static_cast<int>(a.keep_first) : lo);
    const int c0 = lane * PER;   // this lane's channels
    __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(a.out) + (t * H + h) * D + c0;
    float o[PER];
    load_row<PER>(out, o);
    if (kept > 0) {
        const int g = h / (H / G), bs = static_cast<int>(a.block_size), last_row = static_cast<int>(a.dist_rows) - 1;
        const int32_t *bt = a.block_tables + static_cast<int64_t>(b) * a.max_blocks;
        const __nv_bfloat16 *kc = static_cast<const __nv_bfloat16 *>(a.k_cache), *vc = static_cast<const __nv_bfloat16 *>(a.v_cache);
        float qv[PER], ok[PER];
        load_row<PER>(static_cast<const __nv_bfloat16 *>(a.q) + (t * H + h) * D + c0, qv);
#pragma unroll
        for (int i = 0; i < PER; ++i) ok[i] = 0.f;
        float m_k = -INFINITY, l_k = 0.f;
        for (int j = 0; j < kept; ++j) {
            const int64_t slot = static_cast<int64_t>(bt[j / bs]) * bs + j % bs;
            float kv[PER], vv[PER];
            load_row<PER>(kc + (slot * G + g) * D + c0, kv);
            load_row<PER>(vc + (slot * G + g) * D + c0, vv);
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < PER; ++i) dot = fmaf(qv[i], kv[i], dot);
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
            float sc = dot * a.scale;
            if (a.dist_bias) sc += a.dist_bias[static_cast<int64_t>(min(p - j, last_row)) * H + h];
            const float m_new = fmaxf(m_k, sc);
            const float corr = m_k == -INFINITY ? 0.f : expf(m_k - m_new), w = expf(sc - m_new);
            l_k = l_k * corr + w;
#pragma unroll
            for (int i = 0; i < PER; ++i) ok[i] = fmaf(w, vv[i], ok[i] * corr);
            m_k = m_new;
        }
        // the main pass's output is normalised: o_main exp(lse) is its numerator, exp(lse) its denominator
        const float L = lse[static_cast<int64_t>(h) * a.T + t];
        const float M = fmaxf(L, m_k);
        const float w_main = expf(L - M), w_kept = expf(m_k - M);
        const float inv = 1.f / (w_main + w_kept * l_k);
#pragma unroll
        for (int i = 0; i < PER; ++i) o[i] = (w_main * o[i] + w_kept * ok[i]) * inv;
    }
    if (a.gate) {
        float gv[PER];
        load_row<PER>(static_cast<const __nv_bfloat16 *>(a.gate) + t * a.ld_gate + h * D + c0, gv);
#pragma unroll
        for (int i = 0; i < PER; ++i) o[i] *= sigmoidf_(gv[i]);
    }
    if constexpr (PER == 4) {
        uint2 w;
        w.x = pack2<__nv_bfloat16>(o[0], o[1]);
        w.y = pack2<__nv_bfloat16>(o[2], o[3]);
        *reinterpret_cast<uint2 *>(out) = w;
    } else {
        *reinterpret_cast<uint32_t *>(out) = pack2<__nv_bfloat16>(o[0], o[1]);
    }
}

}  // namespace

// Shapes the long-portion path takes: bfloat16, equal key and value head sizes of 64 or 128, sm_100.
bool hyb_softmax_long_ok(const atoma_softmax_attn_args &a) {
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return a.dtype == ATOMA_DTYPE_BF16 && a.dim == a.vdim && (a.dim == 64 || a.dim == 128) && a.long_seqs > 0 && a.long_min_q >= 32 &&
           a.query_start && al(a.q) && al(a.out) && al(a.k_cache) && al(a.v_cache) && (!a.gate || (al(a.gate) && a.ld_gate % 8 == 0)) && a.scale > 0.f && a.T < (1ll << 26) &&
           current_device_info().cc_major == 10 && !(g_hybrid_debug & 2);
}

bool hyb_softmax_attention_long(const atoma_softmax_attn_args &a, cudaStream_t stream) {
    const int64_t row = a.G * a.dim, HD = a.H * a.dim;
    const int64_t kept_ctx = a.window > 0 ? std::min<int64_t>(a.long_ctx_sum, static_cast<int64_t>(a.long_seqs) * (a.window - 1)) : a.long_ctx_sum;
    const int64_t max_keys = a.long_tokens + kept_ctx;
    if (max_keys <= 0) return true;
    auto up = [](int64_t x) { return (x + 255) / 256 * 256; };
    const int64_t rows = max_keys + 128;   // the attention kernel's TMA boxes may start up to a tile before the end
    const int64_t b_int = up((2 * a.B + 2) * 4), b_kv = up(rows * row * 2), b_lse = up(a.H * a.T * 4);
    char *ws = static_cast<char *>(get_workspace(stream, static_cast<size_t>(b_int + 2 * b_kv + b_lse), kWorkspaceLatentExpand));
    if (!ws) return false;
    int32_t *cu_k = reinterpret_cast<int32_t *>(ws), *key_lo = cu_k + a.B + 1;
    __nv_bfloat16 *K = reinterpret_cast<__nv_bfloat16 *>(ws + b_int), *V = reinterpret_cast<__nv_bfloat16 *>(ws + b_int + b_kv);
    float *lse = reinterpret_cast<float *>(ws + b_int + 2 * b_kv);
    if (!hybrid::launched(launch_ex(softmax_long_plan_kernel, dim3(1), dim3(32), 0, stream, a.query_start, a.positions, static_cast<int>(a.B),
                                    static_cast<int>(std::min<int64_t>(a.window, 0x3fffffff)), static_cast<int>(a.long_min_q), cu_k, key_lo),
                          "softmax_long_plan_kernel"))
        return false;
    const int64_t span = a.window > 0 ? std::min<int64_t>(a.max_seq_len, a.window - 1 + a.max_query_len) : a.max_seq_len;
    const dim3 gg(static_cast<unsigned>((span + 7) / 8), static_cast<unsigned>(a.B));
    if (!hybrid::launched(launch_ex(paged_kv_gather_kernel, gg, dim3(256), 0, stream, static_cast<const __nv_bfloat16 *>(a.k_cache),
                                    static_cast<const __nv_bfloat16 *>(a.v_cache), a.block_tables, a.max_blocks, static_cast<const int32_t *>(cu_k),
                                    static_cast<const int32_t *>(key_lo), K, V, static_cast<int>(row), static_cast<int>(a.block_size)),
                          "paged_kv_gather_kernel"))
        return false;
    MhaParams p;
    std::memset(&p, 0, sizeof(p));
    p.q = a.q, p.k = K, p.v = V, p.o = a.out, p.lse = lse;
    p.cu_q = a.query_start, p.cu_k = cu_k;
    p.q_rs = p.o_rs = HD, p.k_rs = p.v_rs = row;
    p.q_hs = p.k_hs = p.v_hs = p.o_hs = a.dim;
    p.b = static_cast<int>(a.B), p.h = static_cast<int>(a.H), p.h_k = static_cast<int>(a.G), p.d = static_cast<int>(a.dim);
    p.seqlen_q = a.max_query_len, p.seqlen_k = static_cast<int>(span);
    p.page = 1;
    p.scale = a.scale, p.scale_log2 = a.scale * 1.4426950408889634f;
    p.is_causal = 1, p.k_cumulative = 1, p.unpadded_lse = 1;
    p.window_left = a.window > 0 ? static_cast<int>(std::min<int64_t>(a.window, 0x3fffffff)) : 0;
    p.min_len_q = a.long_min_q;
    p.dist_bias = a.dist_bias, p.dist_rows = static_cast<int>(a.dist_rows), p.dist_heads = static_cast<int>(a.H);
    const int r = try_launch_prefill_tc(p, true, stream);
    if (r != 1) {
        if (r == 0) set_status(kErrUnsupported, "atoma_softmax_attention_paged: the long portions are outside the tensor-memory attention kernel's envelope");
        return false;
    }
    const bool kept = a.keep_first > 0 && a.window > 0;
    if (!kept && !a.gate) return true;
    const int64_t warps = a.T * a.H;
    const dim3 grid(static_cast<unsigned>((warps + 3) / 4));
    const cudaError_t e = a.dim == 128 ? launch_ex(softmax_kept_merge_gate_kernel<4>, grid, dim3(128), 0, stream, a, static_cast<const float *>(lse))
                                       : launch_ex(softmax_kept_merge_gate_kernel<2>, grid, dim3(128), 0, stream, a, static_cast<const float *>(lse));
    return hybrid::launched(e, "softmax_kept_merge_gate_kernel");
}

}  // namespace atoma
