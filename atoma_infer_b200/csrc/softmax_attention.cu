// Softmax attention over a paged cache for mixed batches, with grouped key/value heads, a sliding window that also keeps
// the first tokens of the sequence, a bias looked up by query-key distance, and a sigmoid gate on the output —
// include/atoma_hybrid.h (atoma_softmax_attention_paged).
//
// A query at position p sees key j <= p when p - j < window or j < keep_first.  Its visible keys are therefore at most two
// runs, [0, min(keep_first, lo)) and [lo, p] with lo = max(0, p - window + 1); the kernels walk them as one list.
//
//  * softmax_attn_general_kernel<T>: one CTA per (query token, head), float32 FMA dot products, 128 keys per pass with a
//    running maximum; the float32 path, and the fallback for head sizes the tiles do not take.
//  * softmax_attn_tc_kernel (softmax_attention_tc.cu): bfloat16 caches on tensor cores.
//  * long prompt portions of bfloat16 heads of 64 / 128 (softmax_attention_long.cu): gathered keys and values on the tcgen05
//    prefill kernel, the kept first tokens merged afterwards.
// Scores, weights, running maxima and sums are float32; a row's tiles depend on its position and the layer's constants
// only, never on the batch.
#include "common.cuh"
#include "hybrid_common.cuh"

#include "atoma_hybrid.h"

#include <algorithm>

namespace atoma {

extern int g_hybrid_debug;
bool hyb_softmax_attention_tc(const atoma_softmax_attn_args &a, cudaStream_t stream, bool *taken);   // softmax_attention_tc.cu
bool hyb_softmax_long_ok(const atoma_softmax_attn_args &a);                                          // softmax_attention_long.cu
bool hyb_softmax_attention_long(const atoma_softmax_attn_args &a, cudaStream_t stream);

namespace {

using namespace hybrid;

constexpr int kGenThreads = 128;
constexpr int kGenOut = 4;       // outputs per thread: vdim <= 512

__device__ __forceinline__ float block_max(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[warp] = v;
    __syncthreads();
    float m = red[0];
    for (int i = 1; i < nwarp; ++i) m = fmaxf(m, red[i]);
    return m;
}

template <typename T>
__global__ void __launch_bounds__(kGenThreads) softmax_attn_general_kernel(const atoma_softmax_attn_args a) {
    extern __shared__ float sm[];
    __shared__ float red[32], w_s[kGenThreads];
    __shared__ int64_t slot_s[kGenThreads];
    pdl_launch_dependents();
    pdl_wait();
    const int H = static_cast<int>(a.H), G = static_cast<int>(a.G), D = static_cast<int>(a.dim), Dv = static_cast<int>(a.vdim);
    const int t = blockIdx.x, h = blockIdx.y, g = h / (H / G);
    const int b = a.token_seq[t];
    if (a.skip_min_q > 0 && a.query_start && a.query_start[b + 1] - a.query_start[b] >= a.skip_min_q) return;
    const int p = static_cast<int>(a.positions[t]);
    const int bs = static_cast<int>(a.block_size);
    const int32_t *bt = a.block_tables + static_cast<int64_t>(b) * a.max_blocks;
    const T *q = static_cast<const T *>(a.q) + (static_cast<int64_t>(t) * H + h) * D;
    const T *kc = static_cast<const T *>(a.k_cache);
    const T *vc = static_cast<const T *>(a.v_cache);
    float *q_s = sm;   // [D]
    for (int i = threadIdx.x; i < D; i += kGenThreads) q_s[i] = to_f(q[i]);
    const int lo = a.window > 0 ? max(0, p - static_cast<int>(a.window) + 1) : 0;
    const int kept = min(max(static_cast<int>(a.keep_first), 0), lo);
    const int n = kept + (p - lo + 1);
    const int last_row = static_cast<int>(a.dist_rows) - 1;
    float acc[kGenOut];
#pragma unroll
    for (int r = 0; r < kGenOut; ++r) acc[r] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    __syncthreads();
    for (int v0 = 0; v0 < n; v0 += kGenThreads) {
        const int v = v0 + threadIdx.x;
        float s = -INFINITY;
        int64_t slot = 0;
        if (v < n) {
            const int j = v < kept ? v : lo + (v - kept);
            slot = static_cast<int64_t>(bt[j / bs]) * bs + j % bs;
            const T *kr = kc + (slot * G + g) * D;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot = fmaf(q_s[d], to_f(kr[d]), dot);
            s = dot * a.scale;
            if (a.dist_bias) s += a.dist_bias[static_cast<int64_t>(min(p - j, last_row)) * H + h];
        }
        const float m_new = fmaxf(m_run, block_max(s, red));
        const float w = v < n ? expf(s - m_new) : 0.f;
        const float tile_sum = block_sum(w, red);   // its barriers also fence the previous pass's reads of w_s / slot_s
        w_s[threadIdx.x] = w;
        slot_s[threadIdx.x] = slot;
        const float corr = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
        l_run = l_run * corr + tile_sum;
        m_run = m_new;
        __syncthreads();
        const int nj = min(kGenThreads, n - v0);
#pragma unroll
        for (int r = 0; r < kGenOut; ++r) {
            const int d = threadIdx.x + r * kGenThreads;
            if (d < Dv) {
                float o = acc[r] * corr;
                for (int jj = 0; jj < nj; ++jj) o = fmaf(w_s[jj], to_f(vc[(slot_s[jj] * G + g) * Dv + d]), o);
                acc[r] = o;
            }
        }
        __syncthreads();
    }
    const float inv = 1.0f / l_run;
    T *o = static_cast<T *>(a.out) + (static_cast<int64_t>(t) * H + h) * Dv;
    const T *gt = a.gate ? static_cast<const T *>(a.gate) + static_cast<int64_t>(t) * a.ld_gate + h * Dv : nullptr;
#pragma unroll
    for (int r = 0; r < kGenOut; ++r) {
        const int d = threadIdx.x + r * kGenThreads;
        if (d < Dv) {
            float v = acc[r] * inv;
            if (gt) v *= sigmoidf_(to_f(gt[d]));
            o[d] = from_f<T>(v);
        }
    }
}

}  // namespace

#define HYB_DISPATCH(dtype, CALL) ((dtype) == ATOMA_DTYPE_BF16 ? CALL(__nv_bfloat16) : CALL(float))

bool hyb_softmax_attention(const atoma_softmax_attn_args &a, cudaStream_t stream) {
    if (a.T <= 0) return true;
    if (!hybrid::known_dtype(a.dtype, "atoma_softmax_attention_paged")) return false;
    if (!a.q || !a.k_cache || !a.v_cache || !a.out || !a.positions || !a.token_seq || !a.block_tables || a.H <= 0 || a.G <= 0 || a.H % a.G ||
        a.dim <= 0 || a.vdim <= 0 || a.block_size <= 0 || a.max_blocks <= 0 || (a.dist_bias && a.dist_rows <= 0) ||
        (a.gate && a.ld_gate < a.H * a.vdim)) {
        set_status(kErrInvalidArg, "atoma_softmax_attention_paged: null argument, inconsistent head counts, an empty distance table or a gate row shorter than the heads");
        return false;
    }
    if (a.skip_min_q == 0 && hyb_softmax_long_ok(a)) {
        // long portions on the tensor-memory kernel; the step's other sequences (if any) on the kernels below, which skip the long ones
        if (a.long_seqs < a.B) {
            atoma_softmax_attn_args rest = a;
            rest.skip_min_q = a.long_min_q;
            rest.long_seqs = 0;
            if (!hyb_softmax_attention(rest, stream)) return false;
        }
        return hyb_softmax_attention_long(a, stream);
    }
    if (!(g_hybrid_debug & 2)) {
        bool taken = false;
        const bool ok = hyb_softmax_attention_tc(a, stream, &taken);
        if (taken) return ok;
    }
    if (a.vdim > kGenThreads * kGenOut) {
        set_status(kErrUnsupported, "atoma_softmax_attention_paged: vdim = %lld exceeds %d", static_cast<long long>(a.vdim), kGenThreads * kGenOut);
        return false;
    }
    const size_t smem = static_cast<size_t>(a.dim) * 4;
    if (smem > 40 * 1024) {
        set_status(kErrUnsupported, "atoma_softmax_attention_paged: dim = %lld", static_cast<long long>(a.dim));
        return false;
    }
    const dim3 grid(static_cast<unsigned>(a.T), static_cast<unsigned>(a.H));
#define CALL(TT) launch_ex(softmax_attn_general_kernel<TT>, grid, dim3(kGenThreads), smem, stream, a)
    return hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "softmax_attn_general_kernel");
#undef CALL
}

}  // namespace atoma

using namespace atoma;

extern "C" void atoma_softmax_attention_paged(const atoma_softmax_attn_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_softmax_attention_paged: args is NULL");
        return;
    }
    hyb_softmax_attention(*args, static_cast<cudaStream_t>(stream));
}
