// Mixture-of-experts feed-forward on a mixed batch — include/atoma_hybrid.h.
//
// Router in float32 (logits in an order that does not depend on the batch, the score function, the `top` largest), then the routed
// experts without a host read: the (token, k) pairs are sorted by expert on the device into segments padded to
// whole row tiles, the pairs' input rows are gathered (scaled by the router's weight when the design scales the
// expert's input), and two grouped products run over the row tiles — gate/up with the clamped gated activation in
// the epilogue, then down.  A row's arithmetic does not depend on which tile or segment position it lands in,
// so a token's result is independent of the batch around it.  The token's rows are summed, in the order of k,
// by the residual kernel (atoma_gated_residual_norm).
#include "common.cuh"
#include "hybrid_common.cuh"
#include "tc_products.cuh"

#include "atoma_hybrid.h"

#include <algorithm>

namespace atoma {

extern int g_hybrid_debug;
int hyb_moe_umma_tile_rows();
bool hyb_moe_umma_ok(const void *x, const void *w, const void *out, int64_t K, int64_t ldo);
bool hyb_moe_grouped_umma(const void *x, const void *w, void *out, int64_t max_tiles, int64_t experts, int64_t N, int64_t K, bool glu,
                          const int32_t *tile_expert, const int32_t *meta, const int32_t *row_pair, const float *out_weight, float limit,
                          float alpha, float shift, int *error, cudaStream_t stream);

namespace {

using namespace hybrid;

constexpr int kTileRows = 64;
static_assert(kTileRows == tc::kTM, "the experts' segments are padded to the tensor-core kernel's row tile");
constexpr int kMaxExperts = 1024;

// ---------------------------------------------------------------------------------------------
// router: float32 logits, then the `top` largest per token
// A warp owns TT tokens x ET router rows (the shared expert's gate row rides as row `experts`).  Whatever the tile shape, a
// (token, row) logit is summed in ONE order — a lane adds its k values in ascending order, then the lanes fold in
// an xor tree — so a token's logits are bit-identical in a decode step and in a prompt's portion.
// ---------------------------------------------------------------------------------------------
template <typename T, int TT, int ET>
__global__ void __launch_bounds__(128) moe_logits_kernel(const T *__restrict__ h, const float *__restrict__ w_router,
                                                         const float *__restrict__ w_row_gate, float *__restrict__ z, int tokens, int width,
                                                         int experts, int rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int n_eg = (rows + ET - 1) / ET;
    const int64_t wid = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    const int t0 = static_cast<int>(wid / n_eg) * TT, e0 = static_cast<int>(wid % n_eg) * ET;
    if (t0 >= tokens) return;
    const T *hp[TT];
    const float *wp[ET];
#pragma unroll
    for (int i = 0; i < TT; ++i) hp[i] = t0 + i < tokens ? h + static_cast<int64_t>(t0 + i) * width : nullptr;
#pragma unroll
    for (int j = 0; j < ET; ++j) {
        const int e = e0 + j;
        wp[j] = e < experts ? w_router + static_cast<int64_t>(e) * width : (e == experts && e < rows ? w_row_gate : nullptr);
    }
    float acc[TT][ET];
#pragma unroll
    for (int i = 0; i < TT; ++i)
#pragma unroll
        for (int j = 0; j < ET; ++j) acc[i][j] = 0.f;
    // With 16-byte aligned rows a lane takes four consecutive k per step (k = 4 l .. 4 l + 3, then + 128, ...), otherwise one
    // (k = l, l + 32, ...): which of the two is a property of the model's width, not of the batch.
    const bool vec = width % 4 == 0 && (reinterpret_cast<uintptr_t>(h) & 15) == 0 && (reinterpret_cast<uintptr_t>(w_router) & 15) == 0 &&
                     (!w_row_gate || (reinterpret_cast<uintptr_t>(w_row_gate) & 15) == 0);
    if (vec) {
        for (int k = 4 * lane; k < width; k += 128) {
            float hv[TT][4], wv[ET][4];
#pragma unroll
            for (int i = 0; i < TT; ++i) {
                if (hp[i]) {
                    if constexpr (sizeof(T) == 2) {
                        const uint2 v = *reinterpret_cast<const uint2 *>(hp[i] + k);
                        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v.x));
                        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v.y));
                        hv[i][0] = a.x, hv[i][1] = a.y, hv[i][2] = c.x, hv[i][3] = c.y;
                    } else {
                        const float4 v = *reinterpret_cast<const float4 *>(hp[i] + k);
                        hv[i][0] = v.x, hv[i][1] = v.y, hv[i][2] = v.z, hv[i][3] = v.w;
                    }
                } else {
                    hv[i][0] = hv[i][1] = hv[i][2] = hv[i][3] = 0.f;
                }
            }
#pragma unroll
            for (int j = 0; j < ET; ++j) {
                const float4 v = wp[j] ? *reinterpret_cast<const float4 *>(wp[j] + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                wv[j][0] = v.x, wv[j][1] = v.y, wv[j][2] = v.z, wv[j][3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < TT; ++i)
#pragma unroll
                for (int j = 0; j < ET; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[i][j] = fmaf(hv[i][e], wv[j][e], acc[i][j]);
        }
    } else {
        for (int k = lane; k < width; k += 32) {
            float hv[TT], wv[ET];
#pragma unroll
            for (int i = 0; i < TT; ++i) hv[i] = hp[i] ? to_f(hp[i][k]) : 0.f;
#pragma unroll
            for (int j = 0; j < ET; ++j) wv[j] = wp[j] ? wp[j][k] : 0.f;
#pragma unroll
            for (int i = 0; i < TT; ++i)
#pragma unroll
                for (int j = 0; j < ET; ++j) acc[i][j] = fmaf(hv[i], wv[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TT; ++i)
#pragma unroll
        for (int j = 0; j < ET; ++j) {
            float v = acc[i][j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && hp[i] && wp[j]) z[static_cast<int64_t>(t0 + i) * rows + e0 + j] = v;
        }
}

// One warp per token: `top` rounds of arg-max over the logits (ties: the lower index), scores = sigmoid(logit).
__global__ void __launch_bounds__(128) moe_topk_kernel(const float *__restrict__ z, int32_t *__restrict__ top_expert,
                                                       float *__restrict__ top_weight, float *__restrict__ row_gate, int tokens, int experts,
                                                       int rows, int top, int renormalize) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const float *zr = z + t * rows;
    if (rows > experts && lane == 0) row_gate[t] = sigmoidf_(zr[experts]);
    uint32_t taken = 0;          // bit i: expert lane + 32 i is already chosen
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int idx = 0x7fffffff;
        for (int e = lane, i = 0; e < experts; e += 32, ++i) {
            const float v = zr[e];
            if (!((taken >> i) & 1u) && v > best) {   // ascending e: the lower index wins a tie
                best = v;
                idx = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ob > best || (ob == best && oi < idx)) {
                best = ob;
                idx = oi;
            }
        }
        if (idx != 0x7fffffff && (idx & 31) == lane) taken |= 1u << (idx >> 5);
        const float s = sigmoidf_(best);
        total += s;
        if (lane == 0) {
            top_expert[t * top + k] = idx == 0x7fffffff ? 0 : idx;
            top_weight[t * top + k] = s;
        }
    }
    __syncwarp();
    if (renormalize && lane == 0)
        for (int k = 0; k < top; ++k) top_weight[t * top + k] /= total;
}

// Router with a restricted choice: one warp per token over the float32 logits of all router outputs.
// s = softmax or sigmoid of the logits; c = s + correction; the outputs form `groups` equal groups of neighbours, a group's
// score is its largest c, only the `keep` best groups (ties: the lower group) can be chosen from; `top` rounds of arg-max of c
// among them (ties: the lower index); the weights are the chosen s, over their sum when renormalize.
constexpr int kMaxRouteGroups = 64;
__global__ void __launch_bounds__(32) moe_route_grouped_kernel(const float *__restrict__ z, const float *__restrict__ correction,
                                                              int32_t *__restrict__ top_expert, float *__restrict__ top_weight, int outputs,
                                                              int top, int groups, int keep, int score_fn, int renormalize) {
    __shared__ float s_s[kMaxExperts], c_s[kMaxExperts], gbest[kMaxRouteGroups];
    __shared__ int gkept[kMaxRouteGroups];
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x;
    const int64_t t = blockIdx.x;
    const float *zr = z + t * outputs;
    if (score_fn == ATOMA_SCORE_SOFTMAX) {
        float m = -INFINITY;
        for (int e = lane; e < outputs; e += 32) m = fmaxf(m, zr[e]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float sum = 0.f;
        for (int e = lane; e < outputs; e += 32) {
            const float v = expf(zr[e] - m);
            s_s[e] = v;
            sum += v;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = 1.0f / sum;
        for (int e = lane; e < outputs; e += 32) s_s[e] *= inv;
    } else {
        for (int e = lane; e < outputs; e += 32) s_s[e] = sigmoidf_(zr[e]);
    }
    for (int e = lane; e < outputs; e += 32) c_s[e] = s_s[e] + (correction ? correction[e] : 0.f);
    __syncwarp();
    if (groups > 1) {
        const int per = outputs / groups;
        for (int g = lane; g < groups; g += 32) {
            float b = -INFINITY;
            for (int e = 0; e < per; ++e) b = fmaxf(b, c_s[g * per + e]);
            gbest[g] = b;
            gkept[g] = 0;
        }
        __syncwarp();
        if (lane == 0) {
            for (int r = 0; r < keep; ++r) {
                int bi = -1;
                for (int g = 0; g < groups; ++g)
                    if (!gkept[g] && (bi < 0 || gbest[g] > gbest[bi])) bi = g;
                if (bi >= 0) gkept[bi] = 1;
            }
        }
        __syncwarp();
        for (int e = lane; e < outputs; e += 32)
            if (!gkept[e / per]) c_s[e] = -INFINITY;
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int idx = 0x7fffffff;
        for (int e = lane; e < outputs; e += 32) {
            const float v = c_s[e];
            if (v > best) {   // ascending e: the lower index wins a tie; chosen and excluded outputs are -inf
                best = v;
                idx = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ob > best || (ob == best && oi < idx)) {
                best = ob;
                idx = oi;
            }
        }
        const bool found = idx != 0x7fffffff;
        const float sv = found ? s_s[idx] : 0.f;
        total += sv;
        __syncwarp();
        if (lane == 0) {
            if (found) c_s[idx] = -INFINITY;
            top_expert[t * top + k] = found ? idx : -1;
            top_weight[t * top + k] = sv;
        }
        __syncwarp();
    }
    if (renormalize && lane == 0) {
        const float inv = 1.0f / (total + 1e-20f);
        for (int k = 0; k < top; ++k) top_weight[t * top + k] *= inv;
    }
}

// ---------------------------------------------------------------------------------------------
// pairs -> expert segments (one CTA)
// meta[0] = row tiles in use, meta[1] = rows in use (padded), meta[2] = error word of the grouped products (reset here)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int32_t *__restrict__ top_expert, int32_t *__restrict__ pair_row,
                                                        int32_t *__restrict__ row_pair, int32_t *__restrict__ tile_expert,
                                                        int32_t *__restrict__ meta, int pairs, int experts, int max_rows, int tile_rows) {
    __shared__ int count[kMaxExperts], base[kMaxExperts];
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    for (int r = threadIdx.x; r < max_rows; r += blockDim.x) row_pair[r] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = top_expert[i];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0;
        for (int e = 0; e < experts; ++e) {
            base[e] = row;
            const int tiles = (count[e] + tile_rows - 1) / tile_rows;
            for (int i = 0; i < tiles; ++i) tile_expert[row / tile_rows + i] = e;
            row += tiles * tile_rows;
            count[e] = 0;   // reused as the segment's cursor
        }
        meta[0] = row / tile_rows;
        meta[1] = row;
        meta[2] = 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
        const int e = top_expert[i];
        if (e < 0 || e >= experts) {
            pair_row[i] = 0;
            continue;
        }
        const int r = base[e] + atomicAdd(&count[e], 1);
        pair_row[i] = r;
        row_pair[r] = i;
    }
}

template <typename T>
__global__ void __launch_bounds__(128) moe_gather_kernel(const T *__restrict__ h, const float *__restrict__ top_weight,
                                                         const int32_t *__restrict__ row_pair, const int32_t *__restrict__ meta,
                                                         T *__restrict__ xs, int width, int top, int scale_input) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    if (row >= meta[1]) return;
    const int pair = row_pair[row];
    T *o = xs + static_cast<int64_t>(row) * width;
    if (pair < 0) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_f<T>(0.f);
        return;
    }
    const float w = scale_input ? top_weight[pair] : 1.f;
    const T *src = h + static_cast<int64_t>(pair / top) * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = from_f<T>(to_f(src[c]) * w);
}

// ---------------------------------------------------------------------------------------------
// grouped products over row tiles: float32 FMA, k ascending
// GLU = true:  out[row, n] = act(x w_gate[n]^T, x w_up[n]^T), weights of expert e at w + e * 2 N K (gate rows, up rows)
// GLU = false: out[row, n] = x w[n]^T (* the pair's router weight when out_weight), weights of expert e at w + e * N K
// ---------------------------------------------------------------------------------------------
template <typename T, bool GLU>
__global__ void __launch_bounds__(256) moe_grouped_kernel(const T *__restrict__ x, const T *__restrict__ w, T *__restrict__ out,
                                                          const int32_t *__restrict__ tile_expert, const int32_t *__restrict__ meta,
                                                          const int32_t *__restrict__ row_pair, const float *__restrict__ out_weight,
                                                          int N, int K, float limit, float alpha, float shift) {
    __shared__ float xs[16][65], ws[16][65], us[GLU ? 16 : 1][65];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.y;
    if (tile >= meta[0]) return;
    const int64_t e = tile_expert[tile];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = tile * kTileRows, n0 = blockIdx.x * 64;
    const T *wg = w + e * (GLU ? 2 : 1) * N * K;
    const T *wu = wg + static_cast<int64_t>(N) * K;
    float acc[4][4] = {}, acu[GLU ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i / 16, k = i % 16;
            const bool kin = k0 + k < K, nin = n0 + r < N;
            xs[k][r] = kin ? to_f(x[static_cast<int64_t>(m0 + r) * K + k0 + k]) : 0.f;
            ws[k][r] = (kin && nin) ? to_f(wg[static_cast<int64_t>(n0 + r) * K + k0 + k]) : 0.f;
            if constexpr (GLU) us[k][r] = (kin && nin) ? to_f(wu[static_cast<int64_t>(n0 + r) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float xv[4], wv[4], uv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                xv[i] = xs[k][ty * 4 + i];
                wv[i] = ws[k][tx * 4 + i];
                if constexpr (GLU) uv[i] = us[k][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
                    if constexpr (GLU) acu[i][j] = fmaf(xv[i], uv[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        float ow = 1.f;
        if (!GLU && out_weight != nullptr) {
            const int pair = row_pair[m];
            ow = pair >= 0 ? out_weight[pair] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v;
            if constexpr (GLU) v = glu_clamped(acc[i][j], acu[i][j], limit, alpha, shift);
            else v = acc[i][j] * ow;
            out[static_cast<int64_t>(m) * N + n] = from_f<T>(v);
        }
    }
}

inline int64_t up256(int64_t x) { return (x + 255) / 256 * 256; }

struct MoeSpace {
    int32_t *pair_row, *row_pair, *tile_expert, *meta;
    char *xs, *act, *y;
    int64_t max_tiles, max_rows, total;
};

MoeSpace carve(int64_t T, int64_t top, int64_t experts, int64_t width, int64_t ff, uint32_t dtype, void *base, int64_t tile_rows = kTileRows) {
    const int64_t es = dtype == ATOMA_DTYPE_F32 ? 4 : 2;
    MoeSpace s{};
    const int64_t pairs = T * top;
    s.max_tiles = std::min<int64_t>((pairs + tile_rows - 1) / tile_rows + experts, pairs);   // every tile in use holds a pair
    s.max_rows = s.max_tiles * tile_rows;
    int64_t off = 0;
    char *b = static_cast<char *>(base);
    auto take = [&](int64_t bytes) {
        char *p = b ? b + off : nullptr;
        off += up256(bytes);
        return p;
    };
    s.pair_row = reinterpret_cast<int32_t *>(take(pairs * 4));
    s.row_pair = reinterpret_cast<int32_t *>(take(s.max_rows * 4));
    s.tile_expert = reinterpret_cast<int32_t *>(take(s.max_tiles * 4));
    s.meta = reinterpret_cast<int32_t *>(take(16));
    s.xs = take(s.max_rows * width * es);
    s.act = take(s.max_rows * ff * es);
    s.y = take(s.max_rows * width * es);
    s.total = off;
    return s;
}

}  // namespace

#define HYB_DISPATCH(dtype, CALL) ((dtype) == ATOMA_DTYPE_BF16 ? CALL(__nv_bfloat16) : CALL(float))

bool hyb_moe_route(const void *h, const float *w_router, const float *w_row_gate, int32_t *top_expert, float *top_weight, float *row_gate,
                   int64_t T, int64_t width, int64_t experts, int64_t top, int32_t renormalize, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_moe_route")) return false;
    if (!h || !w_router || !top_expert || !top_weight || (w_row_gate && !row_gate) || width <= 0 || experts <= 0 || experts > kMaxExperts ||
        top <= 0 || top > experts) {
        set_status(kErrInvalidArg, "atoma_moe_route: null argument, or top %lld of %lld experts (at most %d experts)",
                   static_cast<long long>(top), static_cast<long long>(experts), kMaxExperts);
        return false;
    }
    const int rows = static_cast<int>(experts) + (w_row_gate ? 1 : 0);
    float *z = static_cast<float *>(get_workspace(stream, static_cast<size_t>(T) * rows * 4, kWorkspaceMoeRoute));
    if (!z) return false;
    cudaError_t e;
    if (T >= 256) {   // prompt portions: 8 x 4 (token, row) pairs per warp share their loads
        const int64_t warps = ((T + 7) / 8) * ((rows + 3) / 4);
#define CALL(TT) launch_ex(moe_logits_kernel<TT, 8, 4>, dim3(static_cast<unsigned>((warps + 3) / 4)), dim3(128), 0, stream, \
                           static_cast<const TT *>(h), w_router, w_row_gate, z, static_cast<int>(T), static_cast<int>(width), \
                           static_cast<int>(experts), rows)
        e = HYB_DISPATCH(dtype, CALL);
#undef CALL
    } else {          // decode steps: one pair per warp fills the device
        const int64_t warps = T * rows;
#define CALL(TT) launch_ex(moe_logits_kernel<TT, 1, 1>, dim3(static_cast<unsigned>((warps + 3) / 4)), dim3(128), 0, stream, \
                           static_cast<const TT *>(h), w_router, w_row_gate, z, static_cast<int>(T), static_cast<int>(width), \
                           static_cast<int>(experts), rows)
        e = HYB_DISPATCH(dtype, CALL);
#undef CALL
    }
    if (!hybrid::launched(e, "moe_logits_kernel")) return false;
    return hybrid::launched(launch_ex(moe_topk_kernel, dim3(static_cast<unsigned>((T + 3) / 4)), dim3(128), 0, stream,
                                      static_cast<const float *>(z), top_expert, top_weight, row_gate, static_cast<int>(T),
                                      static_cast<int>(experts), rows, static_cast<int>(top), static_cast<int>(renormalize)),
                            "moe_topk_kernel");
}

bool hyb_moe_route_grouped(const void *h, const float *w_router, const float *correction, int32_t *top_expert, float *top_weight, int64_t T,
                           int64_t width, int64_t outputs, int64_t top, int64_t groups, int64_t keep, int32_t score_fn, int32_t renormalize,
                           uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_moe_route_grouped")) return false;
    if (groups <= 1) groups = 1, keep = 1;
    if (!h || !w_router || !top_expert || !top_weight || width <= 0 || outputs <= 0 || outputs > kMaxExperts || top <= 0 || top > outputs ||
        groups > kMaxRouteGroups || outputs % groups || keep <= 0 || keep > groups || (score_fn != ATOMA_SCORE_SIGMOID && score_fn != ATOMA_SCORE_SOFTMAX)) {
        set_status(kErrInvalidArg, "atoma_moe_route_grouped: null argument, top %lld of %lld outputs (at most %d), or %lld of %lld groups (at most %d, equal sizes)",
                   static_cast<long long>(top), static_cast<long long>(outputs), kMaxExperts, static_cast<long long>(keep),
                   static_cast<long long>(groups), kMaxRouteGroups);
        return false;
    }
    const int rows = static_cast<int>(outputs);
    float *z = static_cast<float *>(get_workspace(stream, static_cast<size_t>(T) * rows * 4, kWorkspaceMoeRoute));
    if (!z) return false;
    const float *none = nullptr;
    cudaError_t e;
    if (T >= 256) {
        const int64_t warps = ((T + 7) / 8) * ((rows + 3) / 4);
#define CALL(TT) launch_ex(moe_logits_kernel<TT, 8, 4>, dim3(static_cast<unsigned>((warps + 3) / 4)), dim3(128), 0, stream, \
                           static_cast<const TT *>(h), w_router, none, z, static_cast<int>(T), static_cast<int>(width), rows, rows)
        e = HYB_DISPATCH(dtype, CALL);
#undef CALL
    } else {
        const int64_t warps = T * rows;
#define CALL(TT) launch_ex(moe_logits_kernel<TT, 1, 1>, dim3(static_cast<unsigned>((warps + 3) / 4)), dim3(128), 0, stream, \
                           static_cast<const TT *>(h), w_router, none, z, static_cast<int>(T), static_cast<int>(width), rows, rows)
        e = HYB_DISPATCH(dtype, CALL);
#undef CALL
    }
    if (!hybrid::launched(e, "moe_logits_kernel")) return false;
    return hybrid::launched(launch_ex(moe_route_grouped_kernel, dim3(static_cast<unsigned>(T)), dim3(32), 0, stream, static_cast<const float *>(z),
                                      correction, top_expert, top_weight, rows, static_cast<int>(top), static_cast<int>(groups),
                                      static_cast<int>(keep), static_cast<int>(score_fn), static_cast<int>(renormalize)),
                            "moe_route_grouped_kernel");
}

int64_t hyb_moe_workspace_bytes(int64_t T, int64_t top, int64_t experts, int64_t width, int64_t ff, uint32_t dtype) {
    if (T < 0 || top <= 0 || experts <= 0 || width <= 0 || ff <= 0) return -1;
    const int64_t t = std::max<int64_t>(T, 1);   // either tile size may be chosen at run time
    return std::max(carve(t, top, experts, width, ff, dtype, nullptr).total,
                    carve(t, top, experts, width, ff, dtype, nullptr, hyb_moe_umma_tile_rows()).total);
}

bool hyb_moe_experts(const atoma_moe_args &a, const void **expert_out, const int32_t **pair_row, cudaStream_t stream) {
    if (a.T <= 0) return true;
    if (!hybrid::known_dtype(a.dtype, "atoma_moe_experts")) return false;
    if (!a.h || !a.top_expert || !a.top_weight || !a.w_gate_up || !a.w_down || !a.workspace || a.width <= 0 || a.ff <= 0 || a.top <= 0 ||
        a.experts <= 0 || a.experts > kMaxExperts) {
        set_status(kErrInvalidArg, "atoma_moe_experts: null argument or empty shape");
        return false;
    }
    // prompt-sized steps in bfloat16: 128-row tiles on tcgen05; decode-sized steps: 64-row tiles on the warp-level path
    const bool umma = a.dtype == ATOMA_DTYPE_BF16 && !(g_hybrid_debug & 1) && (a.T * a.top >= 1024 || (g_hybrid_debug & 8)) &&
                      a.width >= 64 && a.ff >= 64 && hyb_moe_umma_ok(a.workspace, a.w_gate_up, a.workspace, a.width, a.ff) &&
                      hyb_moe_umma_ok(a.workspace, a.w_down, a.workspace, a.ff, a.width);
    const int64_t tile_rows = umma ? hyb_moe_umma_tile_rows() : kTileRows;
    const MoeSpace s = carve(a.T, a.top, a.experts, a.width, a.ff, a.dtype, a.workspace, tile_rows);
    if (s.total > a.workspace_bytes) {
        set_status(kErrInvalidArg, "atoma_moe_experts: workspace of %lld bytes, %lld needed", static_cast<long long>(a.workspace_bytes),
                   static_cast<long long>(s.total));
        return false;
    }
    const int pairs = static_cast<int>(a.T * a.top);
    if (!hybrid::launched(launch_ex(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, a.top_expert, s.pair_row, s.row_pair, s.tile_expert,
                                    s.meta, pairs, static_cast<int>(a.experts), static_cast<int>(s.max_rows), static_cast<int>(tile_rows)),
                          "moe_sort_kernel"))
        return false;
#define CALL(TT) launch_ex(moe_gather_kernel<TT>, dim3(static_cast<unsigned>(s.max_rows)), dim3(128), 0, stream, static_cast<const TT *>(a.h), \
                           a.top_weight, static_cast<const int32_t *>(s.row_pair), static_cast<const int32_t *>(s.meta), \
                           reinterpret_cast<TT *>(s.xs), static_cast<int>(a.width), static_cast<int>(a.top), static_cast<int>(a.scale_input))
    if (!hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "moe_gather_kernel")) return false;
#undef CALL
    const float *ow = a.scale_input ? nullptr : a.top_weight;
    if (umma) {
        if (!hyb_moe_grouped_umma(s.xs, a.w_gate_up, s.act, s.max_tiles, a.experts, a.ff, a.width, true, s.tile_expert, s.meta, s.row_pair,
                                  nullptr, a.limit, a.alpha, a.up_shift, s.meta + 2, stream))
            return false;
        if (!hyb_moe_grouped_umma(s.act, a.w_down, s.y, s.max_tiles, a.experts, a.width, a.ff, false, s.tile_expert, s.meta, s.row_pair, ow,
                                  0.f, 0.f, 0.f, s.meta + 2, stream))
            return false;
        if (expert_out) *expert_out = s.y;
        if (pair_row) *pair_row = s.pair_row;
        return true;
    }
    if (a.dtype == ATOMA_DTYPE_BF16 && !(g_hybrid_debug & 1)) {   // warp-level tensor cores
        tc::GemmArgs p{};
        p.a = s.xs, p.lda = a.width;
        p.b = static_cast<const __nv_bfloat16 *>(a.w_gate_up), p.b_zs = 2 * a.ff * a.width, p.b_ks = 1, p.b_ns = a.width;
        p.o = s.act, p.ldo = a.ff;
        p.M = static_cast<int>(s.max_rows), p.N = static_cast<int>(a.ff), p.K = static_cast<int>(a.width);
        p.tile_expert = s.tile_expert, p.meta = s.meta, p.row_pair = s.row_pair;
        p.limit = a.limit, p.alpha = a.alpha, p.shift = a.up_shift;
        const dim3 t1(static_cast<unsigned>((a.ff + 63) / 64), static_cast<unsigned>(s.max_tiles));
        if (!hybrid::launched(launch_ex(tc::gemm_kernel<__nv_bfloat16, __nv_bfloat16, true>, t1, dim3(128), 0, stream, p), "tc::gemm_kernel<glu>"))
            return false;
        p.a = s.act, p.lda = a.ff;
        p.b = static_cast<const __nv_bfloat16 *>(a.w_down), p.b_zs = a.width * a.ff, p.b_ns = a.ff;
        p.o = s.y, p.ldo = a.width;
        p.N = static_cast<int>(a.width), p.K = static_cast<int>(a.ff);
        p.out_weight = ow;
        const dim3 t2(static_cast<unsigned>((a.width + 63) / 64), static_cast<unsigned>(s.max_tiles));
        if (!hybrid::launched(launch_ex(tc::gemm_kernel<__nv_bfloat16, __nv_bfloat16, false>, t2, dim3(128), 0, stream, p), "tc::gemm_kernel<down>"))
            return false;
        if (expert_out) *expert_out = s.y;
        if (pair_row) *pair_row = s.pair_row;
        return true;
    }
    const float *no_weight = nullptr;
    const dim3 g1(static_cast<unsigned>((a.ff + 63) / 64), static_cast<unsigned>(s.max_tiles));
#define CALL(TT) launch_ex(moe_grouped_kernel<TT, true>, g1, dim3(256), 0, stream, reinterpret_cast<const TT *>(s.xs), \
                           static_cast<const TT *>(a.w_gate_up), reinterpret_cast<TT *>(s.act), static_cast<const int32_t *>(s.tile_expert), \
                           static_cast<const int32_t *>(s.meta), static_cast<const int32_t *>(s.row_pair), no_weight, \
                           static_cast<int>(a.ff), static_cast<int>(a.width), a.limit, a.alpha, a.up_shift)
    if (!hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "moe_grouped_kernel<glu>")) return false;
#undef CALL
    const dim3 g2(static_cast<unsigned>((a.width + 63) / 64), static_cast<unsigned>(s.max_tiles));
#define CALL(TT) launch_ex(moe_grouped_kernel<TT, false>, g2, dim3(256), 0, stream, reinterpret_cast<const TT *>(s.act), \
                           static_cast<const TT *>(a.w_down), reinterpret_cast<TT *>(s.y), static_cast<const int32_t *>(s.tile_expert), \
                           static_cast<const int32_t *>(s.meta), static_cast<const int32_t *>(s.row_pair), ow, static_cast<int>(a.width), \
                           static_cast<int>(a.ff), 0.f, 0.f, 0.f)
    if (!hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "moe_grouped_kernel<down>")) return false;
#undef CALL
    if (expert_out) *expert_out = s.y;
    if (pair_row) *pair_row = s.pair_row;
    return true;
}

}  // namespace atoma

using namespace atoma;

extern "C" void atoma_moe_route(const void *h, const float *w_router, const float *w_row_gate, int32_t *top_expert, float *top_weight,
                                float *row_gate, int64_t T, int64_t width, int64_t experts, int64_t top, int32_t renormalize, uint32_t dtype,
                                atoma_stream_t stream) {
    clear_status();
    hyb_moe_route(h, w_router, w_row_gate, top_expert, top_weight, row_gate, T, width, experts, top, renormalize, dtype,
                  static_cast<cudaStream_t>(stream));
}
extern "C" int64_t atoma_moe_workspace_bytes(int64_t T, int64_t top, int64_t experts, int64_t width, int64_t ff, uint32_t dtype) {
    return hyb_moe_workspace_bytes(T, top, experts, width, ff, dtype);
}
extern "C" void atoma_moe_experts(const atoma_moe_args *args, const void **expert_out, const int32_t **pair_row, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_moe_experts: args is NULL");
        return;
    }
    hyb_moe_experts(*args, expert_out, pair_row, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_moe_route_grouped(const void *h, const float *w_router, const float *correction, int32_t *top_expert, float *top_weight,
                                        int64_t T, int64_t width, int64_t outputs, int64_t top, int64_t groups, int64_t keep, int32_t score_fn,
                                        int32_t renormalize, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_moe_route_grouped(h, w_router, correction, top_expert, top_weight, T, width, outputs, top, groups, keep, score_fn, renormalize, dtype,
                          static_cast<cudaStream_t>(stream));
}
