// Row-wise operators of pre-norm decoder layers with gated residuals — include/atoma_hybrid.h:
// learned positions, RMS norms over groups of the row, the residual update with its sigmoid gate (and the
// sum of a token's expert rows) fused with the next sublayer's norm, the token side input, the clamped
// gated activation.  The residual stream, every statistic and every gate are float32 whatever the
// activation format; each row is reduced in an order that depends on the row alone.
#include "common.cuh"
#include "hybrid_common.cuh"

#include "atoma_hybrid.h"

#include <algorithm>

namespace atoma {
namespace {

using namespace hybrid;

constexpr int kMaxNormGroups = 64;
constexpr int kMaxTopRows = 64;      // expert rows summed per token

template <typename T>
__global__ void __launch_bounds__(128) embed_learned_kernel(const uint32_t *__restrict__ tokens, const int64_t *__restrict__ positions,
                                                            const T *__restrict__ table, const T *__restrict__ pos_table,
                                                            float *__restrict__ out, int width, int64_t vocab, int64_t max_positions) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int64_t tok = tokens[t];
    if (tok >= vocab) tok = vocab - 1;
    int64_t p = positions[t];
    if (p >= max_positions) p = max_positions - 1;
    if (p < 0) p = 0;
    const T *e = table + tok * width, *q = pos_table + p * width;
    float *o = out + static_cast<int64_t>(t) * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = to_f(e[c]) + to_f(q[c]);
}

// Four consecutive elements at once (8 bytes of bfloat16, 16 of float32); the caller has checked the alignment.
__device__ __forceinline__ float4 load4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16 *p) {
    const uint2 v = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float *p, const float4 &v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16 *p, const float4 &v) {
    uint2 w;
    w.x = pack2<__nv_bfloat16>(v.x, v.y);
    w.y = pack2<__nv_bfloat16>(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) = w;
}
__device__ __forceinline__ bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// row [width] float32 in shared memory -> out = row / sqrt(mean over the element's group + eps) * (offset + w).
// Every thread of the CTA must call it.
template <typename T>
__device__ __forceinline__ void group_norm_store(const float *row, int width, int groups, float eps, const float *__restrict__ w,
                                                 float offset, T *__restrict__ out, float *red, float *inv_s) {
    const int gw = width / groups;
    for (int g = 0; g < groups; ++g) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < gw; c += blockDim.x) {
            const float v = row[g * gw + c];
            ss = fmaf(v, v, ss);
        }
        const float tot = block_sum(ss, red);
        if (threadIdx.x == 0) inv_s[g] = 1.0f / sqrtf(tot / static_cast<float>(gw) + eps);
    }
    __syncthreads();
    if (gw % 4 == 0 && aligned16(out) && aligned16(w)) {
        for (int c = 4 * threadIdx.x; c < width; c += 4 * blockDim.x) {
            const float inv = inv_s[c / gw];
            const float4 wv = load4(w + c);
            store4(out + c, make_float4(row[c] * inv * (offset + wv.x), row[c + 1] * inv * (offset + wv.y), row[c + 2] * inv * (offset + wv.z),
                                        row[c + 3] * inv * (offset + wv.w)));
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[c] = from_f<T>(row[c] * inv_s[c / gw] * (offset + w[c]));
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads) group_rmsnorm_rows_kernel(const float *__restrict__ x, const int32_t *__restrict__ rows,
                                                                         const float *__restrict__ weight, float offset, int groups,
                                                                         T *__restrict__ out, int width, float eps) {
    extern __shared__ float row[];
    __shared__ float red[32], inv_s[kMaxNormGroups];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float *xr = x + static_cast<int64_t>(rows ? rows[r] : r) * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = xr[c];
    __syncthreads();
    group_norm_store<T>(row, width, groups, eps, weight, offset, out + static_cast<int64_t>(r) * width, red, inv_s);
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads) gated_residual_norm_kernel(const atoma_gated_residual_args a) {
    extern __shared__ float row[];
    __shared__ float red[32], inv_s[kMaxNormGroups];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    const int width = static_cast<int>(a.width), top = static_cast<int>(a.top);
    const T *y = a.y ? static_cast<const T *>(a.y) + t * a.ld_y : nullptr;
    const T *gate = a.gate ? static_cast<const T *>(a.gate) + t * a.ld_gate : nullptr;
    const T *eo = static_cast<const T *>(a.expert_out);
    const float rs = (y && a.row_scale) ? a.row_scale[t] : 1.f;
    float *x = a.x + t * width;
    T *xc = a.x_cast ? static_cast<T *>(a.x_cast) + t * width : nullptr;
    __shared__ int64_t erow[kMaxTopRows];       // the token's expert rows, read once (not once per channel)
    if (eo) {
        for (int k = threadIdx.x; k < top; k += blockDim.x) erow[k] = static_cast<int64_t>(a.pair_row[t * top + k]) * width;
        __syncthreads();
    }
    const bool vec = width % 4 == 0 && aligned16(x) && (!y || (a.ld_y % 4 == 0 && aligned16(y))) &&
                     (!gate || (a.ld_gate % 4 == 0 && aligned16(gate) && aligned16(a.gate_bias))) && (!eo || aligned16(eo)) &&
                     (!xc || aligned16(xc));
    if (vec) {   // the same arithmetic per element, four elements per load
        for (int c = 4 * threadIdx.x; c < width; c += 4 * blockDim.x) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (y) {
                const float4 t4 = load4(y + c);
                v = make_float4(t4.x * rs, t4.y * rs, t4.z * rs, t4.w * rs);
            }
            if (eo)
                for (int k = 0; k < top; ++k) {
                    const float4 e4 = load4(eo + erow[k] + c);
                    v.x += e4.x, v.y += e4.y, v.z += e4.z, v.w += e4.w;
                }
            if (gate) {
                const float4 g4 = load4(gate + c), b4 = load4(a.gate_bias + c);
                v.x *= sigmoidf_(g4.x + b4.x), v.y *= sigmoidf_(g4.y + b4.y), v.z *= sigmoidf_(g4.z + b4.z), v.w *= sigmoidf_(g4.w + b4.w);
            }
            const float4 x4 = load4(x + c);
            const float4 o4 = make_float4(x4.x + v.x, x4.y + v.y, x4.z + v.z, x4.w + v.w);
            store4(x + c, o4);
            row[c] = o4.x, row[c + 1] = o4.y, row[c + 2] = o4.z, row[c + 3] = o4.w;
            if (xc) store4(xc + c, o4);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            float v = y ? to_f(y[c]) * rs : 0.f;
            if (eo)
                for (int k = 0; k < top; ++k) v += to_f(eo[erow[k] + c]);
            if (gate) v *= sigmoidf_(to_f(gate[c]) + a.gate_bias[c]);
            const float xv = x[c] + v;
            x[c] = xv;
            row[c] = xv;
            if (xc) xc[c] = from_f<T>(xv);
        }
    }
    if (!a.w_next) return;
    __syncthreads();
    group_norm_store<T>(row, width, static_cast<int>(a.groups), a.eps, a.w_next, a.weight_offset, static_cast<T *>(a.h) + t * width, red,
                        inv_s);
}

template <typename T>
__global__ void __launch_bounds__(256) side_gate_kernel(const T *__restrict__ a, int64_t ld_a, const uint32_t *__restrict__ tokens,
                                                        const T *__restrict__ side, int64_t table_width, int64_t part,
                                                        T *__restrict__ out, int64_t total, int dim, int64_t vocab) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = i / dim;
        const int j = static_cast<int>(i % dim);
        int64_t tok = tokens[t];
        if (tok >= vocab) tok = vocab - 1;
        out[i] = from_f<T>(gelu_tanh(to_f(a[t * ld_a + j])) * to_f(side[tok * table_width + part * dim + j]));
    }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads) unitnorm_add_norm_kernel(const T *__restrict__ y, float *__restrict__ x,
                                                                        const float *__restrict__ w_unit,
                                                                        const float *__restrict__ w_next, T *__restrict__ h, int width,
                                                                        int groups, float eps, float offset) {
    extern __shared__ float row[];
    __shared__ float red[32], inv_s[kMaxNormGroups];
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
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = x[base + c] + row[c] * inv * w_unit[c];
        x[base + c] = v;
        row[c] = v;
    }
    if (!w_next) return;
    __syncthreads();
    group_norm_store<T>(row, width, groups, eps, w_next, offset, h + base, red, inv_s);
}

template <typename T>
__global__ void __launch_bounds__(256) glu_clamped_kernel(const T *__restrict__ gu, int64_t ld, const float *__restrict__ bias,
                                                          T *__restrict__ out, int64_t total, int ff, float limit, float alpha, float shift) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = i / ff;
        const int j = static_cast<int>(i % ff);
        float g = to_f(gu[t * ld + j]), u = to_f(gu[t * ld + ff + j]);
        if (bias) g += bias[j], u += bias[ff + j];
        out[i] = from_f<T>(glu_clamped(g, u, limit, alpha, shift));
    }
}

bool row_smem(size_t bytes, const char *what) {
    if (bytes > 200 * 1024) {
        set_status(kErrUnsupported, "%s: a row of %zu bytes does not fit shared memory", what, bytes);
        return false;
    }
    return true;
}

bool groups_ok(int64_t groups, int64_t width, const char *what) {
    if (groups >= 1 && groups <= kMaxNormGroups && width % groups == 0) return true;
    set_status(kErrInvalidArg, "%s: %lld norm groups do not divide a width of %lld (at most %d groups)", what,
               static_cast<long long>(groups), static_cast<long long>(width), kMaxNormGroups);
    return false;
}

unsigned flat_grid(int64_t total) { return static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((total + 255) / 256, 148 * 8))); }

}  // namespace

#define HYB_DISPATCH(dtype, CALL) ((dtype) == ATOMA_DTYPE_BF16 ? CALL(__nv_bfloat16) : CALL(float))
#define HYB_BIG_SMEM(kernel, smem)                                                                                      \
    if ((smem) > 48 * 1024) {                                                                                           \
        cudaFuncSetAttribute(kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
        cudaFuncSetAttribute(kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);                   \
    }

bool hyb_embed_learned(const uint32_t *tokens, const int64_t *positions, const void *table, const void *pos_table, float *out, int64_t T,
                       int64_t width, int64_t vocab, int64_t max_positions, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_embed_learned")) return false;
    if (!tokens || !positions || !table || !pos_table || !out || width <= 0 || vocab <= 0 || max_positions <= 0) {
        set_status(kErrInvalidArg, "atoma_embed_learned: null argument or empty table");
        return false;
    }
#define CALL(TT) launch_ex(embed_learned_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(128), 0, stream, tokens, positions, \
                           static_cast<const TT *>(table), static_cast<const TT *>(pos_table), out, static_cast<int>(width), vocab, max_positions)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "embed_learned_kernel");
#undef CALL
}

bool hyb_group_rmsnorm_rows(const float *x, const int32_t *rows, const float *weight, float offset, int64_t groups, void *out, int64_t R,
                            int64_t width, float eps, uint32_t dtype, cudaStream_t stream) {
    if (R <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_group_rmsnorm_rows")) return false;
    if (!x || !weight || !out || width <= 0) {
        set_status(kErrInvalidArg, "atoma_group_rmsnorm_rows: null argument");
        return false;
    }
    if (groups <= 0) groups = 1;
    const size_t smem = static_cast<size_t>(width) * 4;
    if (!groups_ok(groups, width, "atoma_group_rmsnorm_rows") || !row_smem(smem, "atoma_group_rmsnorm_rows")) return false;
    HYB_BIG_SMEM(group_rmsnorm_rows_kernel, smem)
#define CALL(TT) launch_ex(group_rmsnorm_rows_kernel<TT>, dim3(static_cast<unsigned>(R)), dim3(kRowThreads), smem, stream, x, rows, weight, \
                           offset, static_cast<int>(groups), static_cast<TT *>(out), static_cast<int>(width), eps)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "group_rmsnorm_rows_kernel");
#undef CALL
}

bool hyb_gated_residual_norm(const atoma_gated_residual_args &a_, cudaStream_t stream) {
    atoma_gated_residual_args a = a_;
    if (a.T <= 0) return true;
    if (!hybrid::known_dtype(a.dtype, "atoma_gated_residual_norm")) return false;
    if (a.groups <= 0) a.groups = 1;
    if (!a.x || a.width <= 0 || (!a.y && !a.expert_out) || (a.expert_out && (!a.pair_row || a.top <= 0 || a.top > kMaxTopRows)) || (a.gate && !a.gate_bias) ||
        (a.w_next && !a.h)) {
        set_status(kErrInvalidArg, "atoma_gated_residual_norm: null or inconsistent arguments");
        return false;
    }
    const size_t smem = static_cast<size_t>(a.width) * 4;
    if (!groups_ok(a.groups, a.width, "atoma_gated_residual_norm") || !row_smem(smem, "atoma_gated_residual_norm")) return false;
    HYB_BIG_SMEM(gated_residual_norm_kernel, smem)
#define CALL(TT) launch_ex(gated_residual_norm_kernel<TT>, dim3(static_cast<unsigned>(a.T)), dim3(kRowThreads), smem, stream, a)
    return hybrid::launched(HYB_DISPATCH(a.dtype, CALL), "gated_residual_norm_kernel");
#undef CALL
}

bool hyb_side_gate(const void *a, int64_t ld_a, const uint32_t *tokens, const void *side_table, int64_t table_width, int64_t part,
                   void *out, int64_t T, int64_t dim, int64_t vocab, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0 || dim <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_side_gate")) return false;
    if (!a || !tokens || !side_table || !out || part < 0 || (part + 1) * dim > table_width || vocab <= 0) {
        set_status(kErrInvalidArg, "atoma_side_gate: null argument, or part %lld of %lld columns is outside a table of %lld",
                   static_cast<long long>(part), static_cast<long long>(dim), static_cast<long long>(table_width));
        return false;
    }
    const int64_t total = T * dim;
#define CALL(TT) launch_ex(side_gate_kernel<TT>, dim3(flat_grid(total)), dim3(256), 0, stream, static_cast<const TT *>(a), ld_a, tokens, \
                           static_cast<const TT *>(side_table), table_width, part, static_cast<TT *>(out), total, static_cast<int>(dim), vocab)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "side_gate_kernel");
#undef CALL
}

bool hyb_unitnorm_add_norm(const void *y, float *x, const float *w_unit, const float *w_next, void *h, int64_t T, int64_t width,
                           int64_t groups, float eps, float offset, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_unitnorm_add_norm")) return false;
    if (!y || !x || !w_unit || (w_next && !h) || width <= 0) {
        set_status(kErrInvalidArg, "atoma_unitnorm_add_norm: null argument");
        return false;
    }
    if (groups <= 0) groups = 1;
    const size_t smem = static_cast<size_t>(width) * 4;
    if (!groups_ok(groups, width, "atoma_unitnorm_add_norm") || !row_smem(smem, "atoma_unitnorm_add_norm")) return false;
    HYB_BIG_SMEM(unitnorm_add_norm_kernel, smem)
#define CALL(TT) launch_ex(unitnorm_add_norm_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(kRowThreads), smem, stream, \
                           static_cast<const TT *>(y), x, w_unit, w_next, static_cast<TT *>(h), static_cast<int>(width), \
                           static_cast<int>(groups), eps, offset)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "unitnorm_add_norm_kernel");
#undef CALL
}

bool hyb_glu_clamped_bias(const void *gu, int64_t ld, const float *bias, void *out, int64_t T, int64_t ff, float limit, float alpha,
                          float up_shift, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0 || ff <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_glu_clamped")) return false;
    if (!gu || !out || ld < 2 * ff) {
        set_status(kErrInvalidArg, "atoma_glu_clamped: null argument or a row stride below 2 ff");
        return false;
    }
    const int64_t total = T * ff;
#define CALL(TT) launch_ex(glu_clamped_kernel<TT>, dim3(flat_grid(total)), dim3(256), 0, stream, static_cast<const TT *>(gu), ld, bias, \
                           static_cast<TT *>(out), total, static_cast<int>(ff), limit, alpha, up_shift)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "glu_clamped_kernel");
#undef CALL
}

bool hyb_glu_clamped(const void *gu, int64_t ld, void *out, int64_t T, int64_t ff, float limit, float alpha, float up_shift, uint32_t dtype,
                     cudaStream_t stream) {
    return hyb_glu_clamped_bias(gu, ld, nullptr, out, T, ff, limit, alpha, up_shift, dtype, stream);
}

}  // namespace atoma

using namespace atoma;

extern "C" void atoma_embed_learned(const uint32_t *tokens, const int64_t *positions, const void *table, const void *pos_table, float *out,
                                    int64_t T, int64_t width, int64_t vocab, int64_t max_positions, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_embed_learned(tokens, positions, table, pos_table, out, T, width, vocab, max_positions, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_group_rmsnorm_rows(const float *x, const int32_t *rows, const float *weight, float weight_offset, int64_t groups,
                                         void *out, int64_t R, int64_t width, float eps, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_group_rmsnorm_rows(x, rows, weight, weight_offset, groups, out, R, width, eps, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_gated_residual_norm(const atoma_gated_residual_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_gated_residual_norm: args is NULL");
        return;
    }
    hyb_gated_residual_norm(*args, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_side_gate(const void *a, int64_t ld_a, const uint32_t *tokens, const void *side_table, int64_t table_width,
                                int64_t part, void *out, int64_t T, int64_t dim, int64_t vocab, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_side_gate(a, ld_a, tokens, side_table, table_width, part, out, T, dim, vocab, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_unitnorm_add_norm(const void *y, float *x, const float *w_unit, const float *w_next, void *h, int64_t T, int64_t width,
                                        int64_t groups, float eps, float weight_offset, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_unitnorm_add_norm(y, x, w_unit, w_next, h, T, width, groups, eps, weight_offset, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_glu_clamped(const void *gu, int64_t ld, void *out, int64_t T, int64_t ff, float limit, float alpha, float up_shift,
                                  uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_glu_clamped(gu, ld, out, T, ff, limit, alpha, up_shift, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_glu_clamped_bias(const void *gu, int64_t ld, const float *bias, void *out, int64_t T, int64_t ff, float limit,
                                       float alpha, float up_shift, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_glu_clamped_bias(gu, ld, bias, out, T, ff, limit, alpha, up_shift, dtype, static_cast<cudaStream_t>(stream));
}
