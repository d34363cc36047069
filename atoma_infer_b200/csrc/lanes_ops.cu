// Row-wise operators of decoder layers that keep several residual LANES — include/atoma_hybrid.h.
//
// The residual stream exists `lanes` times, x [T, lanes, width] float32 (a token's lanes are contiguous, so one CTA
// owns everything a token needs).  A sublayer reads u = sum_s w_in[s] x_s, and its result y goes back as
// x'_t = sum_s w_mix[s, t] x_s + w_out[t] y for all lanes at once.  The write-back is fused with the next sublayer's read
// and RMS norm (the lanes are touched once per sublayer), adds the feed-forward's output bias, the rows of the token's
// routed experts and what its identity experts hand through, and can emit the plain sum of the lanes.
// Also here: the scaled embedding into all lanes, and the per-head q/k RMS norm with the cache write (values may be the
// un-normed key projections).  Statistics, lane arithmetic and sums are float32 whatever the activation format; every
// row is reduced in an order that depends on the row alone.
#include "common.cuh"
#include "hybrid_common.cuh"

#include "atoma_hybrid.h"

#include <algorithm>

namespace atoma {
namespace {

using namespace hybrid;

constexpr int kMaxLanes = 16;
constexpr int kMaxTop = 64;   // router choices per token

template <typename T>
__global__ void __launch_bounds__(128) embed_scaled_lanes_kernel(const uint32_t *__restrict__ tokens, const T *__restrict__ table,
                                                                 float scale, float *__restrict__ x, int lanes, int width, int64_t vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t t = blockIdx.x;
    int64_t tok = tokens[t];
    if (tok >= vocab) tok = vocab - 1;
    const T *e = table + tok * width;
    float *o = x + t * lanes * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = to_f(e[c]) * scale;
        for (int s = 0; s < lanes; ++s) o[s * width + c] = v;
    }
}

// row [width] float32 in shared memory -> out = row / sqrt(mean(row^2) + eps) * (offset + w).  Every thread must call it.
template <typename T>
__device__ __forceinline__ void norm_store(const float *row, int width, float eps, const float *__restrict__ w, float offset,
                                           T *__restrict__ out, float *red) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(width) + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[c] = from_f<T>(row[c] * inv * (offset + w[c]));
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads) lanes_read_norm_kernel(const float *__restrict__ x, const float *__restrict__ w_in,
                                                                      const int32_t *__restrict__ rows, const float *__restrict__ weight,
                                                                      float offset, T *__restrict__ out, float *__restrict__ sum_out,
                                                                      int lanes, int width, float eps) {
    extern __shared__ float row[];
    __shared__ float red[32], win_s[kMaxLanes];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t r = blockIdx.x;
    const float *xr = x + static_cast<int64_t>(rows ? rows[r] : r) * lanes * width;
    if (threadIdx.x < lanes) win_s[threadIdx.x] = w_in ? w_in[threadIdx.x] : 1.f;
    __syncthreads();
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float u = 0.f;
        for (int s = 0; s < lanes; ++s) u = fmaf(win_s[s], xr[s * width + c], u);
        row[c] = u;
        if (sum_out) sum_out[r * width + c] = u;
    }
    __syncthreads();
    norm_store<T>(row, width, eps, weight, offset, out + r * width, red);
}

// Four consecutive elements at once (8 bytes of bfloat16, 16 of float32); the caller has checked the alignment.
__device__ __forceinline__ float4 load4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16 *p) {
    const uint2 v = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

// LC = the number of lanes at compile time (the loops over lanes unroll into registers); LC = 0 takes any number up to
// kMaxLanes at run time.  VEC = four channels per thread and step (the host checks widths and alignments).
template <typename T, int LC, bool VEC>
__global__ void __launch_bounds__(kRowThreads) lanes_update_norm_kernel(const atoma_lanes_update_args a) {
    extern __shared__ float row[];
    __shared__ float red[32], mix_s[kMaxLanes * kMaxLanes], out_s[kMaxLanes], in_s[kMaxLanes], tw_s[kMaxTop];
    __shared__ int64_t erow[kMaxTop];   // >= 0: offset of the pair's expert row; -1: identity expert; -2: nothing
    pdl_launch_dependents();
    pdl_wait();
    constexpr int LM = LC > 0 ? LC : kMaxLanes;
    const int64_t t = blockIdx.x;
    const int width = static_cast<int>(a.width), lanes = LC > 0 ? LC : static_cast<int>(a.lanes), top = a.top_expert ? static_cast<int>(a.top) : 0;
    for (int i = threadIdx.x; i < lanes * lanes; i += blockDim.x) mix_s[i] = a.w_mix[i];
    for (int i = threadIdx.x; i < lanes; i += blockDim.x) {
        out_s[i] = a.w_out[i];
        in_s[i] = a.w_in_next ? a.w_in_next[i] : 1.f;
    }
    for (int k = threadIdx.x; k < top; k += blockDim.x) {
        const int e = a.top_expert[t * top + k];
        tw_s[k] = a.top_weight ? a.top_weight[t * top + k] : 0.f;
        erow[k] = e < 0 ? -2 : (e >= a.experts ? -1 : static_cast<int64_t>(a.pair_row[t * top + k]) * width);
    }
    __syncthreads();
    const T *y = a.y ? static_cast<const T *>(a.y) + t * width : nullptr;
    const T *eo = static_cast<const T *>(a.expert_out);
    const T *hin = a.h_in ? static_cast<const T *>(a.h_in) + t * width : nullptr;
    float *x = a.x + t * lanes * width;
    float *ls = a.lane_sum ? a.lane_sum + t * width : nullptr;
    constexpr int C = VEC ? 4 : 1;
    for (int c = C * threadIdx.x; c < width; c += C * blockDim.x) {
        float v[C];
        if constexpr (VEC) {
            float4 v4 = y ? load4(y + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (a.y_bias) {
                const float4 b4 = load4(a.y_bias + c);
                v4.x += b4.x, v4.y += b4.y, v4.z += b4.z, v4.w += b4.w;
            }
            for (int k = 0; k < top; ++k) {
                if (erow[k] >= 0) {
                    const float4 e4 = load4(eo + erow[k] + c);
                    v4.x += e4.x, v4.y += e4.y, v4.z += e4.z, v4.w += e4.w;
                } else if (erow[k] == -1 && hin) {
                    const float4 h4 = load4(hin + c);
                    v4.x = fmaf(tw_s[k], h4.x, v4.x), v4.y = fmaf(tw_s[k], h4.y, v4.y), v4.z = fmaf(tw_s[k], h4.z, v4.z), v4.w = fmaf(tw_s[k], h4.w, v4.w);
                }
            }
            v[0] = v4.x, v[1] = v4.y, v[2] = v4.z, v[3] = v4.w;
        } else {
            v[0] = y ? to_f(y[c]) : 0.f;
            if (a.y_bias) v[0] += a.y_bias[c];
            for (int k = 0; k < top; ++k) {
                if (erow[k] >= 0) v[0] += to_f(eo[erow[k] + c]);
                else if (erow[k] == -1 && hin) v[0] = fmaf(tw_s[k], to_f(hin[c]), v[0]);
            }
        }
        float old[LM][C];
#pragma unroll
        for (int s = 0; s < LM; ++s) {
            if (s < lanes) {
                if constexpr (VEC) {
                    const float4 o4 = load4(x + s * width + c);
                    old[s][0] = o4.x, old[s][1] = o4.y, old[s][2] = o4.z, old[s][3] = o4.w;
                } else {
                    old[s][0] = x[s * width + c];
                }
            }
        }
        float u[C], total[C];
#pragma unroll
        for (int i = 0; i < C; ++i) u[i] = total[i] = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < LM; ++s2) {
            if (s2 < lanes) {
                float nv[C];
#pragma unroll
                for (int i = 0; i < C; ++i) nv[i] = 0.f;
#pragma unroll
                for (int s = 0; s < LM; ++s) {
                    if (s < lanes) {
                        const float m = mix_s[s * lanes + s2];
#pragma unroll
                        for (int i = 0; i < C; ++i) nv[i] = fmaf(m, old[s][i], nv[i]);
                    }
                }
#pragma unroll
                for (int i = 0; i < C; ++i) {
                    nv[i] = fmaf(out_s[s2], v[i], nv[i]);
                    u[i] = fmaf(in_s[s2], nv[i], u[i]);
                    total[i] += nv[i];
                }
                if constexpr (VEC) *reinterpret_cast<float4 *>(x + s2 * width + c) = make_float4(nv[0], nv[1], nv[2], nv[3]);
                else x[s2 * width + c] = nv[0];
            }
        }
#pragma unroll
        for (int i = 0; i < C; ++i) row[c + i] = u[i];
        if (ls) {
            if constexpr (VEC) *reinterpret_cast<float4 *>(ls + c) = make_float4(total[0], total[1], total[2], total[3]);
            else ls[c] = total[0];
        }
    }
    if (!a.w_next) return;
    __syncthreads();   // every channel of h_in has been read before h (possibly the same buffer) is written
    norm_store<T>(row, width, a.eps, a.w_next, a.weight_offset, static_cast<T *>(a.h) + t * width, red);
}

// One CTA per token, its warps take the heads in turn: heads 0 .. H - 1 are queries, H .. H + G - 1 keys (whose raw or
// separate values ride along).
template <typename T>
__global__ void __launch_bounds__(256) qk_headnorm_cache_kernel(const T *__restrict__ proj, int64_t ld, int q_off, int k_off, int v_off,
                                                                const float *__restrict__ q_w, const float *__restrict__ k_w, float offset,
                                                                const int64_t *__restrict__ slots, T *__restrict__ q_out,
                                                                T *__restrict__ k_cache, T *__restrict__ v_cache, int H, int G, int dim,
                                                                int vdim, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int64_t t = blockIdx.x;
    const int64_t slot = slots ? slots[t] : -1;
    for (int hd = warp; hd < H + G; hd += nwarp) {
        const bool is_q = hd < H;
        const int g = hd - H;
        if (!is_q && slot < 0) continue;
        const T *src = proj + t * ld + (is_q ? q_off + hd * dim : k_off + g * dim);
        float ss = 0.f;
        for (int c = lane; c < dim; c += 32) {
            const float v = to_f(src[c]);
            ss = fmaf(v, v, ss);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
        if (is_q) {
            T *dst = q_out + (t * H + hd) * dim;
            for (int c = lane; c < dim; c += 32) dst[c] = from_f<T>(to_f(src[c]) * inv * (offset + q_w[c]));
            continue;
        }
        T *kd = k_cache + (slot * G + g) * dim;
        for (int c = lane; c < dim; c += 32) kd[c] = from_f<T>(to_f(src[c]) * inv * (offset + k_w[c]));
        const T *vs = proj + t * ld + v_off + g * vdim;
        T *vd = v_cache + (slot * G + g) * vdim;
        for (int c = lane; c < vdim; c += 32) vd[c] = vs[c];
    }
}

bool row_fits(size_t bytes, const char *what) {
    if (bytes > 200 * 1024) {
        set_status(kErrUnsupported, "%s: a row of %zu bytes does not fit shared memory", what, bytes);
        return false;
    }
    return true;
}

}  // namespace

#define HYB_DISPATCH(dtype, CALL) ((dtype) == ATOMA_DTYPE_BF16 ? CALL(__nv_bfloat16) : CALL(float))
#define HYB_BIG_SMEM(kernel, smem)                                                                                      \
    if ((smem) > 48 * 1024) {                                                                                           \
        cudaFuncSetAttribute(kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);           \
        cudaFuncSetAttribute(kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);                   \
    }

bool hyb_embed_scaled_lanes(const uint32_t *tokens, const void *table, float scale, float *x, int64_t T, int64_t lanes, int64_t width,
                            int64_t vocab, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_embed_scaled_lanes")) return false;
    if (!tokens || !table || !x || lanes <= 0 || width <= 0 || vocab <= 0) {
        set_status(kErrInvalidArg, "atoma_embed_scaled_lanes: null argument or empty shape");
        return false;
    }
#define CALL(TT) launch_ex(embed_scaled_lanes_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(128), 0, stream, tokens, \
                           static_cast<const TT *>(table), scale, x, static_cast<int>(lanes), static_cast<int>(width), vocab)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "embed_scaled_lanes_kernel");
#undef CALL
}

bool hyb_lanes_read_norm(const float *x, const float *w_in, const int32_t *rows, const float *weight, float offset, void *out,
                         float *sum_out, int64_t R, int64_t lanes, int64_t width, float eps, uint32_t dtype, cudaStream_t stream) {
    if (R <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_lanes_read_norm")) return false;
    if (!x || !weight || !out || width <= 0 || lanes <= 0 || lanes > kMaxLanes) {
        set_status(kErrInvalidArg, "atoma_lanes_read_norm: null argument, or %lld lanes (at most %d)", static_cast<long long>(lanes), kMaxLanes);
        return false;
    }
    const size_t smem = static_cast<size_t>(width) * 4;
    if (!row_fits(smem, "atoma_lanes_read_norm")) return false;
    HYB_BIG_SMEM(lanes_read_norm_kernel, smem)
#define CALL(TT) launch_ex(lanes_read_norm_kernel<TT>, dim3(static_cast<unsigned>(R)), dim3(kRowThreads), smem, stream, x, w_in, rows, weight, \
                           offset, static_cast<TT *>(out), sum_out, static_cast<int>(lanes), static_cast<int>(width), eps)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "lanes_read_norm_kernel");
#undef CALL
}

bool hyb_lanes_update_norm(const atoma_lanes_update_args &a, cudaStream_t stream) {
    if (a.T <= 0) return true;
    if (!hybrid::known_dtype(a.dtype, "atoma_lanes_update_norm")) return false;
    if (!a.x || !a.w_mix || !a.w_out || a.width <= 0 || a.lanes <= 0 || a.lanes > kMaxLanes || (a.w_next && !a.h) ||
        (a.top_expert && (a.top <= 0 || a.top > kMaxTop || !a.top_weight || (a.expert_out && !a.pair_row)))) {
        set_status(kErrInvalidArg, "atoma_lanes_update_norm: null or inconsistent arguments (at most %d lanes, %d choices per token)", kMaxLanes,
                   kMaxTop);
        return false;
    }
    const size_t smem = static_cast<size_t>(a.width) * 4;
    if (!row_fits(smem, "atoma_lanes_update_norm")) return false;
    auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool specialised = a.lanes <= 4 || a.lanes == 6 || a.lanes == 8;   // other counts: run-time loops, one channel per thread
    const bool vec = specialised && a.width % 4 == 0 && al(a.x) && al(a.y) && al(a.y_bias) && al(a.expert_out) && al(a.h_in) && al(a.lane_sum);
    cudaError_t e;
#define LANES_CASE(TT, LC)                                                                                                              \
    {                                                                                                                                   \
        if (smem > 48 * 1024) {                                                                                                         \
            cudaFuncSetAttribute(lanes_update_norm_kernel<TT, LC, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);      \
            cudaFuncSetAttribute(lanes_update_norm_kernel<TT, LC, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);     \
        }                                                                                                                               \
        e = vec ? launch_ex(lanes_update_norm_kernel<TT, LC, true>, dim3(static_cast<unsigned>(a.T)), dim3(kRowThreads), smem, stream, a) \
                : launch_ex(lanes_update_norm_kernel<TT, LC, false>, dim3(static_cast<unsigned>(a.T)), dim3(kRowThreads), smem, stream, a); \
    }
#define LANES_SWITCH(TT)                     \
    switch (a.lanes) {                       \
        case 1: LANES_CASE(TT, 1) break;     \
        case 2: LANES_CASE(TT, 2) break;     \
        case 3: LANES_CASE(TT, 3) break;     \
        case 4: LANES_CASE(TT, 4) break;     \
        case 6: LANES_CASE(TT, 6) break;     \
        case 8: LANES_CASE(TT, 8) break;     \
        default: LANES_CASE(TT, 0) break;    \
    }
    if (a.dtype == ATOMA_DTYPE_BF16) LANES_SWITCH(__nv_bfloat16) else LANES_SWITCH(float)
#undef LANES_SWITCH
#undef LANES_CASE
    return hybrid::launched(e, "lanes_update_norm_kernel");
}

bool hyb_qk_headnorm_cache(const void *proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off, const float *q_w, const float *k_w,
                           float offset, const int64_t *slots, void *q_out, void *k_cache, void *v_cache, int64_t T, int64_t H, int64_t G,
                           int64_t dim, int64_t vdim, float eps, uint32_t dtype, cudaStream_t stream) {
    if (T <= 0) return true;
    if (!hybrid::known_dtype(dtype, "atoma_qk_headnorm_cache")) return false;
    if (!proj || !q_w || !k_w || !q_out || H <= 0 || G <= 0 || H % G || dim <= 0 || vdim <= 0 || (slots && (!k_cache || !v_cache)) ||
        q_off < 0 || k_off < 0 || v_off < 0 || q_off + H * dim > ld || k_off + G * dim > ld || v_off + G * vdim > ld) {
        set_status(kErrInvalidArg, "atoma_qk_headnorm_cache: null argument, kv heads (%lld) that do not divide heads (%lld), or columns outside the row",
                   static_cast<long long>(G), static_cast<long long>(H));
        return false;
    }
    const unsigned threads = static_cast<unsigned>(std::min<int64_t>(8, H + G) * 32);
#define CALL(TT) launch_ex(qk_headnorm_cache_kernel<TT>, dim3(static_cast<unsigned>(T)), dim3(threads), 0, stream, \
                           static_cast<const TT *>(proj), ld, static_cast<int>(q_off), static_cast<int>(k_off), static_cast<int>(v_off), q_w, k_w, \
                           offset, slots, static_cast<TT *>(q_out), static_cast<TT *>(k_cache), static_cast<TT *>(v_cache), \
                           static_cast<int>(H), static_cast<int>(G), static_cast<int>(dim), static_cast<int>(vdim), eps)
    return hybrid::launched(HYB_DISPATCH(dtype, CALL), "qk_headnorm_cache_kernel");
#undef CALL
}

}  // namespace atoma

using namespace atoma;

extern "C" void atoma_embed_scaled_lanes(const uint32_t *tokens, const void *table, float scale, float *x, int64_t T, int64_t lanes,
                                         int64_t width, int64_t vocab, uint32_t dtype, atoma_stream_t stream) {
    clear_status();
    hyb_embed_scaled_lanes(tokens, table, scale, x, T, lanes, width, vocab, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_lanes_read_norm(const float *x, const float *w_in, const int32_t *rows, const float *weight, float weight_offset,
                                      void *out, float *sum_out, int64_t R, int64_t lanes, int64_t width, float eps, uint32_t dtype,
                                      atoma_stream_t stream) {
    clear_status();
    hyb_lanes_read_norm(x, w_in, rows, weight, weight_offset, out, sum_out, R, lanes, width, eps, dtype, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_lanes_update_norm(const atoma_lanes_update_args *args, atoma_stream_t stream) {
    clear_status();
    if (!args) {
        set_status(kErrInvalidArg, "atoma_lanes_update_norm: args is NULL");
        return;
    }
    hyb_lanes_update_norm(*args, static_cast<cudaStream_t>(stream));
}
extern "C" void atoma_qk_headnorm_cache(const void *proj, int64_t ld, int64_t q_off, int64_t k_off, int64_t v_off, const float *q_weight,
                                        const float *k_weight, float weight_offset, const int64_t *slot_mapping, void *q_out, void *k_cache,
                                        void *v_cache, int64_t T, int64_t H, int64_t G, int64_t dim, int64_t vdim, float eps, uint32_t dtype,
                                        atoma_stream_t stream) {
    clear_status();
    hyb_qk_headnorm_cache(proj, ld, q_off, k_off, v_off, q_weight, k_weight, weight_offset, slot_mapping, q_out, k_cache, v_cache, T, H, G,
                          dim, vdim, eps, dtype, static_cast<cudaStream_t>(stream));
}
