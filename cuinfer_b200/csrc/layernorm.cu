// Layer norm with gain and bias around a 32-bit residual stream, for layers that norm a sub-layer's input AND its
// output ("sandwich" layers): x <- x + post(sub(pre(x))).
//
// One pass over a row does, each part optional:
//   x = residual
//   x += post(y)          y: a sub-layer's output; post(y) = (y - mean(y)) / sqrt(var(y) + eps) * g + b,
//                         or x += y when no gain is given (a plain delta)
//   x += extra            a second 32-bit row to add (a model that feeds its embedding output in again)
//   residual = x          (when anything was added)
//   out = pre(x)          the next sub-layer's input, rounded once to the output type
// so the output norm of one sub-layer, the residual sum and the input norm of the next are one kernel and one trip
// through memory.  Mean, variance (mean of squared deviations, two passes over the row in shared memory), the
// normalisation and the sums are 32-bit.  A block per row; the row lives in shared memory.
#include "common.cuh"

namespace cib {

// V values at a time (V = 4 when the row length is a multiple of four: 16-byte loads of 32-bit rows, 8-byte loads of
// bfloat16 rows; else 1).
template <typename T, int V> struct Pack;
template <> struct Pack<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Pack<__nv_bfloat16, 4> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<const uint32_t*>(&a);
        t.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = t;
    }
};
template <typename T> struct Pack<T, 1> {
    static __device__ __forceinline__ void load(const T* p, float* v) { v[0] = to_f32(*p); }
    static __device__ __forceinline__ void store(T* p, const float* v) { *p = from_f32<T>(v[0]); }
};

template <typename TY, typename TO, int V>
__global__ void sandwich_layernorm_kernel(float* __restrict__ residual, const TY* __restrict__ y, AnyVec post_g,
                                          AnyVec post_b, float post_eps, const float* __restrict__ extra,
                                          AnyVec pre_g, AnyVec pre_b, float pre_eps, TO* __restrict__ out, int hidden) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float scratch[33];
    const size_t row = (size_t)blockIdx.x * hidden;
    float* res = residual + row;
    const float inv_n = 1.f / (float)hidden;
    const int first = threadIdx.x * V, step = blockDim.x * V;

    if (y && post_g.ptr) {
        float s = 0.f;
        for (int i = first; i < hidden; i += step) {
            float v[V];
            Pack<TY, V>::load(y + row + i, v);
#pragma unroll
            for (int k = 0; k < V; ++k) { row_s[i + k] = v[k]; s += v[k]; }
        }
        const float mean = block_sum(s, scratch) * inv_n;
        float q = 0.f;
        for (int i = first; i < hidden; i += step) {
#pragma unroll
            for (int k = 0; k < V; ++k) { const float d = row_s[i + k] - mean; q += d * d; }
        }
        const float rstd = 1.f / sqrtf(block_sum(q, scratch) * inv_n + post_eps);
        for (int i = first; i < hidden; i += step) {
            float x[V], e[V];
            Pack<float, V>::load(res + i, x);
            if (extra) Pack<float, V>::load(extra + row + i, e);
#pragma unroll
            for (int k = 0; k < V; ++k) {
                x[k] += (row_s[i + k] - mean) * rstd * post_g[i + k] + post_b[i + k];
                if (extra) x[k] += e[k];
                row_s[i + k] = x[k];
            }
            Pack<float, V>::store(res + i, x);
        }
    } else {
        for (int i = first; i < hidden; i += step) {
            float x[V], d[V];
            Pack<float, V>::load(res + i, x);
            if (y) {
                Pack<TY, V>::load(y + row + i, d);
#pragma unroll
                for (int k = 0; k < V; ++k) x[k] += d[k];
            }
            if (extra) {
                Pack<float, V>::load(extra + row + i, d);
#pragma unroll
                for (int k = 0; k < V; ++k) x[k] += d[k];
            }
            if (y || extra) Pack<float, V>::store(res + i, x);
#pragma unroll
            for (int k = 0; k < V; ++k) row_s[i + k] = x[k];
        }
    }
    if (!out) return;
    float s = 0.f;
    for (int i = first; i < hidden; i += step) {          // each thread reads what it wrote
#pragma unroll
        for (int k = 0; k < V; ++k) s += row_s[i + k];
    }
    const float mean = block_sum(s, scratch) * inv_n;
    float q = 0.f;
    for (int i = first; i < hidden; i += step) {
#pragma unroll
        for (int k = 0; k < V; ++k) { const float d = row_s[i + k] - mean; q += d * d; }
    }
    const float rstd = 1.f / sqrtf(block_sum(q, scratch) * inv_n + pre_eps);
    for (int i = first; i < hidden; i += step) {
        float o[V];
#pragma unroll
        for (int k = 0; k < V; ++k) o[k] = (row_s[i + k] - mean) * rstd * pre_g[i + k] + pre_b[i + k];
        Pack<TO, V>::store(out + row + i, o);
    }
}

template <typename TY, typename TO>
static int launch_sandwich(float* residual, const void* y, AnyVec pg, AnyVec pb, float peps, const float* extra, AnyVec g,
                           AnyVec b, float eps, void* out, int rows, int hidden, cudaStream_t stream) {
    static SmemLimit limit4, limit1;
    const size_t smem = (size_t)hidden * sizeof(float);
    int threads = 64;
    while (threads < hidden / 8 && threads < 512) threads <<= 1;
    if (hidden % 4 == 0) {
        if (smem > 48 * 1024 && raise_smem_limit(limit4, sandwich_layernorm_kernel<TY, TO, 4>, 200 * 1024, "layernorm") != 0) return -2;
        sandwich_layernorm_kernel<TY, TO, 4><<<rows, threads, smem, stream>>>(residual, (const TY*)y, pg, pb, peps, extra, g, b, eps,
                                                                               (TO*)out, hidden);
    } else {
        if (smem > 48 * 1024 && raise_smem_limit(limit1, sandwich_layernorm_kernel<TY, TO, 1>, 200 * 1024, "layernorm") != 0) return -2;
        sandwich_layernorm_kernel<TY, TO, 1><<<rows, threads, smem, stream>>>(residual, (const TY*)y, pg, pb, peps, extra, g, b, eps,
                                                                               (TO*)out, hidden);
    }
    return 0;
}

}  // namespace cib

using namespace cib;

// y, post gain/bias, extra, out may each be null (see the head of this file).  Gains and biases are bf16 or f32
// (`vec_dtype`, one for all four).
extern "C" int cib_sandwich_layernorm(float* residual, const void* y, int y_dtype, const void* post_gain,
                                      const void* post_bias, float post_eps, const float* extra, const void* gain,
                                      const void* bias, float eps, int vec_dtype, void* out, int out_dtype, int rows,
                                      int hidden, cudaStream_t stream) {
    CIB_REQUIRE(rows >= 0 && hidden > 0, "layernorm: bad sizes rows=%d hidden=%d", rows, hidden);
    CIB_REQUIRE(hidden <= 50 * 1024, "layernorm: rows of %d values do not fit shared memory", hidden);
    CIB_REQUIRE(out == nullptr || (gain != nullptr && bias != nullptr), "layernorm: a norm needs its gain and bias");
    CIB_REQUIRE((post_gain == nullptr) == (post_bias == nullptr), "layernorm: the output norm needs gain and bias");
    CIB_REQUIRE(post_gain == nullptr || y != nullptr, "layernorm: an output norm without rows to norm");
    if (rows == 0) return 0;
    const int is_bf16 = vec_dtype == kBF16;
    AnyVec pg{post_gain, is_bf16}, pb{post_bias, is_bf16}, g{gain, is_bf16}, b{bias, is_bf16};
    const int yd = y ? y_dtype : kF32, od = out ? out_dtype : kF32;
    int rc;
    if (yd == kF32 && od == kF32) rc = launch_sandwich<float, float>(residual, y, pg, pb, post_eps, extra, g, b, eps, out, rows, hidden, stream);
    else if (yd == kF32 && od == kBF16) rc = launch_sandwich<float, __nv_bfloat16>(residual, y, pg, pb, post_eps, extra, g, b, eps, out, rows, hidden, stream);
    else if (yd == kBF16 && od == kF32) rc = launch_sandwich<__nv_bfloat16, float>(residual, y, pg, pb, post_eps, extra, g, b, eps, out, rows, hidden, stream);
    else if (yd == kBF16 && od == kBF16) rc = launch_sandwich<__nv_bfloat16, __nv_bfloat16>(residual, y, pg, pb, post_eps, extra, g, b, eps, out, rows, hidden, stream);
    else CIB_REQUIRE(false, "layernorm: unsupported dtypes y=%d out=%d", y_dtype, out_dtype);
    if (rc != 0) return rc;
    CIB_LAUNCH_CHECK("sandwich_layernorm");
    return 0;
}
