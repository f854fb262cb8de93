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

template <typename TY, typename TO>
__global__ void sandwich_layernorm_kernel(float* __restrict__ residual, const TY* __restrict__ y, AnyVec post_g,
                                          AnyVec post_b, float post_eps, const float* __restrict__ extra,
                                          AnyVec pre_g, AnyVec pre_b, float pre_eps, TO* __restrict__ out, int hidden) {
    extern __shared__ float row_s[];
    __shared__ float scratch[33];
    const size_t row = (size_t)blockIdx.x * hidden;
    float* res = residual + row;
    const float inv_n = 1.f / (float)hidden;

    if (y && post_g.ptr) {
        float s = 0.f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float v = to_f32(y[row + i]);
            row_s[i] = v;
            s += v;
        }
        const float mean = block_sum(s, scratch) * inv_n;
        float q = 0.f;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float d = row_s[i] - mean;
            q += d * d;
        }
        const float rstd = 1.f / sqrtf(block_sum(q, scratch) * inv_n + post_eps);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float x = res[i] + ((row_s[i] - mean) * rstd * post_g[i] + post_b[i]);
            if (extra) x += extra[row + i];
            res[i] = x;
            row_s[i] = x;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float x = res[i];
            if (y) x += to_f32(y[row + i]);
            if (extra) x += extra[row + i];
            if (y || extra) res[i] = x;
            row_s[i] = x;
        }
    }
    if (!out) return;
    float s = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) s += row_s[i];      // each thread reads what it wrote
    const float mean = block_sum(s, scratch) * inv_n;
    float q = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_s[i] - mean;
        q += d * d;
    }
    const float rstd = 1.f / sqrtf(block_sum(q, scratch) * inv_n + pre_eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        out[row + i] = from_f32<TO>((row_s[i] - mean) * rstd * pre_g[i] + pre_b[i]);
}

template <typename TY, typename TO>
static int launch_sandwich(float* residual, const void* y, AnyVec pg, AnyVec pb, float peps, const float* extra, AnyVec g,
                           AnyVec b, float eps, void* out, int rows, int hidden, cudaStream_t stream) {
    static SmemLimit limit;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 48 * 1024) {
        if (raise_smem_limit(limit, sandwich_layernorm_kernel<TY, TO>, 200 * 1024, "layernorm") != 0) return -2;
    }
    int threads = 64;
    while (threads < hidden / 4 && threads < 512) threads <<= 1;
    sandwich_layernorm_kernel<TY, TO><<<rows, threads, smem, stream>>>(residual, (const TY*)y, pg, pb, peps, extra, g, b, eps,
                                                                        (TO*)out, hidden);
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
