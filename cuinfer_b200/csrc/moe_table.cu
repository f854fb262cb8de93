// Mixture of gated experts whose choice is a table lookup: expert_table[token id][0..top-1] names the experts of a
// token, each with the same weight.  An expert is down_e( silu(gate_e h) * (up_e h) ), no biases.
//
// The simple kernels: every (token, choice) streams its expert's rows — a matrix-vector product per token, which is
// what a decode step needs (a token's experts are read once) and the 32-bit path.  Two launches:
//   gate_up : act[t, k, j] = silu(Wg[e][j, :] . h_t) * (Wu[e][j, :] . h_t),  e = table[ids[t], k]
//   down    : out[t, i]    = base[t, i] + weight * sum_k Wd[e_k][i, :] . act[t, k, :]
// Dots and the gate are 32-bit with the exact exponential; act and out are rounded once to the rows' type.
// Weights: gate_up [E][2 ff][W] (gate rows, then up rows), down [E][W][ff].  A table entry outside 0..E-1 contributes
// nothing.  `base` (another feed-forward's output, a shared expert's say) may be null.
#include "common.cuh"

namespace cib {

constexpr int kMoeWarps = 8;
constexpr int kMoeOutsPerBlock = 64;

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* __restrict__ x, int n, int lane) {
    float s = 0.f;
    for (int i = lane; i < n; i += 32) s = fmaf(to_f32(w[i]), x[i], s);
    return warp_sum(s);
}

template <typename T>
__global__ void __launch_bounds__(kMoeWarps * 32)
moe_table_gate_up_kernel(const T* __restrict__ h, int h_stride, const int* __restrict__ ids,
                         const int* __restrict__ table, int vocab, int top, int experts,
                         const T* __restrict__ gate_up, T* __restrict__ act, int width, int ff) {
    extern __shared__ float hs[];
    const int t = blockIdx.x / top, k = blockIdx.x % top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < width; i += blockDim.x) hs[i] = to_f32(h[(size_t)t * h_stride + i]);
    __syncthreads();
    const int id = ids[t];
    const int e = (id >= 0 && id < vocab) ? table[(size_t)id * top + k] : -1;
    const bool ok = e >= 0 && e < experts;
    const T* wg = gate_up + (size_t)(ok ? e : 0) * 2 * ff * width;
    const T* wu = wg + (size_t)ff * width;
    const int j0 = blockIdx.y * kMoeOutsPerBlock;
    for (int j = j0 + warp; j < min(ff, j0 + kMoeOutsPerBlock); j += kMoeWarps) {
        float v = 0.f;
        if (ok) {
            const float g = dot_row(wg + (size_t)j * width, hs, width, lane);
            const float u = dot_row(wu + (size_t)j * width, hs, width, lane);
            v = g / (1.f + expf(-g)) * u;
        }
        if (lane == 0) act[((size_t)t * top + k) * ff + j] = from_f32<T>(v);
    }
}

template <typename T>
__global__ void __launch_bounds__(kMoeWarps * 32)
moe_table_down_kernel(const T* __restrict__ act, const int* __restrict__ ids, const int* __restrict__ table, int vocab,
                      int top, int experts, const T* __restrict__ down, const T* __restrict__ base, int base_stride,
                      float weight, T* __restrict__ out, int width, int ff) {
    extern __shared__ float as[];                       // [top][ff]
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) as[i] = to_f32(act[(size_t)t * top * ff + i]);
    __syncthreads();
    const int id = ids[t];
    const bool id_ok = id >= 0 && id < vocab;
    const int i0 = blockIdx.y * kMoeOutsPerBlock;
    for (int i = i0 + warp; i < min(width, i0 + kMoeOutsPerBlock); i += kMoeWarps) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            const int e = id_ok ? table[(size_t)id * top + k] : -1;
            if (e < 0 || e >= experts) continue;
            sum += dot_row(down + ((size_t)e * width + i) * ff, as + k * ff, ff, lane);
        }
        if (lane == 0) {
            float v = sum * weight;
            if (base) v += to_f32(base[(size_t)t * base_stride + i]);
            out[(size_t)t * width + i] = from_f32<T>(v);
        }
    }
}

}  // namespace cib

using namespace cib;

extern "C" int cib_moe_table_gate_up(const void* h, int h_stride, int dtype, const int* ids, const int* table, int vocab,
                                     int top, int experts, const void* gate_up, void* act, int num_tokens, int width,
                                     int ff, cudaStream_t stream) {
    CIB_REQUIRE(num_tokens >= 0 && top > 0 && experts > 0 && width > 0 && ff > 0 && vocab > 0, "moe_table: bad sizes");
    CIB_REQUIRE(width <= 12 * 1024, "moe_table: width %d too large for this kernel", width);
    if (num_tokens == 0) return 0;
    dim3 grid(num_tokens * top, (ff + kMoeOutsPerBlock - 1) / kMoeOutsPerBlock);
    const size_t smem = (size_t)width * sizeof(float);
    if (dtype == kF32)
        moe_table_gate_up_kernel<float><<<grid, kMoeWarps * 32, smem, stream>>>((const float*)h, h_stride, ids, table, vocab, top, experts, (const float*)gate_up, (float*)act, width, ff);
    else if (dtype == kBF16)
        moe_table_gate_up_kernel<__nv_bfloat16><<<grid, kMoeWarps * 32, smem, stream>>>((const __nv_bfloat16*)h, h_stride, ids, table, vocab, top, experts, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)act, width, ff);
    else
        CIB_REQUIRE(false, "moe_table: unsupported dtype %d", dtype);
    CIB_LAUNCH_CHECK("moe_table_gate_up");
    return 0;
}

extern "C" int cib_moe_table_down(const void* act, int dtype, const int* ids, const int* table, int vocab, int top,
                                  int experts, const void* down, const void* base, int base_stride, float weight,
                                  void* out, int num_tokens, int width, int ff, cudaStream_t stream) {
    CIB_REQUIRE(num_tokens >= 0 && top > 0 && experts > 0 && width > 0 && ff > 0 && vocab > 0, "moe_table: bad sizes");
    CIB_REQUIRE((size_t)top * ff <= 12 * 1024, "moe_table: %d x %d activations too large for this kernel", top, ff);
    if (num_tokens == 0) return 0;
    dim3 grid(num_tokens, (width + kMoeOutsPerBlock - 1) / kMoeOutsPerBlock);
    const size_t smem = (size_t)top * ff * sizeof(float);
    if (dtype == kF32)
        moe_table_down_kernel<float><<<grid, kMoeWarps * 32, smem, stream>>>((const float*)act, ids, table, vocab, top, experts, (const float*)down, (const float*)base, base_stride, weight, (float*)out, width, ff);
    else if (dtype == kBF16)
        moe_table_down_kernel<__nv_bfloat16><<<grid, kMoeWarps * 32, smem, stream>>>((const __nv_bfloat16*)act, ids, table, vocab, top, experts, (const __nv_bfloat16*)down, (const __nv_bfloat16*)base, base_stride, weight, (__nv_bfloat16*)out, width, ff);
    else
        CIB_REQUIRE(false, "moe_table: unsupported dtype %d", dtype);
    CIB_LAUNCH_CHECK("moe_table_down");
    return 0;
}
