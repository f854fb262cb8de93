// Choice of experts by a router: from 32-bit logits z[t, 0..E-1] the `top` largest (the lower index wins a tie) and
// their weights, the softmax over the chosen logits only.  A warp per token; everything 32-bit.
#include "common.cuh"

namespace cib {

constexpr int kRouterWarps = 8;
constexpr int kRouterPerLane = 32;           // up to 1024 experts

__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const float* __restrict__ logits, int stride, int experts, int top, int* __restrict__ choice,
                   float* __restrict__ weight, int num_tokens) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
    if (t >= num_tokens) return;
    float z[kRouterPerLane];
#pragma unroll
    for (int c = 0; c < kRouterPerLane; ++c) {
        const int e = c * 32 + lane;
        z[c] = e < experts ? logits[(size_t)t * stride + e] : -INFINITY;
        if (z[c] != z[c]) z[c] = -INFINITY;               // a NaN logit is never chosen
    }
    float first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
#pragma unroll
        for (int c = 0; c < kRouterPerLane; ++c) {
            const int e = c * 32 + lane;
            if (e < experts && (z[c] > best || (z[c] == best && e < at))) { best = z[c]; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) at = -1;
        if (k == 0) first = best;
        const float p = at >= 0 ? expf(best - first) : 0.f;
        sum += p;
        if (lane == 0) {
            choice[(size_t)t * top + k] = at;
            weight[(size_t)t * top + k] = p;
        }
#pragma unroll
        for (int c = 0; c < kRouterPerLane; ++c)
            if (c * 32 + lane == at) z[c] = -INFINITY;
    }
    __syncwarp();
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] *= inv;
}

}  // namespace cib

extern "C" int cib_router_topk(const float* logits, int stride, int experts, int top, int* choice, float* weight,
                               int num_tokens, cudaStream_t stream) {
    using namespace cib;
    CIB_REQUIRE(experts > 0 && top > 0 && top <= experts, "router_topk: top %d of %d experts", top, experts);
    CIB_REQUIRE(experts <= 32 * kRouterPerLane, "router_topk: %d experts are beyond %d", experts, 32 * kRouterPerLane);
    if (num_tokens == 0) return 0;
    router_topk_kernel<<<(num_tokens + kRouterWarps - 1) / kRouterWarps, kRouterWarps * 32, 0, stream>>>(logits, stride, experts, top, choice, weight, num_tokens);
    CIB_LAUNCH_CHECK("router_topk");
    return 0;
}
