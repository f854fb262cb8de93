// Mixers that carry a matrix per head from token to token instead of a cache of keys: a matrix memory with
// exponential gates and a running maximum, and the gated delta rule with its short causal convolutions.
//
// A request's tokens of a step are the rows query_start_loc[r] .. query_start_loc[r + 1] - 1, in order; its state lives
// in slot state_slots[r] of a 32-bit pool and is read at the start of the step and written back at its end.  A slot of
// -1 (a padding request of a captured step) starts from zero and stores nothing.  Everything that enters a recurrence
// is 32-bit: gates, decays, their exponentials and logarithms, the state, the read-out.
//
// The scans: column j of a head's matrix, S[:, j], depends on S_(t-1)[:, j], the token's key, the j-th value and
// scalars only, so columns never talk to each other.  A column is held in registers by DP / 32 neighbouring lanes, 32
// values each (DP: the key size rounded up to 32, 64, 128 or 256), so a warp holds 32 / (DP / 32) columns; the dot
// products of a column with the token's key and query are finished by shuffles among its lanes.  The token's key and
// query are staged in shared memory per warp, and the token after the one being computed is fetched meanwhile.
#include "common.cuh"

namespace cib {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

constexpr int kScanWarps = 4;
constexpr int kScanChunk = 16;          // tokens staged in shared memory at a time

// index of key element i in the staging rows: four floats of padding after every 32, so that the lanes of a column
// (which read elements 32 apart, four at a time) hit different banks
__device__ __forceinline__ int pad32(int i) { return i + 4 * (i >> 5); }
template <int DP> constexpr int padded_len() { return DP + 4 * (DP / 32); }

template <int SPLIT>
__device__ __forceinline__ float split_sum(float v) {
#pragma unroll
    for (int o = SPLIT / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// The gates of every token at once, before the scans walk the tokens one by one (in place, 32-bit):
//   kind 0: z[t, h] -> cap * tanh((z + b0[h]) / cap);  z[t, H + h] -> logsigmoid(cap * tanh((z + b1[h]) / cap))
//   kind 1: z[t, h] -> sigmoid(z);                     z[t, H + h] -> exp(-exp(b0[h]) * softplus(z + b1[h]))
__global__ void scan_gates_kernel(float* __restrict__ gates, int stride, int H, long long total, int kind, AnyVec b0, AnyVec b1,
                                  float cap) {
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const long long t = e / H;
    const int h = (int)(e % H);
    float* row = gates + t * stride;
    if (kind == 0) {
        row[h] = cap * tanhf((row[h] + b0[h]) / cap);
        row[H + h] = logsigmoidf_(cap * tanhf((row[H + h] + b1[h]) / cap));
    } else {
        row[h] = sigmoidf_(row[h]);
        row[H + h] = expf(-expf(b0[h]) * softplusf_(row[H + h] + b1[h]));
    }
}

// Stage the rows of `count` tokens (from token `base` on) of one head into shared memory: keys and queries padded as
// above (query times q_scale), this block's value columns, the two gates.  All threads of the block take part.
template <typename TK, typename TV, int DP, int COLS>
__device__ __forceinline__ void stage_chunk(float (*ksm)[padded_len<DP>()], float (*qsm)[padded_len<DP>()], float (*vsm)[COLS],
                                            float (*gsm)[2], const TK* __restrict__ k, const TK* __restrict__ q, size_t kq_stride,
                                            const TV* __restrict__ v, size_t v_stride, int col0, int dv,
                                            const float* __restrict__ gates, int gates_stride, int H, int h, int base,
                                            int count, int d, float q_scale) {
    for (int idx = threadIdx.x; idx < kScanChunk * DP; idx += blockDim.x) {
        const int tt = idx / DP, i = idx % DP;
        const bool ok = tt < count && i < d;
        ksm[tt][pad32(i)] = ok ? to_f32(k[(size_t)(base + tt) * kq_stride + i]) : 0.f;
        qsm[tt][pad32(i)] = ok ? to_f32(q[(size_t)(base + tt) * kq_stride + i]) * q_scale : 0.f;
    }
    for (int idx = threadIdx.x; idx < kScanChunk * COLS; idx += blockDim.x) {
        const int tt = idx / COLS, c = idx % COLS;
        vsm[tt][c] = (tt < count && col0 + c < dv) ? to_f32(v[(size_t)(base + tt) * v_stride + col0 + c]) : 0.f;
    }
    for (int idx = threadIdx.x; idx < kScanChunk * 2; idx += blockDim.x) {
        const int tt = idx >> 1, which = idx & 1;
        gsm[tt][which] = tt < count ? gates[(size_t)(base + tt) * gates_stride + which * H + h] : 0.f;
    }
}

// ---- matrix memory with exponential gates ----------------------------------------------------------------------------
// Per head, with log input gate i and log forget gate f (see scan_gates_kernel), running maximum m (0 at the start):
//   m' = max(f + m, i);  S' = exp(f + m - m') S + exp(i - m') k v^T;  n' likewise with k alone;
//   o = S'^T q / (max(|n' . q|, exp(-m')) + floor),   q scaled by q_scale.
// State of a head: S [d][dv] row-major, then n [d], then m.
template <typename T, int DP>
__global__ void __launch_bounds__(kScanWarps * 32)
mlstm_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int stride,
                  const float* __restrict__ gates, int gates_stride, float q_scale, float floor_, float* __restrict__ state,
                  const int* __restrict__ query_start_loc, const int* __restrict__ state_slots, int num_slots,
                  float* __restrict__ out, int H, int d, int dv) {
    constexpr int SPLIT = DP / 32, CPW = 32 / SPLIT, COLS = CPW * kScanWarps;
    __shared__ __align__(16) float ksm[kScanChunk][padded_len<DP>()];
    __shared__ __align__(16) float qsm[kScanChunk][padded_len<DP>()];
    __shared__ float vsm[kScanChunk][COLS];
    __shared__ float gsm[kScanChunk][2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x, h = blockIdx.y;
    const int col0 = blockIdx.z * COLS;
    const int cb = warp * CPW + lane / SPLIT;                 // column within the block
    const int j = col0 + cb, part = lane % SPLIT, i0 = part * 32;
    const bool col = j < dv;
    const int t0 = query_start_loc[r], t1 = query_start_loc[r + 1];
    if (t1 <= t0) return;
    const int slot = state_slots[r];
    const bool has = slot >= 0 && slot < num_slots;
    const size_t per_head = (size_t)d * dv + d + 1;
    float* st = has ? state + ((size_t)slot * H + h) * per_head : nullptr;
    float S[32], n[SPLIT];
#pragma unroll
    for (int i = 0; i < 32; ++i) S[i] = (has && col && i0 + i < d) ? st[(size_t)(i0 + i) * dv + j] : 0.f;
#pragma unroll
    for (int c = 0; c < SPLIT; ++c) n[c] = (has && c * 32 + lane < d) ? st[(size_t)d * dv + c * 32 + lane] : 0.f;
    float m = has ? st[(size_t)d * dv + d] : 0.f;
    for (int base = t0; base < t1; base += kScanChunk) {
        const int count = min(kScanChunk, t1 - base);
        __syncthreads();
        stage_chunk<T, T, DP, COLS>(ksm, qsm, vsm, gsm, k + (size_t)h * d, q + (size_t)h * d, stride, v + (size_t)h * dv, stride,
                                    col0, dv, gates, gates_stride, H, h, base, count, d, q_scale);
        __syncthreads();
        for (int tt = 0; tt < count; ++tt) {
            const float ig = gsm[tt][0], fg = gsm[tt][1];
            const float m_new = fmaxf(fg + m, ig);
            const float a = expf(fg + m - m_new), b = expf(ig - m_new);
            m = m_new;
            float nq = 0.f;
#pragma unroll
            for (int c = 0; c < SPLIT; ++c) {
                n[c] = a * n[c] + b * ksm[tt][c * 36 + lane];
                nq = fmaf(n[c], qsm[tt][c * 36 + lane], nq);
            }
            nq = warp_sum(nq);
            const float bv = b * vsm[tt][cb];
            float o4[4] = {0.f, 0.f, 0.f, 0.f};          // four partial sums: no long chain of dependent operations
            const float* kseg = &ksm[tt][part * 36];
            const float* qseg = &qsm[tt][part * 36];
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kseg + i);
                const float4 q4 = *reinterpret_cast<const float4*>(qseg + i);
                S[i] = fmaf(a, S[i], bv * k4.x);
                S[i + 1] = fmaf(a, S[i + 1], bv * k4.y);
                S[i + 2] = fmaf(a, S[i + 2], bv * k4.z);
                S[i + 3] = fmaf(a, S[i + 3], bv * k4.w);
                o4[0] = fmaf(S[i], q4.x, o4[0]);
                o4[1] = fmaf(S[i + 1], q4.y, o4[1]);
                o4[2] = fmaf(S[i + 2], q4.z, o4[2]);
                o4[3] = fmaf(S[i + 3], q4.w, o4[3]);
            }
            const float o = split_sum<SPLIT>((o4[0] + o4[1]) + (o4[2] + o4[3]));
            const float den = fmaxf(fabsf(nq), expf(-m)) + floor_;
            if (col && part == 0) out[(size_t)(base + tt) * H * dv + (size_t)h * dv + j] = o / den;
        }
    }
    if (!has) return;
    if (col) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i0 + i < d) st[(size_t)(i0 + i) * dv + j] = S[i];
    }
    if (blockIdx.z == 0 && warp == 0) {
#pragma unroll
        for (int c = 0; c < SPLIT; ++c)
            if (c * 32 + lane < d) st[(size_t)d * dv + c * 32 + lane] = n[c];
        if (lane == 0) st[(size_t)d * dv + d] = m;
    }
}

// ---- gated delta rule ------------------------------------------------------------------------------------------------------
// Step before the scan: a causal convolution over time per channel of the packed rows [q | k | v] (taps [C][K], the
// last column is the current token's; inputs before the step's rows come from the request's conv state
// [K - 1][C], oldest first; zeros before the start of a sequence), SiLU, then q and k heads made unit vectors
// (x / sqrt(sum x^2 + unit_eps)) and q multiplied by q_scale.  A warp per (token, head vector); output 32-bit [T][C].
constexpr int kConvWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kConvWarps * 32)
delta_prep_kernel(const T* __restrict__ x, int stride, const T* __restrict__ taps, int K, const float* __restrict__ conv_state,
                  const int* __restrict__ query_start_loc, const int* __restrict__ token_request,
                  const int* __restrict__ state_slots, int num_slots, int G, int H, int d, int dv, float unit_eps,
                  float q_scale, float* __restrict__ out, int num_tokens) {
    const int lane = threadIdx.x & 31;
    const int vectors = 2 * G + H;
    const long long w = (long long)blockIdx.x * kConvWarps + (threadIdx.x >> 5);
    if (w >= (long long)num_tokens * vectors) return;
    const int t = (int)(w / vectors), vec = (int)(w % vectors);
    const int C = 2 * G * d + H * dv;
    const int len = vec < 2 * G ? d : dv;
    const int c0 = vec < 2 * G ? vec * d : 2 * G * d + (vec - 2 * G) * dv;
    const int r = token_request[t];
    const int start = query_start_loc[r];
    const int slot = state_slots[r];
    const float* cs = (slot >= 0 && slot < num_slots) ? conv_state + (size_t)slot * (K - 1) * C : nullptr;
    float ss = 0.f;
    for (int i = lane; i < len; i += 32) {
        const int c = c0 + i;
        float y = 0.f;
        for (int jb = 0; jb < K; ++jb) {                  // jb tokens back
            const int tt = t - jb;
            float xv = 0.f;
            if (tt >= start) xv = to_f32(x[(size_t)tt * stride + c]);
            else if (cs) xv = cs[(size_t)(K - 1 - (start - tt)) * C + c];
            y = fmaf(to_f32(taps[(size_t)c * K + K - 1 - jb]), xv, y);
        }
        y = y / (1.f + expf(-y));
        out[(size_t)t * C + c] = y;
        ss += y * y;
    }
    if (vec >= 2 * G) return;
    ss = warp_sum(ss);
    const float factor = (vec < G ? q_scale : 1.f) / sqrtf(ss + unit_eps);
    __syncwarp();
    for (int i = lane; i < len; i += 32) out[(size_t)t * C + c0 + i] *= factor;
}

// The conv state after the step: the last K - 1 inputs of (old state ++ the step's rows).  A thread per (request,
// channel) walks its K - 1 entries oldest first, so an entry is read before it is overwritten.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ x, int stride, int K, float* __restrict__ conv_state,
                                         const int* __restrict__ query_start_loc, const int* __restrict__ state_slots,
                                         int num_slots, int C) {
    const int r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int slot = state_slots[r];
    if (slot < 0 || slot >= num_slots) return;
    const int start = query_start_loc[r], n = query_start_loc[r + 1] - start;
    if (n <= 0) return;
    float* cs = conv_state + (size_t)slot * (K - 1) * C;
    for (int i = 0; i < K - 1; ++i) {
        const int at = n + i;                              // index into old state (K - 1 entries) followed by the rows
        cs[(size_t)i * C + c] = at < K - 1 ? cs[(size_t)at * C + c] : to_f32(x[(size_t)(start + at - (K - 1)) * stride + c]);
    }
}

// The scan.  Per head h (its q and k are those of head h / (H / G)), decay g = exp(-exp(A_log) * softplus(z_a + dt_bias))
// and beta = sigmoid(z_b):
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
// Column j: with r = S_old[:, j].k and p = S_old[:, j].q, u_j = beta (v_j - g r) and o_j = g p + u_j (k.q).
template <int DP>
__global__ void __launch_bounds__(kScanWarps * 32)
delta_scan_kernel(const float* __restrict__ qkv, int G, const float* __restrict__ gates, int gates_stride,
                  float* __restrict__ state, const int* __restrict__ query_start_loc, const int* __restrict__ state_slots,
                  int num_slots, float* __restrict__ out, int H, int d, int dv) {
    constexpr int SPLIT = DP / 32, CPW = 32 / SPLIT, COLS = CPW * kScanWarps;
    __shared__ __align__(16) float ksm[kScanChunk][padded_len<DP>()];
    __shared__ __align__(16) float qsm[kScanChunk][padded_len<DP>()];
    __shared__ float vsm[kScanChunk][COLS];
    __shared__ float gsm[kScanChunk][2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x, h = blockIdx.y;
    const int col0 = blockIdx.z * COLS;
    const int cb = warp * CPW + lane / SPLIT;
    const int j = col0 + cb, part = lane % SPLIT, i0 = part * 32;
    const bool col = j < dv;
    const int t0 = query_start_loc[r], t1 = query_start_loc[r + 1];
    if (t1 <= t0) return;
    const int slot = state_slots[r];
    const bool has = slot >= 0 && slot < num_slots;
    float* st = has ? state + ((size_t)slot * H + h) * d * dv : nullptr;
    float S[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) S[i] = (has && col && i0 + i < d) ? st[(size_t)(i0 + i) * dv + j] : 0.f;
    const int C = 2 * G * d + H * dv;
    const int g_head = h / (H / G);
    for (int base = t0; base < t1; base += kScanChunk) {
        const int count = min(kScanChunk, t1 - base);
        __syncthreads();
        stage_chunk<float, float, DP, COLS>(ksm, qsm, vsm, gsm, qkv + (size_t)G * d + (size_t)g_head * d, qkv + (size_t)g_head * d, C,
                                            qkv + (size_t)2 * G * d + (size_t)h * dv, C, col0, dv, gates, gates_stride, H, h, base,
                                            count, d, 1.f);
        __syncthreads();
        for (int tt = 0; tt < count; ++tt) {
            const float beta = gsm[tt][0], decay = gsm[tt][1];
            float kq = 0.f;
#pragma unroll
            for (int c = 0; c < SPLIT; ++c) kq = fmaf(ksm[tt][c * 36 + lane], qsm[tt][c * 36 + lane], kq);
            kq = warp_sum(kq);
            const float* kseg = &ksm[tt][part * 36];
            const float* qseg = &qsm[tt][part * 36];
            float rk4[4] = {0.f, 0.f, 0.f, 0.f}, pq4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kseg + i);
                const float4 q4 = *reinterpret_cast<const float4*>(qseg + i);
                rk4[0] = fmaf(S[i], k4.x, rk4[0]);
                rk4[1] = fmaf(S[i + 1], k4.y, rk4[1]);
                rk4[2] = fmaf(S[i + 2], k4.z, rk4[2]);
                rk4[3] = fmaf(S[i + 3], k4.w, rk4[3]);
                pq4[0] = fmaf(S[i], q4.x, pq4[0]);
                pq4[1] = fmaf(S[i + 1], q4.y, pq4[1]);
                pq4[2] = fmaf(S[i + 2], q4.z, pq4[2]);
                pq4[3] = fmaf(S[i + 3], q4.w, pq4[3]);
            }
            const float rk = split_sum<SPLIT>((rk4[0] + rk4[1]) + (rk4[2] + rk4[3]));
            const float pq = split_sum<SPLIT>((pq4[0] + pq4[1]) + (pq4[2] + pq4[3]));
            const float u = beta * (vsm[tt][cb] - decay * rk);
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kseg + i);
                S[i] = fmaf(decay, S[i], k4.x * u);
                S[i + 1] = fmaf(decay, S[i + 1], k4.y * u);
                S[i + 2] = fmaf(decay, S[i + 2], k4.z * u);
                S[i + 3] = fmaf(decay, S[i + 3], k4.w * u);
            }
            if (col && part == 0) out[(size_t)(base + tt) * H * dv + (size_t)h * dv + j] = decay * pq + u * kq;
        }
    }
    if (has && col) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i0 + i < d) st[(size_t)(i0 + i) * dv + j] = S[i];
    }
}

// ---- after a scan: per-head RMS norm, gain, output gate -----------------------------------------------------------------------
// out[t, h, j] = o[t, h, j] / sqrt(mean_j o[t, h, :]^2 + eps) * gain[(per_head ? h * dv : 0) + j] * act(gate[t, h * dv + j]),
// act = sigmoid (0) or SiLU (1).  A warp per (token, head); o is 32-bit.
constexpr int kGateWarps = 8;
template <typename T>
__global__ void __launch_bounds__(kGateWarps * 32)
head_rms_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride, AnyVec gain, int per_head,
                     float eps, int act, T* __restrict__ out, int H, int dv, int num_tokens) {
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * kGateWarps + (threadIdx.x >> 5);
    if (w >= (long long)num_tokens * H) return;
    const int t = (int)(w / H), h = (int)(w % H);
    const float* src = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const float factor = 1.f / sqrtf(ss / (float)dv + eps);
    for (int i = lane; i < dv; i += 32) {
        const float z = to_f32(gate[(size_t)t * gate_stride + (size_t)h * dv + i]);
        const float s = 1.f / (1.f + expf(-z));
        const float a = act == 1 ? z * s : s;
        out[((size_t)t * H + h) * dv + i] = from_f32<T>(src[i] * factor * gain[(per_head ? h * dv : 0) + i] * a);
    }
}

}  // namespace cib

using namespace cib;

#define CIB_SCAN_DISPATCH(d, CALL)                         \
    do {                                                   \
        if (d <= 32) { constexpr int DP = 32; CALL; }      \
        else if (d <= 64) { constexpr int DP = 64; CALL; } \
        else if (d <= 128) { constexpr int DP = 128; CALL; } \
        else { constexpr int DP = 256; CALL; }             \
    } while (0)

extern "C" int cib_mlstm_scan(const void* q, const void* k, const void* v, int dtype, int stride, float* gates,
                              int gates_stride, const void* i_bias, const void* f_bias, int bias_dtype, float cap,
                              float q_scale, float floor_, float* state, const int* query_start_loc, const int* state_slots,
                              int num_slots, int num_requests, int num_tokens, float* out, int H, int d, int dv, cudaStream_t stream) {
    CIB_REQUIRE(H > 0 && d > 0 && dv > 0 && cap > 0.f, "mlstm_scan: bad sizes");
    CIB_REQUIRE(d <= 256, "mlstm_scan: key size %d is beyond 256", d);
    if (num_requests == 0) return 0;
    const int dp = d <= 32 ? 32 : d <= 64 ? 64 : d <= 128 ? 128 : 256;
    const int cols = (32 / (dp / 32)) * kScanWarps;               // columns of the matrix a block holds
    dim3 grid(num_requests, H, (dv + cols - 1) / cols);
    AnyVec bi{i_bias, bias_dtype == kBF16}, bf{f_bias, bias_dtype == kBF16};
    CIB_REQUIRE(num_tokens >= 0, "mlstm_scan: bad token count");
    if (num_tokens == 0) return 0;
    {
        const long long total = (long long)num_tokens * H;
        scan_gates_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(gates, gates_stride, H, total, 0, bi, bf, cap);
        CIB_LAUNCH_CHECK("scan_gates");
    }
    if (dtype == kF32) {
        CIB_SCAN_DISPATCH(d, (mlstm_scan_kernel<float, DP><<<grid, kScanWarps * 32, 0, stream>>>((const float*)q, (const float*)k, (const float*)v, stride, gates, gates_stride, q_scale, floor_, state, query_start_loc, state_slots, num_slots, out, H, d, dv)));
    } else if (dtype == kBF16) {
        CIB_SCAN_DISPATCH(d, (mlstm_scan_kernel<__nv_bfloat16, DP><<<grid, kScanWarps * 32, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, stride, gates, gates_stride, q_scale, floor_, state, query_start_loc, state_slots, num_slots, out, H, d, dv)));
    } else {
        CIB_REQUIRE(false, "mlstm_scan: bad dtype %d", dtype);
    }
    CIB_LAUNCH_CHECK("mlstm_scan");
    return 0;
}

extern "C" int cib_delta_prep(const void* x, int dtype, int stride, const void* taps, int K, float* conv_state,
                              const int* query_start_loc, const int* token_request, const int* state_slots, int num_slots,
                              int num_requests, int G, int H, int d, int dv, float unit_eps, float q_scale, float* out,
                              int num_tokens, cudaStream_t stream) {
    CIB_REQUIRE(G > 0 && H > 0 && H % G == 0 && d > 0 && dv > 0 && K >= 1, "delta_prep: bad sizes");
    if (num_tokens == 0) return 0;
    const long long warps = (long long)num_tokens * (2 * G + H);
    const int blocks = (int)((warps + kConvWarps - 1) / kConvWarps);
    const int C = 2 * G * d + H * dv;
    dim3 ugrid((C + 127) / 128, num_requests);
    if (dtype == kF32) {
        delta_prep_kernel<float><<<blocks, kConvWarps * 32, 0, stream>>>((const float*)x, stride, (const float*)taps, K, conv_state, query_start_loc, token_request, state_slots, num_slots, G, H, d, dv, unit_eps, q_scale, out, num_tokens);
        CIB_LAUNCH_CHECK("delta_prep");
        if (K > 1) conv_state_update_kernel<float><<<ugrid, 128, 0, stream>>>((const float*)x, stride, K, conv_state, query_start_loc, state_slots, num_slots, C);
    } else if (dtype == kBF16) {
        delta_prep_kernel<__nv_bfloat16><<<blocks, kConvWarps * 32, 0, stream>>>((const __nv_bfloat16*)x, stride, (const __nv_bfloat16*)taps, K, conv_state, query_start_loc, token_request, state_slots, num_slots, G, H, d, dv, unit_eps, q_scale, out, num_tokens);
        CIB_LAUNCH_CHECK("delta_prep");
        if (K > 1) conv_state_update_kernel<__nv_bfloat16><<<ugrid, 128, 0, stream>>>((const __nv_bfloat16*)x, stride, K, conv_state, query_start_loc, state_slots, num_slots, C);
    } else {
        CIB_REQUIRE(false, "delta_prep: bad dtype %d", dtype);
    }
    CIB_LAUNCH_CHECK("conv_state_update");
    return 0;
}

extern "C" int cib_delta_scan(const float* qkv, int G, float* gates, int gates_stride, const void* a_log,
                              const void* dt_bias, int vec_dtype, float* state, const int* query_start_loc,
                              const int* state_slots, int num_slots, int num_requests, int num_tokens, float* out, int H, int d,
                              int dv, cudaStream_t stream) {
    CIB_REQUIRE(G > 0 && H > 0 && H % G == 0 && d > 0 && dv > 0, "delta_scan: bad sizes");
    CIB_REQUIRE(d <= 256, "delta_scan: key size %d is beyond 256", d);
    if (num_requests == 0) return 0;
    const int dp = d <= 32 ? 32 : d <= 64 ? 64 : d <= 128 ? 128 : 256;
    const int cols = (32 / (dp / 32)) * kScanWarps;               // columns of the matrix a block holds
    dim3 grid(num_requests, H, (dv + cols - 1) / cols);
    AnyVec al{a_log, vec_dtype == kBF16}, db{dt_bias, vec_dtype == kBF16};
    CIB_REQUIRE(num_tokens >= 0, "delta_scan: bad token count");
    if (num_tokens == 0) return 0;
    {
        const long long total = (long long)num_tokens * H;
        scan_gates_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(gates, gates_stride, H, total, 1, al, db, 1.f);
        CIB_LAUNCH_CHECK("scan_gates");
    }
    CIB_SCAN_DISPATCH(d, (delta_scan_kernel<DP><<<grid, kScanWarps * 32, 0, stream>>>(qkv, G, gates, gates_stride, state, query_start_loc, state_slots, num_slots, out, H, d, dv)));
    CIB_LAUNCH_CHECK("delta_scan");
    return 0;
}

extern "C" int cib_head_rms_gate(const float* o, const void* gate, int dtype, int gate_stride, const void* gain, int gain_dtype,
                                 int per_head, float eps, int act, void* out, int H, int dv, int num_tokens,
                                 cudaStream_t stream) {
    CIB_REQUIRE(H > 0 && dv > 0 && (act == 0 || act == 1), "head_rms_gate: bad sizes");
    if (num_tokens == 0) return 0;
    const long long warps = (long long)num_tokens * H;
    const int blocks = (int)((warps + kGateWarps - 1) / kGateWarps);
    AnyVec gv{gain, gain_dtype == kBF16};
    if (dtype == kF32)
        head_rms_gate_kernel<float><<<blocks, kGateWarps * 32, 0, stream>>>(o, (const float*)gate, gate_stride, gv, per_head, eps, act, (float*)out, H, dv, num_tokens);
    else if (dtype == kBF16)
        head_rms_gate_kernel<__nv_bfloat16><<<blocks, kGateWarps * 32, 0, stream>>>(o, (const __nv_bfloat16*)gate, gate_stride, gv, per_head, eps, act, (__nv_bfloat16*)out, H, dv, num_tokens);
    else
        CIB_REQUIRE(false, "head_rms_gate: bad dtype %d", dtype);
    CIB_LAUNCH_CHECK("head_rms_gate");
    return 0;
}
