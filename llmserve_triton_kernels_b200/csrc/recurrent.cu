// Element-wise gated recurrences over a flat batch: every request's new tokens are walked in order from the state
// that its slot holds, and the slot is left with the state after the last of them.
//
// The state, the gates, the candidate and the output gate are 32-bit; only the result is rounded to the element type.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

// minGRU.  proj row: [z pre-activation | candidate pre-activation | output-gate pre-activation], each `width` wide.
//   z = sigmoid(pz + bz);  u = pu + bu;  c = u >= 0 ? u + 1/2 : sigmoid(u);  S = (1 - z) S + z c;  out = S * silu(pg)
// One thread per (request, channel).  Nothing but S is carried from token to token, so the loads of the next tokens
// are in flight while a token is worked out.
template <typename TP, typename TO, int UNROLL>
__global__ void __launch_bounds__(128)
mingru_scan_kernel(const TP* __restrict__ proj, int ldp, const float* __restrict__ bias_z, const float* __restrict__ bias_u,
                   float* __restrict__ states, const int* __restrict__ state_slots, const int* __restrict__ cu_tokens,
                   TO* __restrict__ out, int ldo, int width) {
    pdl_trigger();
    const int r = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    const int begin = cu_tokens[r], end = cu_tokens[r + 1], slot = state_slots[r];
    const float bz = bias_z ? bias_z[c] : 0.f, bu = bias_u ? bias_u[c] : 0.f;
    pdl_wait();
    float S = states[(size_t)slot * width + c];
    int t = begin;
    for (; t + UNROLL <= end; t += UNROLL) {
        float pz[UNROLL], pu[UNROLL], pg[UNROLL];
#pragma unroll
        for (int e = 0; e < UNROLL; ++e) {
            const TP* row = proj + (size_t)(t + e) * ldp + c;
            pz[e] = to_float(row[0]);
            pu[e] = to_float(row[width]);
            pg[e] = to_float(row[2 * width]);
        }
#pragma unroll
        for (int e = 0; e < UNROLL; ++e) {
            const float z = sigmoid_f(pz[e] + bz), u = pu[e] + bu;
            const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
            S = (1.f - z) * S + z * cand;
            out[(size_t)(t + e) * ldo + c] = from_float<TO>(S * (pg[e] * sigmoid_f(pg[e])));
        }
    }
    for (; t < end; ++t) {
        const TP* row = proj + (size_t)t * ldp + c;
        const float z = sigmoid_f(to_float(row[0]) + bz), u = to_float(row[width]) + bu, g = to_float(row[2 * width]);
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        S = (1.f - z) * S + z * cand;
        out[(size_t)t * ldo + c] = from_float<TO>(S * (g * sigmoid_f(g)));
    }
    states[(size_t)slot * width + c] = S;
}

// The same for requests that bring many tokens: a CTA owns 32 channels of one request, its 32 warps a stretch of the
// request's tokens each.  The recurrence S_t = a_t S_(t-1) + b_t (a = 1 - z, b = z c) is linear in S, so a stretch is
// summed up by (A, B) = (product of its a, its result from S = 0); the states at the starts of the stretches follow
// from those through shared memory, and each warp then walks its stretch from its true start state.  The gate and the
// candidate are read twice, the second time from L2.
template <typename TP, typename TO, int UNROLL>
__global__ void __launch_bounds__(1024)
mingru_scan_stretches_kernel(const TP* __restrict__ proj, int ldp, const float* __restrict__ bias_z,
                             const float* __restrict__ bias_u, float* __restrict__ states, const int* __restrict__ state_slots,
                             const int* __restrict__ cu_tokens, TO* __restrict__ out, int ldo, int width) {
    __shared__ float sA[32][33], sB[32][33];
    pdl_trigger();
    const int r = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    const bool live = c < width;
    const int cc = live ? c : width - 1;
    const int begin = cu_tokens[r], end = cu_tokens[r + 1], slot = state_slots[r];
    const int stretch = (end - begin + 31) / 32;
    const int t0 = min(end, begin + warp * stretch), t1 = min(end, t0 + stretch);
    const float bz = bias_z ? bias_z[cc] : 0.f, bu = bias_u ? bias_u[cc] : 0.f;
    pdl_wait();
    float A = 1.f, B = 0.f;
    int t = t0;
    for (; t + UNROLL <= t1; t += UNROLL) {
        float pz[UNROLL], pu[UNROLL];
#pragma unroll
        for (int e = 0; e < UNROLL; ++e) {
            const TP* row = proj + (size_t)(t + e) * ldp + cc;
            pz[e] = to_float(row[0]);
            pu[e] = to_float(row[width]);
        }
#pragma unroll
        for (int e = 0; e < UNROLL; ++e) {
            const float z = sigmoid_f(pz[e] + bz), u = pu[e] + bu;
            const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
            B = (1.f - z) * B + z * cand;
            A *= 1.f - z;
        }
    }
    for (; t < t1; ++t) {
        const TP* row = proj + (size_t)t * ldp + cc;
        const float z = sigmoid_f(to_float(row[0]) + bz), u = to_float(row[width]) + bu;
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        B = (1.f - z) * B + z * cand;
        A *= 1.f - z;
    }
    sA[warp][lane] = A;
    sB[warp][lane] = B;
    __syncthreads();
    float S = states[(size_t)slot * width + cc];
    for (int s = 0; s < warp; ++s) S = sA[s][lane] * S + sB[s][lane];
    t = t0;
    for (; t + UNROLL <= t1; t += UNROLL) {
        float pz[UNROLL], pu[UNROLL], pg[UNROLL];
#pragma unroll
        for (int e = 0; e < UNROLL; ++e) {
            const TP* row = proj + (size_t)(t + e) * ldp + cc;
            pz[e] = to_float(row[0]);
            pu[e] = to_float(row[width]);
            pg[e] = to_float(row[2 * width]);
        }
#pragma unroll
        for (int e = 0; e < UNROLL; ++e) {
            const float z = sigmoid_f(pz[e] + bz), u = pu[e] + bu;
            const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
            S = (1.f - z) * S + z * cand;
            if (live) out[(size_t)(t + e) * ldo + c] = from_float<TO>(S * (pg[e] * sigmoid_f(pg[e])));
        }
    }
    for (; t < t1; ++t) {
        const TP* row = proj + (size_t)t * ldp + cc;
        const float z = sigmoid_f(to_float(row[0]) + bz), u = to_float(row[width]) + bu, g = to_float(row[2 * width]);
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        S = (1.f - z) * S + z * cand;
        if (live) out[(size_t)t * ldo + c] = from_float<TO>(S * (g * sigmoid_f(g)));
    }
    if (live && t1 == end && t0 < t1) states[(size_t)slot * width + c] = S;  // the warp that holds the request's last token
}

}  // namespace

LLM_EXPORT int llm_mingru_scan(const void* proj, int proj_dtype, int ldp, const float* bias_z, const float* bias_u,
                               float* states, const int* state_slots, const int* cu_tokens, void* out, int out_dtype,
                               int ldo, int requests, int width, int max_query_len, cudaStream_t stream) {
    if (requests <= 0 || width <= 0) return 0;
    if (ldp < 3 * width || ldo < width || requests > 65535) return LLM_ERR_BAD_ARGUMENT;
    using bf = __nv_bfloat16;
    // requests of at most 64 tokens: a thread walks a channel; longer ones: 32 warps share a request's tokens
    const bool stretches = max_query_len > 64;
    const dim3 grid(stretches ? (width + 31) / 32 : (width + 127) / 128, requests), block(stretches ? 1024 : 128);
    auto go = [&](auto kernel, auto* p, auto* o) {
        return launch_pdl(kernel, grid, block, 0, stream, p, ldp, bias_z, bias_u, states, state_slots, cu_tokens, o, ldo, width);
    };
    if (stretches) {
        if (proj_dtype == LLM_F32 && out_dtype == LLM_F32) return go(mingru_scan_stretches_kernel<float, float, 4>, (const float*)proj, (float*)out);
        if (proj_dtype == LLM_F32 && out_dtype == LLM_BF16) return go(mingru_scan_stretches_kernel<float, bf, 4>, (const float*)proj, (bf*)out);
        if (proj_dtype == LLM_BF16 && out_dtype == LLM_BF16) return go(mingru_scan_stretches_kernel<bf, bf, 4>, (const bf*)proj, (bf*)out);
        return LLM_ERR_BAD_ARGUMENT;
    }
    if (proj_dtype == LLM_F32 && out_dtype == LLM_F32) return go(mingru_scan_kernel<float, float, 8>, (const float*)proj, (float*)out);
    if (proj_dtype == LLM_F32 && out_dtype == LLM_BF16) return go(mingru_scan_kernel<float, bf, 8>, (const float*)proj, (bf*)out);
    if (proj_dtype == LLM_BF16 && out_dtype == LLM_BF16) return go(mingru_scan_kernel<bf, bf, 8>, (const bf*)proj, (bf*)out);
    return LLM_ERR_BAD_ARGUMENT;
}
