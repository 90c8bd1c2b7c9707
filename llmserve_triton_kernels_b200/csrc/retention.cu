// Retention: linear attention with one fixed decay per head and a matrix of state per (request, head).
//
//   S_t = decay_h S_(t-1) + k_t v_t^T        o_t = S_t^T q_t            S: [D, V] float32, zero when a request starts
//
// Queries, keys, values, the state and the sums are 32-bit.  Column v of S is all that o_t[v] needs, so the columns
// are shared out: a CTA owns 16 columns of one (request, head), eight threads a column, each with D / 8 rows of it in
// registers.  The request's new tokens are walked in order and the slot is left with the state after the last.
//
// Also here: the step behind it, each head's o divided by its root mean square and multiplied by a gate.
#include "common.cuh"

namespace {

constexpr int COLS = 16;  // columns of the state a CTA owns
constexpr int TPC = 8;    // threads a column

// q, k: [N, H, D] float32 (row pitches ldq, ldk); v: [N, H, V] (pitch ldv, any type); states: [slots, H, D, V]
// out: [N, H, V] float32
template <typename TV, int DPT>
__global__ void __launch_bounds__(COLS * TPC)
retention_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk, const TV* __restrict__ v, int ldv,
                      const float* __restrict__ decay, float* __restrict__ states, const int* __restrict__ state_slots,
                      const int* __restrict__ cu_tokens, float* __restrict__ out, int H, int D, int V) {
    extern __shared__ float tile[];  // [D][COLS + 1]
    pdl_trigger();
    const int r = blockIdx.z, h = blockIdx.y, v0 = blockIdx.x * COLS;
    const int sub = threadIdx.x % TPC, col = threadIdx.x / TPC;
    const int begin = cu_tokens[r], end = cu_tokens[r + 1], slot = state_slots[r];
    const float gamma = decay[h];
    float* state = states + ((size_t)slot * H + h) * D * V;
    pdl_wait();
    for (int i = threadIdx.x; i < D * COLS; i += blockDim.x) {
        const int d = i / COLS, c = i % COLS;
        tile[d * (COLS + 1) + c] = v0 + c < V ? state[(size_t)d * V + v0 + c] : 0.f;
    }
    __syncthreads();
    float S[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = sub + TPC * i;
        S[i] = d < D ? tile[d * (COLS + 1) + col] : 0.f;
    }
    const bool live = v0 + col < V;
    const int vc = live ? v0 + col : V - 1;
    for (int t = begin; t < end; ++t) {
        const float* qt = q + (size_t)t * ldq + (size_t)h * D;
        const float* kt = k + (size_t)t * ldk + (size_t)h * D;
        const float vt = to_float(v[(size_t)t * ldv + (size_t)h * V + vc]);
        float kk[DPT], qq[DPT];
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = sub + TPC * i;
            kk[i] = d < D ? kt[d] : 0.f;
            qq[i] = d < D ? qt[d] : 0.f;
        }
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            S[i] = fmaf(gamma, S[i], kk[i] * vt);
            o = fmaf(S[i], qq[i], o);
        }
        o += __shfl_xor_sync(0xffffffffu, o, 1);
        o += __shfl_xor_sync(0xffffffffu, o, 2);
        o += __shfl_xor_sync(0xffffffffu, o, 4);
        if (sub == 0 && live) out[((size_t)t * H + h) * V + v0 + col] = o;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = sub + TPC * i;
        if (d < D) tile[d * (COLS + 1) + col] = S[i];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D * COLS; i += blockDim.x) {
        const int d = i / COLS, c = i % COLS;
        if (v0 + c < V) state[(size_t)d * V + v0 + c] = tile[d * (COLS + 1) + c];
    }
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * gate(g[t, h, :]), one warp per (token, head).
// gate_kind: 0 sigmoid(g), 1 silu(g), -1 none.  eps < 0: no norm.
template <typename TG, typename TO>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const TG* __restrict__ g, int ldg, TO* __restrict__ out, int rows, int heads,
                      int V, float eps, int gate_kind) {
    pdl_trigger();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_wait();
    if (row >= rows) return;
    const int t = row / heads, h = row % heads;
    const float* src = o + (size_t)row * V;
    float ss = 0.f;
    for (int i = lane; i < V; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const float scale = eps >= 0.f ? 1.f / sqrtf(ss / (float)V + eps) : 1.f;
    for (int i = lane; i < V; i += 32) {
        float y = src[i] * scale;
        if (gate_kind >= 0) {
            const float z = to_float(g[(size_t)t * ldg + (size_t)h * V + i]);
            const float s = 1.f / (1.f + expf(-z));
            y *= gate_kind == 1 ? z * s : s;
        }
        out[(size_t)row * V + i] = from_float<TO>(y);
    }
}

}  // namespace

LLM_EXPORT int llm_retention_scan(const float* q, int ldq, const float* k, int ldk, const void* v, int v_dtype, int ldv,
                                  const float* decay, float* states, const int* state_slots, const int* cu_tokens, float* out,
                                  int requests, int H, int D, int V, cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || D > 256 || requests > 65535 || H > 65535) return LLM_ERR_BAD_ARGUMENT;
    const dim3 grid((V + COLS - 1) / COLS, H, requests), block(COLS * TPC);
    const size_t smem = (size_t)D * (COLS + 1) * sizeof(float);
    using bf = __nv_bfloat16;
    auto go = [&](auto kernel, auto* vp) {
        return launch_pdl(kernel, grid, block, smem, stream, q, ldq, k, ldk, vp, ldv, decay, states, state_slots, cu_tokens, out, H, D, V);
    };
#define LLM_RET(DPT) (v_dtype == LLM_F32 ? go(retention_scan_kernel<float, DPT>, (const float*)v) : go(retention_scan_kernel<bf, DPT>, (const bf*)v))
    if (D <= 32) return LLM_RET(4);
    if (D <= 64) return LLM_RET(8);
    if (D <= 128) return LLM_RET(16);
    return LLM_RET(32);
#undef LLM_RET
}

LLM_EXPORT int llm_head_norm_gate(const float* o, const void* g, int g_dtype, int ldg, void* out, int out_dtype, int N, int heads,
                                  int V, float eps, int gate_kind, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (heads <= 0 || V <= 0 || (gate_kind >= 0 && !g)) return LLM_ERR_BAD_ARGUMENT;
    const int rows = N * heads;
    const dim3 grid((rows + 3) / 4), block(128);
    using bf = __nv_bfloat16;
    auto go = [&](auto kernel, auto* gp, auto* op) { return launch_pdl(kernel, grid, block, 0, stream, o, gp, ldg, op, rows, heads, V, eps, gate_kind); };
    if (g_dtype == LLM_F32 && out_dtype == LLM_F32) return go(head_norm_gate_kernel<float, float>, (const float*)g, (float*)out);
    if (g_dtype == LLM_F32 && out_dtype == LLM_BF16) return go(head_norm_gate_kernel<float, bf>, (const float*)g, (bf*)out);
    if (g_dtype == LLM_BF16 && out_dtype == LLM_BF16) return go(head_norm_gate_kernel<bf, bf>, (const bf*)g, (bf*)out);
    return LLM_ERR_UNSUPPORTED;
}
