// Attention without a softmax: the weight of a visible key is a sigmoid of its capped score plus a number per head,
// and the heads' weights are mixed by a matrix before they meet the values.
//
//   s_g(i, j)  = cap * tanh(scale * q_g(i) . k_c(g)(j) / cap)            (cap == 0: no cap)
//   p_g(i, j)  = sigmoid(s_g(i, j) + bias[g])  for first(i) <= j <= i,   0 elsewhere
//   w_h(i, j)  = sum_g mix[h, g] p_g(i, j)                               (mix == null: w = p)
//   out_h(i)   = sum_j w_h(i, j) v_c(h)(j)
//
// Nothing is normalised over keys, so the sum over keys may be cut anywhere and the pieces added: a long context is
// shared out over `splits` CTAs in stretches of a fixed number of keys, counted from position 0, and the partial sums
// are added in the order of the stretches.  Scores, weights and sums are 32-bit.
//
// Also here: what a token's projections go through before they are keys and queries (an RMS norm over the whole
// projection, a rotation of the first lanes of every head, a factor on the keys) together with the cache write.
#include "common.cuh"

#include <type_traits>

namespace {

constexpr int CHUNK = 32;  // keys a warp scores at once, one a lane; chunks start at multiples of 32 keys

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

// One CTA per (query token, block of 32 output heads, stretch of keys); warp w scores heads w, w + W, ... and sums
// up output head 32 * block + w.
//   q:     [N, H, D]  (row pitch ldq)
//   pool:  [pages, 2, KV, page_size, Dp] keys in plane 0, values in plane 1
//   out:   [splits, N, H * V] float32 partial sums when splits > 1, else [N, H * V] of type TO
template <typename TQ, typename TC, typename TO, int VPL>
__global__ void __launch_bounds__(1024)
sigmoid_attention_kernel(const TQ* __restrict__ q, int ldq, const TC* __restrict__ pool, const int* __restrict__ page_table,
                         int table_width, const int* __restrict__ positions, const int* __restrict__ token_request,
                         const float* __restrict__ bias, const float* __restrict__ mix, void* __restrict__ out_, int N,
                         int H, int KV, int D, int V, int Dp, int page_size, float scale, float cap, int window,
                         int split_keys, int splits) {
    extern __shared__ float smem[];
    float* sq = smem;                    // [H][D] the token's queries
    float* sp = sq + (size_t)H * D;      // [H][CHUNK] weights of the chunk before mixing
    float* smix = sp + (size_t)H * CHUNK;  // [32][H] this block's rows of the mixing matrix
    const int t = blockIdx.x, hb = blockIdx.y, split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, W = blockDim.x >> 5;
    const int h_out = hb * 32 + warp;
    const bool has_out = h_out < H;
    const int group = H / KV;
    pdl_trigger();
    const int pos = positions[t], req = token_request[t];
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    // a stretch none of whose keys the token sees leaves its partial sums unwritten: the sum reads only stretches that have some
    if (splits > 1 && (split * split_keys > pos || (split + 1) * split_keys <= first)) return;
    const int* table = page_table + (size_t)req * table_width;
    if (mix)
        for (int i = threadIdx.x; i < 32 * H; i += blockDim.x) {
            const int r = hb * 32 + i / H;
            smix[i] = r < H ? mix[(size_t)r * H + i % H] : 0.f;
        }
    pdl_wait();
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) sq[i] = to_float(q[(size_t)t * ldq + i]);
    __syncthreads();
    int j_lo = max(first, split * split_keys), j_hi = min(pos, (split + 1) * split_keys - 1);  // inclusive
    float acc[VPL];
#pragma unroll
    for (int m = 0; m < VPL; ++m) acc[m] = 0.f;
    const size_t plane = (size_t)KV * page_size * Dp;
    const int c_out = has_out ? h_out / group : 0;
    for (int j0 = (j_lo / CHUNK) * CHUNK; j0 <= j_hi; j0 += CHUNK) {
        const int j = j0 + lane;
        const bool seen = j >= j_lo && j <= j_hi;
        size_t row = 0;  // of key j in a plane of one key/value head, in elements
        size_t page_base = 0;
        if (seen) {
            const int page = table[j / page_size];
            page_base = (size_t)page * 2 * plane;
            row = (size_t)(j % page_size) * Dp;
        }
        for (int g = warp; g < H; g += W) {
            float p = 0.f;
            if (seen) {
                const TC* k = pool + page_base + (size_t)(g / group) * page_size * Dp + row;
                const float* qg = sq + (size_t)g * D;
                float s = 0.f;
                for (int d = 0; d < D; ++d) s = fmaf(qg[d], to_float(k[d]), s);
                s *= scale;
                if (cap > 0.f) s = cap * tanhf(s / cap);
                p = sigmoid_f(s + (bias ? bias[g] : 0.f));
            }
            sp[g * CHUNK + lane] = p;
        }
        __syncthreads();
        if (has_out) {
            float w;
            if (mix) {
                w = 0.f;
                const float* mrow = smix + (size_t)warp * H;
                for (int g = 0; g < H; ++g) w = fmaf(mrow[g], sp[g * CHUNK + lane], w);
            } else {
                w = sp[h_out * CHUNK + lane];
            }
            // the chunk's keys one after the other, every lane summing up its lanes of the value rows
            const int last = min(CHUNK - 1, j_hi - j0);
            for (int jj = max(0, j_lo - j0); jj <= last; ++jj) {
                const float wj = __shfl_sync(0xffffffffu, w, jj);
                const size_t pb = __shfl_sync(0xffffffffu, (unsigned long long)page_base, jj);
                const size_t rw = __shfl_sync(0xffffffffu, (unsigned long long)row, jj);
                const TC* v = pool + pb + plane + (size_t)c_out * page_size * Dp + rw;
#pragma unroll
                for (int m = 0; m < VPL; ++m) {
                    const int dv = lane + 32 * m;
                    if (dv < V) acc[m] = fmaf(wj, to_float(v[dv]), acc[m]);
                }
            }
        }
        __syncthreads();
    }
    if (!has_out) return;
    if (splits > 1) {
        float* out = reinterpret_cast<float*>(out_) + ((size_t)split * N + t) * H * V + (size_t)h_out * V;
#pragma unroll
        for (int m = 0; m < VPL; ++m)
            if (lane + 32 * m < V) out[lane + 32 * m] = acc[m];
    } else {
        TO* out = reinterpret_cast<TO*>(out_) + (size_t)t * H * V + (size_t)h_out * V;
#pragma unroll
        for (int m = 0; m < VPL; ++m)
            if (lane + 32 * m < V) out[lane + 32 * m] = from_float<TO>(acc[m]);
    }
}

// out[i] = sum over the stretches, in their order, of part[s][i]
template <typename TO>
__global__ void __launch_bounds__(256)
sum_parts_kernel(const float* __restrict__ part, TO* __restrict__ out, const int* __restrict__ positions, int row, size_t count,
                 int split_keys, int window, int shares) {
    pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const int pos = positions[i / row];
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    pdl_wait();
    float s = 0.f;
    // stretch k lies in share k % shares; a token with more stretches than shares has keys in every share
    const int k_lo = first / split_keys, k_hi = min(pos / split_keys, k_lo + shares - 1);
    for (int k = k_lo; k <= k_hi; ++k) s += part[(size_t)(k % shares) * count + i];
    out[i] = from_float<TO>(s);
}

// What a token's stacked projections become before they are queries and keys.  proj row: [Hq x D | Hk x D | Hk x V | ...].
//   norm:    the whole query projection (all heads at once) is divided by sqrt(mean(x^2) + eps) and multiplied by qw,
//            the whole key projection likewise by kw (qw == null: no norms)
//   rotate:  in every head, lanes i and i + rot/2 (i < rot/2) turn by position * freq[i]; lanes >= rot pass
//   keys:    times k_scale
//   queries go to q_out [N, Hq * D]; keys to k_out [N, Hk * D], or with the values into the token's slot of
//   pool [pages, 2, Hk, page_size, Dp].  One CTA per token.
template <typename TI, typename TQ, typename TK>
__global__ void __launch_bounds__(256)
qk_prepare_kernel(const TI* __restrict__ proj, int ldp, TQ* __restrict__ q_out, int ldq, TK* __restrict__ k_out, int ldk,
                  TK* __restrict__ pool, const int* __restrict__ slot_map, int page_size, int Dp, const float* __restrict__ qw,
                  const float* __restrict__ kw, float eps, const float* __restrict__ freq, int rot,
                  const int* __restrict__ positions, float k_scale, int Hq, int Hk, int D, int V) {
    extern __shared__ float2 turn[];  // (cos, sin) of the token's angles
    __shared__ float scratch[33];
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = rot >> 1;
    const float position = half > 0 ? (float)positions[t] : 0.f;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(position * freq[i], &s, &c);
        turn[i] = make_float2(c, s);
    }
    const int slot = pool ? slot_map[t] : 0;
    pdl_wait();
    const TI* row = proj + (size_t)t * ldp;
    float q_scale = 1.f, kn_scale = 1.f;
    if (qw) {
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < Hq * D; i += blockDim.x) { const float v = to_float(row[i]); sq = fmaf(v, v, sq); }
        for (int i = threadIdx.x; i < Hk * D; i += blockDim.x) { const float v = to_float(row[Hq * D + i]); sk = fmaf(v, v, sk); }
        sq = block_sum(sq, scratch);
        sk = block_sum(sk, scratch);
        q_scale = 1.f / sqrtf(sq / (float)(Hq * D) + eps);
        kn_scale = 1.f / sqrtf(sk / (float)(Hk * D) + eps);
    }
    __syncthreads();
    const int per_head = D - half;  // work items a head: `half` pairs, then the lanes that pass
    const int page = slot / page_size, off = slot % page_size;
    for (int it = threadIdx.x; it < (Hq + Hk) * per_head; it += blockDim.x) {
        const int head = it / per_head, i = it % per_head;
        const bool is_q = head < Hq;
        const int base = head * D;  // keys follow the queries in the row
        const float* w = is_q ? qw : kw;
        const int wbase = is_q ? base : base - Hq * D;
        const float ns = is_q ? q_scale : kn_scale, post = is_q ? 1.f : k_scale;
        float a, b = 0.f;
        int da, db = -1;
        if (i < half) {
            da = i; db = i + half;
            float u = to_float(row[base + da]) * ns, v = to_float(row[base + db]) * ns;
            if (w) { u *= w[wbase + da]; v *= w[wbase + db]; }
            const float c = turn[i].x, s = turn[i].y;
            a = (u * c - v * s) * post;
            b = (v * c + u * s) * post;
        } else {
            da = i + half;
            float u = to_float(row[base + da]) * ns;
            if (w) u *= w[wbase + da];
            a = u * post;
        }
        if (is_q) {
            TQ* dst = q_out + (size_t)t * ldq + base;
            dst[da] = from_float<TQ>(a);
            if (db >= 0) dst[db] = from_float<TQ>(b);
        } else {
            const int kh = head - Hq;
            TK* dst = pool ? pool + (((size_t)page * 2 * Hk + kh) * page_size + off) * Dp : k_out + (size_t)t * ldk + (size_t)kh * D;
            dst[da] = from_float<TK>(a);
            if (db >= 0) dst[db] = from_float<TK>(b);
        }
    }
    if (pool) {
        const TI* vals = row + (size_t)(Hq + Hk) * D;
        for (int i = threadIdx.x; i < Hk * V; i += blockDim.x) {
            const int kh = i / V, d = i % V;
            pool[((((size_t)page * 2 + 1) * Hk + kh) * page_size + off) * Dp + d] = from_float<TK>(to_float(vals[i]));
        }
    }
}

}  // namespace

LLM_EXPORT int llm_sigmoid_attention(const void* q, int q_dtype, int ldq, const void* pool, int pool_dtype,
                                     const int* page_table, int table_width, const int* positions, const int* token_request,
                                     const float* bias, const float* mix, void* out, int out_dtype, float* parts, int N, int H,
                                     int KV, int D, int V, int Dp, int page_size, float scale, float cap, int window,
                                     int split_keys, int splits, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || KV <= 0 || H % KV || D <= 0 || V <= 0 || V > 256 || Dp < D || Dp < V || splits < 1 || split_keys < CHUNK ||
        split_keys % CHUNK || splits > 65535 || (splits > 1 && !parts) || q_dtype != pool_dtype || out_dtype != q_dtype)
        return LLM_ERR_BAD_ARGUMENT;
    if (splits == 1) split_keys = 1 << 30;  // one CTA sums up all of a token's keys
    const int warps = H < 32 ? H : 32;
    const size_t smem = ((size_t)H * D + (size_t)H * CHUNK + (mix ? (size_t)32 * H : 0)) * sizeof(float);
    if (smem > 200 * 1024) return LLM_ERR_UNSUPPORTED;
    const dim3 grid(N, (H + 31) / 32, splits), block(32 * warps);
    void* dst = splits > 1 ? (void*)parts : out;
    using bf = __nv_bfloat16;
    auto go = [&](auto kernel, auto* qp, auto* pp) -> int {
        if (smem > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        return launch_pdl(kernel, grid, block, smem, stream, qp, ldq, pp, page_table, table_width, positions, token_request, bias,
                          mix, dst, N, H, KV, D, V, Dp, page_size, scale, cap, window, split_keys, splits);
    };
    int code;
    const int vpl = (V + 31) / 32;
#define LLM_SIGATT(VPL)                                                                                             \
    (q_dtype == LLM_F32 ? go(sigmoid_attention_kernel<float, float, float, VPL>, (const float*)q, (const float*)pool) \
                        : go(sigmoid_attention_kernel<bf, bf, bf, VPL>, (const bf*)q, (const bf*)pool))
    if (vpl <= 1) code = LLM_SIGATT(1);
    else if (vpl <= 2) code = LLM_SIGATT(2);
    else if (vpl <= 4) code = LLM_SIGATT(4);
    else code = LLM_SIGATT(8);
#undef LLM_SIGATT
    if (code != 0 || splits == 1) return code;
    const size_t count = (size_t)N * H * V;
    const dim3 g2((unsigned)((count + 255) / 256));
    if (out_dtype == LLM_F32)
        return launch_pdl(sum_parts_kernel<float>, g2, dim3(256), 0, stream, (const float*)parts, (float*)out, positions, H * V, count, split_keys, window, splits);
    return launch_pdl(sum_parts_kernel<bf>, g2, dim3(256), 0, stream, (const float*)parts, (bf*)out, positions, H * V, count, split_keys, window, splits);
}

// out[t, :] = the sum of parts[s][t, :] over the stretches s in which token t has keys, in their order.
LLM_EXPORT int llm_sigmoid_sum_parts(const float* parts, void* out, int out_dtype, const int* positions, int N, int row, int split_keys,
                                     int window, int shares, cudaStream_t stream) {
    if (N <= 0 || row <= 0) return 0;
    const size_t count = (size_t)N * row;
    const dim3 grid((unsigned)((count + 255) / 256));
    if (out_dtype == LLM_F32) return launch_pdl(sum_parts_kernel<float>, grid, dim3(256), 0, stream, parts, (float*)out, positions, row, count, split_keys, window, shares);
    return launch_pdl(sum_parts_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, parts, (__nv_bfloat16*)out, positions, row, count, split_keys, window, shares);
}

// in_dtype: the projections' type; q_dtype: the queries' type on their way out; k_dtype: the keys' (and the pool's).
LLM_EXPORT int llm_qk_prepare(const void* proj, int in_dtype, int ldp, void* q_out, int q_dtype, int ldq, void* k_out, int ldk,
                              void* pool, int k_dtype, const int* slot_map, int page_size, int Dp, const float* qw, const float* kw,
                              float eps, const float* freq, int rot, const int* positions, float k_scale, int N, int Hq, int Hk,
                              int D, int V, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (rot < 0 || rot % 2 || rot > D || Hq < 0 || Hk < 0 || (!pool && !k_out && Hk > 0) || (pool && (Dp < D || Dp < V || !slot_map)) ||
        (rot > 0 && (!freq || !positions)) || ((qw == nullptr) != (kw == nullptr)))
        return LLM_ERR_BAD_ARGUMENT;
    using bf = __nv_bfloat16;
    const size_t smem = (size_t)(rot / 2 + 1) * sizeof(float2);
    auto go = [&](auto kernel, auto* in, auto* qo, auto* ko) {
        using TK = std::remove_pointer_t<decltype(ko)>;
        return launch_pdl(kernel, dim3(N), dim3(256), smem, stream, in, ldp, qo, ldq, ko, ldk, (TK*)pool, slot_map, page_size, Dp, qw, kw,
                          eps, freq, rot, positions, k_scale, Hq, Hk, D, V);
    };
    if (in_dtype == LLM_F32 && q_dtype == LLM_F32 && k_dtype == LLM_F32)
        return go(qk_prepare_kernel<float, float, float>, (const float*)proj, (float*)q_out, (float*)k_out);
    if (in_dtype == LLM_F32 && q_dtype == LLM_BF16 && k_dtype == LLM_BF16)
        return go(qk_prepare_kernel<float, bf, bf>, (const float*)proj, (bf*)q_out, (bf*)k_out);
    if (in_dtype == LLM_BF16 && q_dtype == LLM_BF16 && k_dtype == LLM_BF16)
        return go(qk_prepare_kernel<bf, bf, bf>, (const bf*)proj, (bf*)q_out, (bf*)k_out);
    return LLM_ERR_UNSUPPORTED;
}
