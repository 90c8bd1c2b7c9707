// Sigmoid attention with mixed heads (see sigmoid_attention.cu for the mechanism) on the tensor cores, for prompt portions
// in bfloat16.
//
// A CTA owns 16 consecutive query tokens of one request and up to 16 output heads, and walks the keys in tiles of BN.
// Per tile:
//   1. scores of ALL heads (the mixing needs every head's weight of a pair): S_g = Q_g K_c(g)^T by mma.sync m16n8k16,
//      warp w taking heads w, w + W, ...; scale, cap, bias, sigmoid and the causal mask in 32-bit; weights to shared
//      memory as float32
//   2. the mixing w_h = sum_g mix[h, g] p_g in 32-bit on the CUDA cores, a thread holding 8 heads x 2 pairs in
//      registers; the mixed weights go back to shared memory as bfloat16
//   3. O_h += W_h V_c(h) by mma.sync, one warp per output head, accumulators in registers over all key tiles
// Keys and values come through cp.async; the next tile's keys are asked for as soon as the scores are done.
#include "attention_tile.cuh"

namespace {

using namespace attn;

constexpr int BM = 16;   // query tokens a CTA
constexpr int HB = 16;   // output heads a CTA
constexpr int THREADS = 512;
constexpr int MAX_SHARES = 16;  // CTAs that share a tile's keys: stretch s goes to CTA s % 16, so that a step whose grid is made for the
                                // longest context a pool allows does not launch hundreds of CTAs without keys

struct SigMmaParams {
    const __nv_bfloat16* q;
    int ldq;
    const __nv_bfloat16* pool;
    const int *page_table, *positions, *cu_tokens;
    int table_width;
    const float *bias, *mix;
    __nv_bfloat16* out;
    float* parts;  // [grid.z][N][H * V] partial sums when the keys are shared out over several CTAs (else null)
    int N, R, H, KV, D, V, Dp, page_size, window, split_keys, splits;
    float scale, cap;
};

template <int NV8, int BN>
__global__ void __launch_bounds__(THREADS)
sigmoid_attention_mma_kernel(const SigMmaParams p) {
    using bf = __nv_bfloat16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int tile_info[2];
    const int H = p.H, KV = p.KV, D = p.D, group = H / KV;
    constexpr int V = NV8 * 8;
    const int DQ = D + 8, VQ = V + 8;
    constexpr int PP = BN + 4;  // pitch of a row of float32 weights
    constexpr int WP = BN + 8;  // pitch of a row of bfloat16 mixed weights
    bf* sQ = reinterpret_cast<bf*>(smem_raw);                  // [H][BM][DQ]
    bf* sK = sQ + (size_t)H * BM * DQ;                         // [KV][BN][DQ]
    bf* sV = sK + (size_t)KV * BN * DQ;                        // [KV][BN][VQ]
    float* sP = reinterpret_cast<float*>(sV + (size_t)KV * BN * VQ);  // [H][BM][PP]
    bf* sW = reinterpret_cast<bf*>(sP);                        // [HB][BM][WP], over the weights once they are mixed
    const size_t weights_bytes = max((size_t)H * BM * PP * 4, (size_t)HB * BM * WP * 2);
    float* sT = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(sP) + weights_bytes);  // [H][HB]: sT[g][hl] = mix[hb * HB + hl][g]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, W = THREADS / 32;
    const int hb = blockIdx.y, split = blockIdx.z;
    pdl_trigger();
    // which request and which of its tiles: the tiles of the requests lie one after the other
    if (tid == 0) {
        int rest = gridDim.x - 1 - blockIdx.x, r = 0;  // the last tiles of a request see the most keys: they start first
        for (; r < p.R; ++r) {
            const int tiles = (p.cu_tokens[r + 1] - p.cu_tokens[r] + BM - 1) / BM;
            if (rest < tiles) break;
            rest -= tiles;
        }
        tile_info[0] = r;
        tile_info[1] = rest;
    }
    for (int i = tid; i < H * HB; i += THREADS) {
        const int g = i / HB, h = hb * HB + i % HB;
        sT[i] = h < H ? (p.mix ? p.mix[(size_t)h * H + g] : (h == g ? 1.f : 0.f)) : 0.f;
    }
    __syncthreads();
    const int r = tile_info[0];
    if (r >= p.R) return;
    const int t0 = p.cu_tokens[r] + tile_info[1] * BM;
    const int rows = min(BM, p.cu_tokens[r + 1] - t0);
    const int pos0 = p.positions[t0];  // the tile's tokens stand at pos0, pos0 + 1, ...
    const int* table = p.page_table + (size_t)r * p.table_width;
    const size_t plane = (size_t)KV * p.page_size * p.Dp;
    // the keys that any row of the tile sees; this CTA takes the stretches split, split + gridDim.z, ... of them
    const int tile_first = p.window > 0 ? max(0, pos0 - p.window + 1) : 0, tile_last = pos0 + rows - 1;
    {
        bool any = false;
        for (int s = split; s < p.splits && !any; s += gridDim.z)
            any = max(tile_first, s * p.split_keys) <= min(tile_last, (s + 1) * p.split_keys - 1);
        if (!any) return;  // the sum reads only the partial sums of CTAs that had keys
    }
    int first = 0, last = -1;  // of the stretch at hand
    pdl_wait();
    // the tile's queries, every head: 16 bytes a thread and turn; rows beyond the request's tokens are zeros
    {
        const int chunks = D / 8;
        for (int i = tid; i < H * BM * chunks; i += THREADS) {
            const int ch = i % chunks, row = (i / chunks) % BM, g = i / (chunks * BM);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < rows) v = *reinterpret_cast<const uint4*>(p.q + (size_t)(t0 + row) * p.ldq + (size_t)g * D + ch * 8);
            *reinterpret_cast<uint4*>(sQ + ((size_t)g * BM + row) * DQ + ch * 8) = v;
        }
    }

    // a thread copies the same 16 bytes of a key's row for every key/value head: one look at the page table a row
    auto load_rows = [&](int j0, bf* dst, int pitch, int chunks, size_t second_plane, int c_lo, int c_hi) {
        for (int i = tid; i < BN * chunks; i += THREADS) {
            const int jj = i / chunks, ch = i - jj * chunks;
            const int j = j0 + jj;
            const bool ok = j <= last;
            const bf* src = p.pool;
            if (ok) src += (size_t)table[j / p.page_size] * 2 * plane + second_plane + (size_t)(j % p.page_size) * p.Dp + ch * 8;
            bf* to = dst + (size_t)jj * pitch + ch * 8;
            for (int c = c_lo; c <= c_hi; ++c) cp_async16(to + (size_t)c * BN * pitch, ok ? src + (size_t)c * p.page_size * p.Dp : src, ok);
        }
    };
    // keys of every key/value head (the scores of all heads are wanted); values only of the heads behind this CTA's output heads
    const int v_lo = (hb * HB) / group, v_hi = min(H - 1, hb * HB + HB - 1) / group;
    auto load_keys = [&](int j0) { load_rows(j0, sK, DQ, D / 8, 0, 0, KV - 1); };
    auto load_values = [&](int j0) { load_rows(j0, sV, VQ, V / 8, plane, v_lo, v_hi); };

    float O[NV8][4];
#pragma unroll
    for (int n = 0; n < NV8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) O[n][e] = 0.f;
    const float inv_cap = p.cap > 0.f ? 1.f / p.cap : 0.f;
    const int h_out = hb * HB + warp;          // the output head of this warp (phase 3)
    const bool has_out = warp < HB && h_out < H;
    const int c_out = has_out ? h_out / group : 0;
    // mixing: a thread owns 2 neighbouring pairs of one row and 8 output heads
    constexpr int SLOTS = BM * BN / 2;
    const int slot = tid % SLOTS, oct = tid / SLOTS;  // oct 0, 1: heads 0..7, 8..15 of the block; beyond: idle
    const int mi = slot / (BN / 2), mj = (slot % (BN / 2)) * 2;
    const bool mixes = oct < 2;
    const bool mix_row = mixes && mi < rows;  // rows beyond the request's tokens keep weights of zero

    for (int stretch = split; stretch < p.splits; stretch += gridDim.z) {
    first = max(tile_first, stretch * p.split_keys);
    last = min(tile_last, (stretch + 1) * p.split_keys - 1);
    if (first > last) continue;
    const int j_begin = (first / BN) * BN;
    load_keys(j_begin);
    load_values(j_begin);
    cp_async_commit();
    for (int j0 = j_begin; j0 <= last; j0 += BN) {
        cp_async_wait<0>();
        __syncthreads();  // (A) this tile's keys and values have landed; everybody is done with the tile before
        // ---- 1. scores and weights of every head
        for (int g = warp; g < H; g += W) {
            float S[BN / 8][4];
#pragma unroll
            for (int n = 0; n < BN / 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) S[n][e] = 0.f;
            const bf* qg = sQ + (size_t)g * BM * DQ;
            const bf* kc = sK + (size_t)(g / group) * BN * DQ;
            for (int ks = 0; ks < D / 16; ++ks) {
                unsigned a[4];
                ldmatrix_x4(a, qg + (size_t)(lane & 15) * DQ + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int np = 0; np < BN / 16; ++np) {
                    unsigned b[4];
                    ldmatrix_x4(b, kc + (size_t)(np * 16 + (lane & 7) + (lane >> 4) * 8) * DQ + ks * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(S[2 * np], a, b[0], b[1]);
                    mma_bf16(S[2 * np + 1], a, b[2], b[3]);
                }
            }
            // cap * tanh(x / cap) = cap * (1 - 2 / (1 + 2^(x c1))) with c1 = 2 log2(e) / cap, the sigmoid 1 / (1 + 2^(-y log2 e)):
            // two ex2.approx and two rcp.approx a weight (relative error about 2^-22 each), everything else folded into constants
            const float bg = p.bias ? p.bias[g] : 0.f;
            const float LOG2E = 1.4426950408889634f;
            const float c1 = p.scale * 2.f * inv_cap * LOG2E, c2 = -p.scale * LOG2E, nb = -bg * LOG2E, ncap = -p.cap * LOG2E;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int i = (lane >> 2) + half * 8;
                const int pos = pos0 + i;
                const int hi = i < rows ? min(pos, last) : -1;
                const int lo = max(p.window > 0 ? max(0, pos - p.window + 1) : 0, first);
                if (hi < max(lo, j0)) {  // a row without a key in this tile (one beyond the request's tokens, as most rows of a decode step's tile)
#pragma unroll
                    for (int n = 0; n < BN / 8; ++n)
                        *reinterpret_cast<float2*>(sP + ((size_t)g * BM + i) * PP + n * 8 + (lane & 3) * 2) = make_float2(0.f, 0.f);
                    continue;
                }
#pragma unroll
                for (int n = 0; n < BN / 8; ++n) {
                    float w2[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int j = j0 + n * 8 + (lane & 3) * 2 + e;
                        const float sc = S[n][half * 2 + e];
                        float y;  // -(capped score + bias) * log2(e)
                        if (p.cap > 0.f) {
                            const float t = 1.f - __fdividef(2.f, 1.f + fast_exp2(fminf(sc * c1, 100.f)));
                            y = fmaf(ncap, t, nb);
                        } else {
                            y = fmaf(sc, c2, nb);
                        }
                        const float w = __fdividef(1.f, 1.f + fast_exp2(fminf(y, 100.f)));
                        w2[e] = (j <= hi && j >= lo) ? w : 0.f;
                    }
                    *reinterpret_cast<float2*>(sP + ((size_t)g * BM + i) * PP + n * 8 + (lane & 3) * 2) = make_float2(w2[0], w2[1]);
                }
            }
        }
        __syncthreads();  // (B) every head's weights are in shared memory; nobody reads the keys any more
        if (j0 + BN <= last) load_keys(j0 + BN);
        cp_async_commit();
        // ---- 2. the heads' weights mixed, in 32-bit
        float m[8][2];
#pragma unroll
        for (int k = 0; k < 8; ++k) m[k][0] = m[k][1] = 0.f;
        if (mix_row) {
            const float* pp = sP + (size_t)mi * PP + mj;
            const float* tt = sT + oct * 8;
            for (int g = 0; g < H; ++g) {
                const float2 pv = *reinterpret_cast<const float2*>(pp + (size_t)g * BM * PP);
                const float4 ta = *reinterpret_cast<const float4*>(tt + g * HB), tb = *reinterpret_cast<const float4*>(tt + g * HB + 4);
                const float tv[8] = {ta.x, ta.y, ta.z, ta.w, tb.x, tb.y, tb.z, tb.w};
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    m[k][0] = fmaf(tv[k], pv.x, m[k][0]);
                    m[k][1] = fmaf(tv[k], pv.y, m[k][1]);
                }
            }
        }
        __syncthreads();  // (C) all reads of the unmixed weights are done: the mixed ones may take their place
        if (mixes) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                *reinterpret_cast<unsigned*>(sW + ((size_t)(oct * 8 + k) * BM + mi) * WP + mj) = pack_bf16(m[k][0], m[k][1]);
        }
        __syncthreads();  // (D)
        // ---- 3. the output heads' sums over the tile's values
        if (has_out) {
            const bf* wh = sW + (size_t)warp * BM * WP;
            const bf* vc = sV + (size_t)c_out * BN * VQ;
#pragma unroll
            for (int ks = 0; ks < BN / 16; ++ks) {
                unsigned a[4];
                ldmatrix_x4(a, wh + (size_t)(lane & 15) * WP + ks * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int np = 0; np < NV8 / 2; ++np) {
                    unsigned b[4];
                    ldmatrix_x4_trans(b, vc + (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VQ + np * 16 + (lane >> 4) * 8);
                    mma_bf16(O[2 * np], a, b[0], b[1]);
                    mma_bf16(O[2 * np + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();  // (E) nobody reads this tile's values any more
        if (j0 + BN <= last) load_values(j0 + BN);
        cp_async_commit();
    }
    cp_async_wait<0>();
    }  // stretches
    if (!has_out) return;
#pragma unroll
    for (int n = 0; n < NV8; ++n)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int i = (lane >> 2) + half * 8;
            if (i >= rows) continue;
            const size_t at = (size_t)(t0 + i) * H * V + (size_t)h_out * V + n * 8 + (lane & 3) * 2;
            if (p.splits > 1)
                *reinterpret_cast<float2*>(p.parts + (size_t)split * p.N * H * V + at) = make_float2(O[n][half * 2], O[n][half * 2 + 1]);
            else
                *reinterpret_cast<unsigned*>(p.out + at) = pack_bf16(O[n][half * 2], O[n][half * 2 + 1]);
        }
}

template <int NV8, int BN>
int launch(const SigMmaParams& p, int tiles, size_t smem, cudaStream_t stream) {
    auto kernel = sigmoid_attention_mma_kernel<NV8, BN>;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(kernel, dim3(tiles, (p.H + HB - 1) / HB, p.splits < MAX_SHARES ? p.splits : MAX_SHARES), dim3(THREADS), smem, stream, p);
}

size_t smem_bytes(int H, int KV, int D, int V, int BN) {
    const size_t plain = (size_t)H * BM * (BN + 4) * 4, mixed = (size_t)HB * BM * (BN + 8) * 2;  // the mixed weights lie over the plain ones
    return (size_t)H * BM * (D + 8) * 2 + (size_t)KV * BN * (D + 8) * 2 + (size_t)KV * BN * (V + 8) * 2 + (plain > mixed ? plain : mixed) +
           (size_t)H * HB * 4;
}

}  // namespace

// `tiles`: the sum over the requests of ceil(tokens / 16).  Returns LLM_ERR_UNSUPPORTED for sizes it does not take
// (lanes that are no multiples of 16, values wider than 128 lanes, heads that do not fit the shared memory).
// `splits` > 1: the keys are shared out in stretches of `split_keys` (a multiple of 32), stretch s to share s % shares with
// shares = min(splits, 16), and the partial sums left in `parts [shares][N][H * V]` for llm_sigmoid_sum_parts.
LLM_EXPORT int llm_sigmoid_attention_mma(const void* q, int ldq, const void* pool, const int* page_table, int table_width,
                                         const int* positions, const int* cu_tokens, const float* bias, const float* mix, void* out,
                                         float* parts, int tiles, int N, int R, int H, int KV, int D, int V, int Dp, int page_size,
                                         float scale, float cap, int window, int split_keys, int splits, cudaStream_t stream) {
    if (tiles <= 0) return 0;
    if (H <= 0 || KV <= 0 || H % KV || Dp < D || Dp < V || splits < 1 || splits > 65535 || (splits > 1 && (!parts || split_keys % 32 || split_keys < 32)))
        return LLM_ERR_BAD_ARGUMENT;
    if (splits == 1) split_keys = 1 << 30;
    if (D % 16 || V % 16 || V > 128 || D > 256 || Dp % 8 || ldq % 8 || tiles > 1 << 30) return LLM_ERR_UNSUPPORTED;
    const size_t limit = 227 * 1024 - 64;
    int bn = 32;
    if (smem_bytes(H, KV, D, V, bn) > limit) bn = 16;
    const size_t smem = smem_bytes(H, KV, D, V, bn);
    if (smem > limit) return LLM_ERR_UNSUPPORTED;
    SigMmaParams p{(const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)pool, page_table, positions, cu_tokens, table_width, bias, mix,
                   (__nv_bfloat16*)out, parts, N, R, H, KV, D, V, Dp, page_size, window, split_keys, splits, scale, cap};
#define LLM_SIGMMA(NV8) (bn == 32 ? launch<NV8, 32>(p, tiles, smem, stream) : launch<NV8, 16>(p, tiles, smem, stream))
    switch (V / 16) {
        case 1: return LLM_SIGMMA(2);
        case 2: return LLM_SIGMMA(4);
        case 3: return LLM_SIGMMA(6);
        case 4: return LLM_SIGMMA(8);
        case 5: return LLM_SIGMMA(10);
        case 6: return LLM_SIGMMA(12);
        case 7: return LLM_SIGMMA(14);
        default: return LLM_SIGMMA(16);
    }
#undef LLM_SIGMMA
}
