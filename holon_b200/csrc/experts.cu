// Routed experts: the router's choice, the layout of (token, choice) pairs expert by expert, the experts' products
// over those rows, and the weighted sum back per token. Nothing is decided on the host: the number of rows an expert
// gets is only known on the device, so the products launch the most tiles the step can need and a tile that finds no
// rows returns at once.
//
// hb_route_top       z [tokens, ld] (32-bit logits) -> chosen [tokens, top], weight [tokens, top], counts[e] += 1
// hb_expert_rows     counts -> first row of every expert; place[pair] = its row, token_of[row] = its token
// hb_expert_linear   out[row] = act(x[token_of ? token_of[row] : row] · w[e(row)]ᵀ), any dtype, CUDA cores
// hb_expert_combine  out[t] = sum_k weight[t, k] · y[place[t, k]] (+ sigmoid(gate_t) · shared[t]); rows of identity experts read x[t]
#include "common.cuh"

// ---------------------------------------------------------------- the router's choice
// One block per token. softmax over all experts in 32-bit; the `top` largest scores, equal scores by ascending
// expert; weight = score · scale, with `renormalize` divided by the chosen scores' sum first.
__global__ void route_top_kernel(int32_t* __restrict__ chosen, float* __restrict__ weight, int32_t* __restrict__ counts,
                                 const float* __restrict__ z, int ld, int experts, int top, float scale, int renormalize,
                                 const float* __restrict__ bias) {
    extern __shared__ float sc[];                       // experts scores
    __shared__ float scratch[33];
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const float* zr = z + (size_t)t * ld;
    float m = -INFINITY;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) m = fmaxf(m, zr[e] + (bias ? bias[e] : 0.f));
    m = block_max(m, scratch);
    float sum = 0.f;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) { const float p = expf(zr[e] + (bias ? bias[e] : 0.f) - m); sc[e] = p; sum += p; }
    sum = block_sum(sum, scratch);
    const float inv = 1.f / sum;
    float taken = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -1.f; int bi = 0x7fffffff;
        for (int e = threadIdx.x; e < experts; e += blockDim.x) {
            const float v = sc[e];
            if (v > bv) { bv = v; bi = e; }              // (ascending e: the first of equals stays)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < warps; ++w)
                if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
            chosen[(size_t)t * top + k] = bi;
            weight[(size_t)t * top + k] = bv * inv;
            sc[bi] = -2.f;                               // out of the running
            atomicAdd(counts + bi, 1);
            taken += bv * inv;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const float f = renormalize ? scale / taken : scale;
        for (int k = 0; k < top; ++k) weight[(size_t)t * top + k] *= f;
    }
}

// The choice with a correction and in groups, one warp per token. sc [experts] holds the token's exponentials, inv one
// over their sum; ch [experts] and gm [groups] are scratch of this warp. The choice runs on s + correction (which may be
// negative: what is out of the running is minus infinity); with `groups` > 1 the experts form that many equal groups of
// neighbours, a group counts by its best choice score, and only the `keep` best groups (equal ones by ascending group)
// stay in the running. The weights are the chosen experts' s, with `renormalize` divided by their sum + tiny.
__device__ __forceinline__ void route_choice_warp(int lane, const float* sc, float* ch, float* gm, float inv,
                                                  const float* __restrict__ correction, int experts, int top, int groups,
                                                  int keep, int32_t* chosen, float* weight, int* cnt, float scale,
                                                  int renormalize, float tiny) {
    for (int e = lane; e < experts; e += 32) ch[e] = sc[e] * inv + (correction ? correction[e] : 0.f);
    __syncwarp();
    if (groups > 1) {
        const int per = experts / groups;
        for (int g = lane; g < groups; g += 32) {
            float m = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) m = fmaxf(m, ch[e]);
            gm[g] = m;
        }
        __syncwarp();
        for (int r = 0; r < keep; ++r) {                     // a kept group is marked by plus infinity
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float v = gm[g];
                if (v != INFINITY && (v > bv || (v == bv && g < bi))) { bv = v; bi = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
            }
            if (lane == 0 && bi != 0x7fffffff) gm[bi] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32) if (gm[e / per] != INFINITY) ch[e] = -INFINITY;
        __syncwarp();
    }
    float taken = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = ch[e];
            if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        const float share = sc[bi] * inv;
        if (lane == 0) {
            chosen[k] = bi;
            weight[k] = share;
            ch[bi] = -INFINITY;
            atomicAdd(cnt + bi, 1);
        }
        taken += share;
        __syncwarp();
    }
    const float f = renormalize ? scale / (taken + tiny) : scale;
    for (int k = lane; k < top; k += 32) weight[k] *= f;
}

// hb_route_top with a correction or groups: a warp a token, eight tokens a block; shared memory 3 x 8 x experts floats.
__global__ void __launch_bounds__(256) route_choice_kernel(int32_t* __restrict__ chosen, float* __restrict__ weight,
                                                           int32_t* __restrict__ counts, const float* __restrict__ z, int ld,
                                                           int tokens, int experts, int top, float scale, int renormalize,
                                                           const float* __restrict__ bias, const float* __restrict__ correction,
                                                           int groups, int keep, float tiny) {
    extern __shared__ float rc_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 8 + warp;
    if (t >= tokens) return;
    float* my = rc_smem + (size_t)warp * experts;
    float* ch = rc_smem + (size_t)(8 + warp) * experts;
    float* gm = rc_smem + (size_t)(16 + warp) * experts;
    const float* zr = z + (size_t)t * ld;
    float m = -INFINITY;
    for (int e = lane; e < experts; e += 32) m = fmaxf(m, zr[e] + (bias ? bias[e] : 0.f));
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) { const float p = expf(zr[e] + (bias ? bias[e] : 0.f) - m); my[e] = p; sum += p; }
    sum = warp_sum(sum);
    __syncwarp();
    route_choice_warp(lane, my, ch, gm, 1.f / sum, correction, experts, top, groups, keep, chosen + (size_t)t * top,
                      weight + (size_t)t * top, counts, scale, renormalize, tiny);
}

extern "C" int hb_route_top(int32_t* chosen, float* weight, int32_t* counts, const float* z, const float* bias, int ld,
                            int tokens, int experts, int top, float scale, int renormalize, const float* correction,
                            int groups, int keep, float tiny, hb_stream stream) {
    if (tokens == 0) return 0;
    if (experts < 1 || top < 1 || top > experts || ld < experts) HB_REFUSE("route_top: top %d of %d experts in rows of %d", top, experts, ld);
    if (experts > 8192) HB_REFUSE("route_top: %d experts are above 8192", experts);
    if (groups < 1 || experts % groups || keep < 1 || keep > groups || (long)keep * (experts / groups) < top)
        HB_REFUSE("route_top: %d groups of which %d are kept, for top %d of %d experts", groups, keep, top, experts);
    if (correction || groups > 1 || tiny != 0.f) {
        const size_t smem = (size_t)24 * experts * sizeof(float);
        if (smem > 200 * 1024) HB_REFUSE("route_top: a choice in groups takes up to 2133 experts, not %d", experts);
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(route_choice_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        route_choice_kernel<<<(tokens + 7) / 8, 256, smem, (cudaStream_t)stream>>>(chosen, weight, counts, z, ld, tokens, experts, top,
                                                                                  scale, renormalize, bias, correction, groups, keep, tiny);
        HB_LAUNCH_CHECK("route_choice");
        return 0;
    }
    const int threads = experts > 256 ? 256 : experts > 64 ? 128 : 64;
    route_top_kernel<<<tokens, threads, (size_t)experts * sizeof(float), (cudaStream_t)stream>>>(
        chosen, weight, counts, z, ld, experts, top, scale, renormalize, bias);
    HB_LAUNCH_CHECK("route_top");
    return 0;
}

// ---------------------------------------------------------------- rows expert by expert
// counts [2 experts + 1]: [0, experts) the tokens of each expert (from hb_route_top), [experts, 2 experts] receives the
// first row of each expert and the end. The counts are used as cursors meanwhile and hold the counts again afterwards.
__global__ void expert_starts_kernel(int32_t* counts, int experts) {
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int e0 = 0; e0 < experts; e0 += blockDim.x) {          // a block-wide scan, a stretch of blockDim.x at a time
        const int e = e0 + threadIdx.x;
        const int c = e < experts ? counts[e] : 0;
        int v = c;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        __shared__ int sums[32];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, v, o); if (lane >= o) v += u; }
        if (lane == 31) sums[warp] = v;
        __syncthreads();
        if (warp == 0) {
            int w = lane < (int)(blockDim.x >> 5) ? sums[lane] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, w, o); if (lane >= o) w += u; }
            sums[lane] = w;
        }
        __syncthreads();
        const int before = carry + (warp ? sums[warp - 1] : 0) + v - c;
        if (e < experts) { counts[experts + e] = before; counts[e] = 0; }
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + c;
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[2 * experts] = carry;
}

__global__ void expert_scatter_kernel(int32_t* __restrict__ place, int32_t* __restrict__ token_of, int32_t* counts,
                                      const int32_t* __restrict__ chosen, int pairs, int top, int experts) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pairs) return;
    const int e = chosen[i];
    if (e < 0 || e >= experts) { place[i] = -1; return; }
    const int p = counts[experts + e] + atomicAdd(counts + e, 1);
    place[i] = p;
    token_of[p] = i / top;
}

extern "C" int hb_expert_rows(int32_t* place, int32_t* token_of, int32_t* counts, const int32_t* chosen, int tokens,
                              int top, int experts, hb_stream stream) {
    if (tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    expert_starts_kernel<<<1, 256, 0, s>>>(counts, experts);
    HB_LAUNCH_CHECK("expert_starts");
    const int pairs = tokens * top;
    expert_scatter_kernel<<<(pairs + 255) / 256, 256, 0, s>>>(place, token_of, counts, chosen, pairs, top, experts);
    HB_LAUNCH_CHECK("expert_scatter");
    return 0;
}

// ---------------------------------------------------------------- choice and rows in one launch (few tokens)
// One CTA of eight warps does what hb_route_top and hb_expert_rows do for up to RS_TOKENS tokens and RS_EXPERTS
// experts: a warp routes a token at a time; counts, first rows and the pairs' rows are worked out in shared memory.
// counts [2 experts + 3] is written whole: counts, first rows, the end, and the pair (0, tokens), which serves as the
// `starts` of one expert that takes every token (the shared expert's product with its activation).
#define RS_TOKENS 256
#define RS_EXPERTS 1024
__global__ void __launch_bounds__(256) route_rows_small_kernel(int32_t* __restrict__ chosen, float* __restrict__ weight,
                                                               int32_t* __restrict__ counts, int32_t* __restrict__ place,
                                                               int32_t* __restrict__ token_of, const float* __restrict__ z,
                                                               int ld, int tokens, int experts, int top, float scale,
                                                               int renormalize, const float* __restrict__ bias,
                                                               const float* __restrict__ correction, int groups, int keep,
                                                               float tiny, int grouped) {
    extern __shared__ float rs_smem[];
    float* sc = rs_smem;                                   // [8][experts]
    int* cnt = (int*)(sc + 8 * (size_t)experts);           // [experts]: counts, then cursors
    int* start = cnt + experts;                            // [experts + 1]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    float* my = sc + (size_t)warp * experts;
    for (int t = warp; t < tokens; t += 8) {
        const float* zr = z + (size_t)t * ld;
        float m = -INFINITY;
        for (int e = lane; e < experts; e += 32) m = fmaxf(m, zr[e] + (bias ? bias[e] : 0.f));
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < experts; e += 32) { const float p = expf(zr[e] + (bias ? bias[e] : 0.f) - m); my[e] = p; sum += p; }
        sum = warp_sum(sum);
        __syncwarp();
        const float inv = 1.f / sum;
        if (grouped) {                                      // (scratch behind the first rows: [8][experts] twice)
            float* extra = (float*)(start + experts + 1);
            route_choice_warp(lane, my, extra + (size_t)warp * experts, extra + (size_t)(8 + warp) * experts, inv, correction,
                              experts, top, groups, keep, chosen + (size_t)t * top, weight + (size_t)t * top, cnt, scale,
                              renormalize, tiny);
            continue;
        }
        float taken = 0.f;
        for (int k = 0; k < top; ++k) {
            float bv = -1.f; int bi = 0x7fffffff;
            for (int e = lane; e < experts; e += 32) { const float v = my[e]; if (v > bv) { bv = v; bi = e; } }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) {
                chosen[(size_t)t * top + k] = bi;
                weight[(size_t)t * top + k] = bv * inv;
                my[bi] = -2.f;
                atomicAdd(cnt + bi, 1);
            }
            taken += bv * inv;
            __syncwarp();
        }
        const float f = renormalize ? scale / taken : scale;
        for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] *= f;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) { start[e] = at; at += cnt[e]; }
        start[experts] = at;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) { counts[e] = cnt[e]; counts[experts + e] = start[e]; cnt[e] = 0; }
    if (threadIdx.x == 0) { counts[2 * experts] = start[experts]; counts[2 * experts + 1] = 0; counts[2 * experts + 2] = tokens; }
    __syncthreads();
    for (int i = threadIdx.x; i < tokens * top; i += blockDim.x) {
        const int e = chosen[i];                            // (written by this block: visible after the barrier)
        const int p = start[e] + atomicAdd(cnt + e, 1);
        place[i] = p;
        token_of[p] = i / top;
    }
}

__global__ void expert_whole_kernel(int32_t* counts, int experts, int tokens) {
    counts[2 * experts + 1] = 0;
    counts[2 * experts + 2] = tokens;
}

// hb_route_top and hb_expert_rows as one call. counts [2 experts + 3] need not be zeroed; afterwards it also holds, at
// 2 experts + 1, the pair (0, tokens).
extern "C" int hb_route_rows(int32_t* chosen, float* weight, int32_t* counts, int32_t* place, int32_t* token_of,
                             const float* z, const float* bias, int ld, int tokens, int experts, int top, float scale,
                             int renormalize, const float* correction, int groups, int keep, float tiny, hb_stream stream) {
    if (tokens == 0) return 0;
    if (experts < 1 || top < 1 || top > experts || ld < experts) HB_REFUSE("route_rows: top %d of %d experts in rows of %d", top, experts, ld);
    if (groups < 1 || experts % groups || keep < 1 || keep > groups || (long)keep * (experts / groups) < top)
        HB_REFUSE("route_rows: %d groups of which %d are kept, for top %d of %d experts", groups, keep, top, experts);
    cudaStream_t s = (cudaStream_t)stream;
    const int grouped = correction || groups > 1 || tiny != 0.f;
    if (tokens <= RS_TOKENS && experts <= RS_EXPERTS) {
        const size_t smem = ((size_t)(grouped ? 24 : 8) * experts + 2 * experts + 1) * sizeof(float);
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(route_rows_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        route_rows_small_kernel<<<1, 256, smem, s>>>(chosen, weight, counts, place, token_of, z, ld, tokens, experts, top, scale,
                                                     renormalize, bias, correction, groups, keep, tiny, grouped);
        HB_LAUNCH_CHECK("route_rows_small");
        return 0;
    }
    HB_CUDA(cudaMemsetAsync(counts, 0, (size_t)(2 * experts + 3) * sizeof(int32_t), s));
    int rc = hb_route_top(chosen, weight, counts, z, bias, ld, tokens, experts, top, scale, renormalize, correction, groups, keep,
                          tiny, stream);
    if (rc) return rc;
    rc = hb_expert_rows(place, token_of, counts, chosen, tokens, top, experts, stream);
    if (rc) return rc;
    expert_whole_kernel<<<1, 1, 0, s>>>(counts, experts, tokens);
    HB_LAUNCH_CHECK("expert_whole");
    return 0;
}

// ---------------------------------------------------------------- the experts' products, any dtype, CUDA cores
__device__ __forceinline__ float expert_act(float v, int act) {
    if (act == 1) { v = fmaxf(v, 0.f); return v * v; }            // the square of relu
    if (act == 2) return v / (1.f + expf(-v));                   // silu
    if (act == 3) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));   // gelu, tanh form
    return v;
}

#define EBM 64
#define EBN 64
#define EBK 16

// Finds the expert and the first row of m-tile `tile` (tiles of `bm` rows, counted expert by expert). Called by every
// thread of the block; the first warp reads the experts' first rows 32 at a time and adds up their tile counts with
// shuffles; info[0] = the expert (-1: no such tile), info[1] = the tile's first row, info[2] = the expert's end.
__device__ __forceinline__ void expert_tile(const int32_t* __restrict__ starts, int experts, int tile, int bm, int* info) {
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int base = 0, found = -1, row0 = 0, row_end = 0;
        for (int e0 = 0; e0 < experts && found < 0; e0 += 32) {
            const int e = e0 + lane;
            const int a = e < experts ? starts[e] : 0, b = e < experts ? starts[e + 1] : 0;
            const int tiles = (b - a + bm - 1) / bm;
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
            const int before = base + incl - tiles;
            const bool hit = tile >= before && tile < before + tiles;
            const unsigned who = __ballot_sync(0xffffffffu, hit);
            if (who) {
                const int src = __ffs(who) - 1;
                found = e0 + src;
                row0 = __shfl_sync(0xffffffffu, a, src) + (tile - __shfl_sync(0xffffffffu, before, src)) * bm;
                row_end = __shfl_sync(0xffffffffu, b, src);
            }
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) { info[0] = found; info[1] = row0; info[2] = row_end; }
    }
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(256) expert_linear_kernel(T* __restrict__ out, const T* __restrict__ x,
                                                            const int32_t* __restrict__ token_of, const T* __restrict__ w,
                                                            const int32_t* __restrict__ starts, int experts, int n, int k,
                                                            int act) {
    __shared__ float xs[EBK][EBM + 4];
    __shared__ float ws[EBK][EBN + 4];
    __shared__ int src[EBM];
    __shared__ int tile_info[3];
    expert_tile(starts, experts, blockIdx.y, EBM, tile_info);
    const int e = tile_info[0], m0 = tile_info[1], m_end = tile_info[2];
    if (e < 0) return;
    const int tid = threadIdx.x;
    if (tid < EBM) src[tid] = m0 + tid < m_end ? (token_of ? token_of[m0 + tid] : m0 + tid) : -1;
    __syncthreads();
    const int n0 = blockIdx.x * EBN;
    const T* we = w + (size_t)e * n * k;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4] = {};
    const int xr = src[lr], wr = n0 + lr;
    for (int k0 = 0; k0 < k; k0 += EBK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = k0 + lk + i;
            xs[lk + i][lr] = xr >= 0 && kk < k ? to_f32(x[(size_t)xr * k + kk]) : 0.f;
            ws[lk + i][lr] = wr < n && kk < k ? to_f32(we[(size_t)wr * k + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk2 = 0; kk2 < EBK; ++kk2) {
            const float4 a = *(const float4*)&xs[kk2][ty * 4];
            const float4 b = *(const float4*)&ws[kk2][tx * 4];
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = m0 + ty * 4 + i;
        if (r >= m_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c < n) out[(size_t)r * n + c] = from_f32<T>(expert_act(acc[i][j], act));
        }
    }
}

extern "C" int hb_expert_linear(void* out, const void* x, int dtype, const int32_t* token_of, const void* w,
                                const int32_t* starts, int rows, int experts, int n, int k, int act, hb_stream stream) {
    if (rows == 0 || n == 0) return 0;
    if (k <= 0 || experts < 1) HB_REFUSE("expert_linear: k = %d, %d experts", k, experts);
    const long tiles = (rows + EBM - 1) / EBM + (experts < rows ? experts : rows);   // the most m-tiles any split of the rows can have:
                                                                                      // an expert with rows adds at most one partial tile
    if (tiles > 65535) HB_REFUSE("expert_linear: %d rows over %d experts are above the kernel's limit", rows, experts);
    dim3 grid((n + EBN - 1) / EBN, (unsigned)tiles);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_F32)
        expert_linear_kernel<float><<<grid, 256, 0, s>>>((float*)out, (const float*)x, token_of, (const float*)w, starts,
                                                          experts, n, k, act);
    else if (dtype == HB_BF16)
        expert_linear_kernel<bf16><<<grid, 256, 0, s>>>((bf16*)out, (const bf16*)x, token_of, (const bf16*)w, starts,
                                                         experts, n, k, act);
    else HB_REFUSE("expert_linear: dtype %d", dtype);
    HB_LAUNCH_CHECK("expert_linear");
    return 0;
}

// ---------------------------------------------------------------- elementwise
// act 4 (xielu, with two numbers p, q): softplus(p) v^2 + v / 2 for v > 0, (1/2 + softplus(q)) (exp(v) - 1 - v) + v / 2
// otherwise; act 5: tanh. Both for this kernel alone (the experts' products know 1 to 3).
__device__ __forceinline__ float softplus_e(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float any_act(float v, int act, float up, float down) {
    if (act == 4) return v > 0.f ? fmaf(up * v, v, 0.5f * v) : fmaf(down, expm1f(v) - v, 0.5f * v);
    if (act == 5) return tanhf(v);
    return expert_act(v, act);
}
template <typename T>
__global__ void activation_kernel(T* __restrict__ x, long count, int act, const float* __restrict__ numbers) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float up = act == 4 ? softplus_e(numbers[0]) : 0.f, down = act == 4 ? 0.5f + softplus_e(numbers[1]) : 0.f;
    x[i] = from_f32<T>(any_act(to_f32(x[i]), act, up, down));
}
// The same, 16 bytes a thread (x on a 16-byte boundary; the few elements behind the last whole piece go one by one).
template <typename T>
__global__ void activation_wide_kernel(T* __restrict__ x, long count, int act, const float* __restrict__ numbers) {
    constexpr int N = 16 / sizeof(T);
    const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * N;
    if (i >= count) return;
    const float up = act == 4 ? softplus_e(numbers[0]) : 0.f, down = act == 4 ? 0.5f + softplus_e(numbers[1]) : 0.f;
    if (i + N > count) {
        for (long j = i; j < count; ++j) x[j] = from_f32<T>(any_act(to_f32(x[j]), act, up, down));
        return;
    }
    uint4 v = *(const uint4*)(x + i);
    T* e = (T*)&v;
#pragma unroll
    for (int j = 0; j < N; ++j) e[j] = from_f32<T>(any_act(to_f32(e[j]), act, up, down));
    *(uint4*)(x + i) = v;
}

extern "C" int hb_activation(void* x, int dtype, long count, int act, const float* numbers, hb_stream stream) {
    if (count == 0) return 0;
    if (act == 4 && !numbers) HB_REFUSE("activation: xielu needs its two numbers");
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (((uintptr_t)x & 15) == 0 && count >= 4096) {
        const long per = dtype == HB_F32 ? 4 : 8;
        const unsigned wide = (unsigned)(((count + per - 1) / per + 255) / 256);
        if (dtype == HB_F32) activation_wide_kernel<float><<<wide, 256, 0, (cudaStream_t)stream>>>((float*)x, count, act, numbers);
        else if (dtype == HB_BF16) activation_wide_kernel<bf16><<<wide, 256, 0, (cudaStream_t)stream>>>((bf16*)x, count, act, numbers);
        else HB_REFUSE("activation: dtype %d", dtype);
        HB_LAUNCH_CHECK("activation");
        return 0;
    }
    if (dtype == HB_F32) activation_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((float*)x, count, act, numbers);
    else if (dtype == HB_BF16) activation_kernel<bf16><<<blocks, 256, 0, (cudaStream_t)stream>>>((bf16*)x, count, act, numbers);
    else HB_REFUSE("activation: dtype %d", dtype);
    HB_LAUNCH_CHECK("activation");
    return 0;
}

// o[t, i] *= sigmoid(g[t * ld + i]) in 32-bit, rounded once.
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ o, const T* __restrict__ g, int n, long ld) {
    const size_t t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) o[t * n + i] = from_f32<T>(to_f32(o[t * n + i]) / (1.f + expf(-to_f32(g[t * ld + i]))));
}

extern "C" int hb_sigmoid_gate(void* o, const void* g, int dtype, int tokens, int n, long ld, hb_stream stream) {
    if (tokens == 0 || n == 0) return 0;
    if (tokens > 65535) HB_REFUSE("sigmoid_gate: %d rows are above 65535", tokens);
    dim3 grid((n + 255) / 256, tokens);
    if (dtype == HB_F32) sigmoid_gate_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((float*)o, (const float*)g, n, ld);
    else if (dtype == HB_BF16) sigmoid_gate_kernel<bf16><<<grid, 256, 0, (cudaStream_t)stream>>>((bf16*)o, (const bf16*)g, n, ld);
    else HB_REFUSE("sigmoid_gate: dtype %d", dtype);
    HB_LAUNCH_CHECK("sigmoid_gate");
    return 0;
}

// ---------------------------------------------------------------- the weighted sum per token
#define XC_TOP 64
template <typename T>
__global__ void expert_combine_kernel(T* __restrict__ out, const T* __restrict__ y, const int32_t* __restrict__ place,
                                      const float* __restrict__ weight, const T* __restrict__ shared,
                                      const float* __restrict__ z, int ldz, int gate_at, int top, int hidden,
                                      const T* __restrict__ x, const int32_t* __restrict__ identity_from) {
    __shared__ int rows[XC_TOP];                            // the token's rows and weights, read once
    const int ident = identity_from ? *identity_from : 0x7fffffff;   // rows from here on belong to identity experts: x[t]
    __shared__ float wgt[XC_TOP];
    const size_t t = blockIdx.x;
    const bool kept = top <= XC_TOP;
    if (kept && threadIdx.x < top) { rows[threadIdx.x] = place[t * top + threadIdx.x]; wgt[threadIdx.x] = weight[t * top + threadIdx.x]; }
    __syncthreads();
    const float gate = shared ? (z ? 1.f / (1.f + expf(-z[t * ldz + gate_at])) : 1.f) : 0.f;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int p = kept ? rows[k] : place[t * top + k];
            if (p >= 0) acc = fmaf(kept ? wgt[k] : weight[t * top + k],
                                   to_f32(p >= ident ? x[t * hidden + i] : y[(size_t)p * hidden + i]), acc);
        }
        if (shared) acc = fmaf(gate, to_f32(shared[t * hidden + i]), acc);
        out[t * hidden + i] = from_f32<T>(acc);
    }
}

// The same in bfloat16 for rows of a multiple of 8 columns: a thread adds 8 columns at a time (16-byte loads).
__global__ void expert_combine_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ y, const int32_t* __restrict__ place,
                                             const float* __restrict__ weight, const bf16* __restrict__ shared,
                                             const float* __restrict__ z, int ldz, int gate_at, int top, int hidden,
                                             const bf16* __restrict__ x, const int32_t* __restrict__ identity_from) {
    __shared__ int rows[XC_TOP];
    __shared__ float wgt[XC_TOP];
    const int ident = identity_from ? *identity_from : 0x7fffffff;
    const size_t t = blockIdx.x;
    if (threadIdx.x < top) { rows[threadIdx.x] = place[t * top + threadIdx.x]; wgt[threadIdx.x] = weight[t * top + threadIdx.x]; }
    __syncthreads();
    const float gate = shared ? (z ? 1.f / (1.f + expf(-z[t * ldz + gate_at])) : 1.f) : 0.f;
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8; i < hidden; i += gridDim.y * blockDim.x * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < top; ++k) {
            const int p = rows[k];
            if (p < 0) continue;
            const uint4 v = __ldg((const uint4*)(p >= ident ? x + t * hidden + i : y + (size_t)p * hidden + i));
            const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
            const float w = wgt[k];
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); acc[2 * j] = fmaf(w, f.x, acc[2 * j]); acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]); }
        }
        if (shared) {
            const uint4 v = __ldg((const uint4*)(shared + t * hidden + i));
            const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); acc[2 * j] = fmaf(gate, f.x, acc[2 * j]); acc[2 * j + 1] = fmaf(gate, f.y, acc[2 * j + 1]); }
        }
        uint4 o;
        __nv_bfloat162 a0 = __floats2bfloat162_rn(acc[0], acc[1]), a1 = __floats2bfloat162_rn(acc[2], acc[3]);
        __nv_bfloat162 a2 = __floats2bfloat162_rn(acc[4], acc[5]), a3 = __floats2bfloat162_rn(acc[6], acc[7]);
        o.x = *(uint32_t*)&a0; o.y = *(uint32_t*)&a1; o.z = *(uint32_t*)&a2; o.w = *(uint32_t*)&a3;
        *(uint4*)(out + t * hidden + i) = o;
    }
}

extern "C" int hb_expert_combine(void* out, const void* y, int dtype, const int32_t* place, const float* weight,
                                 const void* shared, const float* z, int ldz, int gate_at, int tokens, int top, int hidden,
                                 const void* x, const int32_t* identity_from, hb_stream stream) {
    if (tokens == 0) return 0;
    if (shared && z && gate_at >= ldz) HB_REFUSE("expert_combine: the shared expert's gate lies outside the logits' rows");
    if ((x == nullptr) != (identity_from == nullptr)) HB_REFUSE("expert_combine: identity experts need the input rows and their first row");
    if (hidden > 65535 * 128) HB_REFUSE("expert_combine: %d columns", hidden);
    const int threads = hidden >= 256 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(tokens, (hidden + threads - 1) / threads);                        // a block every `threads` columns of a token
    if (dtype == HB_BF16 && hidden % 8 == 0 && top <= XC_TOP && (((uintptr_t)out | (uintptr_t)y | (uintptr_t)shared | (uintptr_t)x) % 16) == 0) {
        const int th = hidden >= 1024 ? 128 : 64;                   // 8 columns a thread
        dim3 g8(tokens, (hidden / 8 + th - 1) / th);
        expert_combine_bf16x8_kernel<<<g8, th, 0, s>>>((bf16*)out, (const bf16*)y, place, weight, (const bf16*)shared, z, ldz,
                                                      gate_at, top, hidden, (const bf16*)x, identity_from);
        HB_LAUNCH_CHECK("expert_combine");
        return 0;
    }
    if (dtype == HB_F32)
        expert_combine_kernel<float><<<grid, threads, 0, s>>>((float*)out, (const float*)y, place, weight,
                                                                (const float*)shared, z, ldz, gate_at, top, hidden, (const float*)x, identity_from);
    else if (dtype == HB_BF16)
        expert_combine_kernel<bf16><<<grid, threads, 0, s>>>((bf16*)out, (const bf16*)y, place, weight,
                                                               (const bf16*)shared, z, ldz, gate_at, top, hidden, (const bf16*)x, identity_from);
    else HB_REFUSE("expert_combine: dtype %d", dtype);
    HB_LAUNCH_CHECK("expert_combine");
    return 0;
}

// ---------------------------------------------------------------- the experts' products in bfloat16 on tensor cores
// The same tiles (expert by expert, at most ceil(rows / BM) + experts of them), mma.sync m16n8k16 with 32-bit sums:
// BM x 128 outputs a CTA (four warps; eight for BM = 128), the k range in steps of 32 through a three-stage cp.async ring. x rows are
// gathered by token_of while they are copied (rows past the expert's end are zero-filled), the weight tile is 128 rows
// of w[e]. BM = 128 or 64 for prompts (hundreds or dozens of rows an expert), 16 for decode steps (a row or two an
// expert: the weight streams once either way, and a 16-row tile wastes a quarter of the tensor work a 64-row tile
// would). k and n multiples of 8.
#define XB_BN 128
#define XB_BK 32
#define XB_LD (XB_BK + 8)
#define XB_STAGES 3

__device__ __forceinline__ void xb_cp16(void* dst, const void* src, int bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void xb_ldsm4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void xb_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int BM>
__global__ void __launch_bounds__(BM == 128 ? 256 : 128) expert_linear_bf16_kernel(bf16* __restrict__ out, const bf16* __restrict__ x,
                                                                 const int32_t* __restrict__ token_of,
                                                                 const bf16* __restrict__ w,
                                                                 const int32_t* __restrict__ starts, int experts, int n,
                                                                 int k, int act) {
    constexpr int WARPS = BM == 128 ? 8 : 4, THREADS = WARPS * 32;
    constexpr int WARPS_M = BM == 128 ? 4 : BM == 64 ? 2 : 1, WARPS_N = WARPS / WARPS_M;
    constexpr int MF = BM / 16 / WARPS_M;                       // 16-row fragments a warp
    constexpr int NF = XB_BN / 8 / WARPS_N;                     // 8-column fragments a warp
    extern __shared__ __align__(16) unsigned char xb_smem[];
    bf16 (*as)[BM][XB_LD] = (bf16 (*)[BM][XB_LD])xb_smem;                                              // [stages][BM][ld]
    bf16 (*bs)[XB_BN][XB_LD] = (bf16 (*)[XB_BN][XB_LD])(xb_smem + sizeof(bf16) * XB_STAGES * BM * XB_LD);   // [stages][128][ld]
    __shared__ int src[BM];
    __shared__ int tile_info[3];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    expert_tile(starts, experts, blockIdx.y, BM, tile_info);
    const int e = tile_info[0], m0 = tile_info[1], m_end = tile_info[2];
    if (e < 0) return;
    if (tid < BM) src[tid] = m0 + tid < m_end ? (token_of ? token_of[m0 + tid] : m0 + tid) : -1;
    __syncthreads();
    const int n0 = blockIdx.x * XB_BN;
    const bf16* we = w + (size_t)e * n * k;
    const int k_tiles = (k + XB_BK - 1) / XB_BK;

    auto load = [&](int kt, int stage) {
        const int k0 = kt * XB_BK;
        for (int c = tid; c < (BM + XB_BN) * 4; c += THREADS) {  // 16-byte pieces: four a row
            const int r = c >> 2, col = (c & 3) * 8;
            const bool in_k = k0 + col < k;
            if (r < BM) {
                const int s = src[r];
                const bool ok = s >= 0 && in_k;
                xb_cp16(&as[stage][r][col], x + (ok ? (size_t)s * k + k0 + col : 0), ok ? 16 : 0);
            } else {
                const int wr = n0 + r - BM;
                const bool ok = wr < n && in_k;
                xb_cp16(&bs[stage][r - BM][col], we + (ok ? (size_t)wr * k + k0 + col : 0), ok ? 16 : 0);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    const int wm = warp / WARPS_N, wn = warp % WARPS_N;
    float acc[MF][NF][4];
#pragma unroll
    for (int i = 0; i < MF; ++i)
#pragma unroll
        for (int j = 0; j < NF; ++j) { acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f; }

#pragma unroll
    for (int s = 0; s < XB_STAGES - 1; ++s) {
        if (s < k_tiles) load(s, s); else asm volatile("cp.async.commit_group;\n" ::);
    }
    for (int kt = 0; kt < k_tiles; ++kt) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(XB_STAGES - 2));
        __syncthreads();                                         // tile kt has landed; the stage of tile kt - 1 is free
        if (kt + XB_STAGES - 1 < k_tiles) load(kt + XB_STAGES - 1, (kt + XB_STAGES - 1) % XB_STAGES);
        else asm volatile("cp.async.commit_group;\n" ::);
        const int stage = kt % XB_STAGES;
#pragma unroll
        for (int kk = 0; kk < XB_BK; kk += 16) {
            uint32_t a[MF][4];
#pragma unroll
            for (int i = 0; i < MF; ++i)
                xb_ldsm4(a[i], &as[stage][(wm * MF + i) * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int jp = 0; jp < NF / 2; ++jp) {
                uint32_t b[4];
                xb_ldsm4(b, &bs[stage][wn * NF * 8 + jp * 16 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
                for (int i = 0; i < MF; ++i) {
                    xb_mma(acc[i][2 * jp], a[i], b[0], b[1]);
                    xb_mma(acc[i][2 * jp + 1], a[i], b[2], b[3]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
#pragma unroll
    for (int i = 0; i < MF; ++i) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = m0 + (wm * MF + i) * 16 + (lane >> 2) + half * 8;
            if (r >= m_end) continue;
#pragma unroll
            for (int j = 0; j < NF; ++j) {
                const int c = n0 + wn * NF * 8 + j * 8 + (lane & 3) * 2;
                if (c < n)
                    *(__nv_bfloat162*)(out + (size_t)r * n + c) =
                        __floats2bfloat162_rn(expert_act(acc[i][j][half * 2], act), expert_act(acc[i][j][half * 2 + 1], act));
            }
        }
    }
}

// ---------------------------------------------------------------- a row or two an expert (decode steps)
// Tiles of 8 rows; the product is bound by reading each chosen expert's weight once, and what counts is how many bytes
// are on their way: a CTA of eight warps keeps the tile's rows of x in shared memory and takes 32 weight rows, four a
// warp; a lane reads 16 bytes of each of them per step of 256 columns (two steps in flight) and multiplies on the CUDA
// cores in 32-bit; the lanes' sums meet by shuffles. No tensor cores: with one or two rows they would idle anyway.
#define XF_ROWS 8
#define XF_WROWS 4

__global__ void __launch_bounds__(256) expert_linear_few_kernel(bf16* __restrict__ out, const bf16* __restrict__ x,
                                                                const int32_t* __restrict__ token_of,
                                                                const bf16* __restrict__ w,
                                                                const int32_t* __restrict__ starts, int experts, int n,
                                                                int k, int act) {
    extern __shared__ __align__(16) unsigned char xf_smem[];
    bf16* xs = (bf16*)xf_smem;                              // [XF_ROWS][k]
    __shared__ int tile_info[3];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    expert_tile(starts, experts, blockIdx.y, XF_ROWS, tile_info);
    const int e = tile_info[0], m0 = tile_info[1];
    if (e < 0) return;
    const int nrows = min(XF_ROWS, tile_info[2] - m0);
    const int chunks = k >> 3;
    for (int c = tid; c < nrows * chunks; c += 256) {
        const int r = c / chunks, col = (c % chunks) * 8;
        const int src = token_of ? token_of[m0 + r] : m0 + r;
        *(uint4*)(xs + (size_t)r * k + col) = __ldg((const uint4*)(x + (size_t)src * k + col));
    }
    __syncthreads();
    const int nr = blockIdx.x * 32 + warp * XF_WROWS;       // this warp's first weight row
    if (nr >= n) return;
    const bf16* we = w + (size_t)e * n * k;
    float acc[XF_WROWS][XF_ROWS];
#pragma unroll
    for (int j = 0; j < XF_WROWS; ++j)
#pragma unroll
        for (int r = 0; r < XF_ROWS; ++r) acc[j][r] = 0.f;
#pragma unroll 2
    for (int kc = lane * 8; kc < k; kc += 256) {
        uint4 wv[XF_WROWS];
#pragma unroll
        for (int j = 0; j < XF_WROWS; ++j)
            wv[j] = nr + j < n ? __ldg((const uint4*)(we + (size_t)(nr + j) * k + kc)) : make_uint4(0u, 0u, 0u, 0u);
        float wf[XF_WROWS][8];
#pragma unroll
        for (int j = 0; j < XF_WROWS; ++j) {
            const __nv_bfloat162* h = (const __nv_bfloat162*)&wv[j];
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); wf[j][2 * i] = f.x; wf[j][2 * i + 1] = f.y; }
        }
#pragma unroll
        for (int r = 0; r < XF_ROWS; ++r) {
            if (r < nrows) {
                const uint4 xv = *(const uint4*)(xs + (size_t)r * k + kc);
                const __nv_bfloat162* h = (const __nv_bfloat162*)&xv;
                float xf[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); xf[2 * i] = f.x; xf[2 * i + 1] = f.y; }
#pragma unroll
                for (int j = 0; j < XF_WROWS; ++j)
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[j][r] = fmaf(wf[j][i], xf[i], acc[j][r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < XF_ROWS; ++r) {
        if (r < nrows) {
#pragma unroll
            for (int j = 0; j < XF_WROWS; ++j) {
                const float v = warp_sum(acc[j][r]);
                if (lane == 0 && nr + j < n) out[(size_t)(m0 + r) * n + nr + j] = __float2bfloat16_rn(expert_act(v, act));
            }
        }
    }
}

// tile_rows: 8 (the kernel above), 16, 64 or 128 rows a tile (0: chosen from the rows an expert gets on average).
extern "C" int hb_expert_linear_bf16(void* out, const void* x, const int32_t* token_of, const void* w,
                                     const int32_t* starts, int rows, int experts, int n, int k, int act, int tile_rows,
                                     hb_stream stream) {
    if (rows == 0 || n == 0) return 0;
    if (k <= 0 || k % 8 || n % 8 || experts < 1) HB_REFUSE("expert_linear_bf16: k = %d and n = %d must be multiples of 8", k, n);
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) % 16) HB_REFUSE("expert_linear_bf16: pointers must be 16-byte aligned");
    const bool fits = (size_t)XF_ROWS * k * sizeof(bf16) <= 200 * 1024;
    const int bm = tile_rows ? tile_rows : (rows <= 8 * experts && fits ? 8 : rows <= 16 * experts ? 16 : rows <= 96 * experts ? 64 : 128);
    if (bm != 8 && bm != 16 && bm != 64 && bm != 128) HB_REFUSE("expert_linear_bf16: tiles of %d rows; 8, 16, 64 or 128", bm);
    if (bm == 8 && !fits) HB_REFUSE("expert_linear_bf16: rows of %d columns do not fit the 8-row kernel's shared memory", k);
    const long tiles = (rows + bm - 1) / bm + (experts < rows ? experts : rows);
    if (tiles > 65535) HB_REFUSE("expert_linear_bf16: %d rows over %d experts are above the kernel's limit", rows, experts);
    dim3 grid((n + XB_BN - 1) / XB_BN, (unsigned)tiles);
    cudaStream_t s = (cudaStream_t)stream;
    if (bm == 8) {
        const size_t smem = (size_t)XF_ROWS * k * sizeof(bf16);
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(expert_linear_few_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dim3 few((n + 31) / 32, (unsigned)tiles);
        expert_linear_few_kernel<<<few, 256, smem, s>>>((bf16*)out, (const bf16*)x, token_of, (const bf16*)w, starts, experts, n, k, act);
        HB_LAUNCH_CHECK("expert_linear_few");
        return 0;
    }
    const size_t smem = sizeof(bf16) * XB_STAGES * (size_t)(bm + XB_BN) * XB_LD;
#define XB_GO(BM_, T_) do { \
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(expert_linear_bf16_kernel<BM_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        expert_linear_bf16_kernel<BM_><<<grid, T_, smem, s>>>((bf16*)out, (const bf16*)x, token_of, (const bf16*)w, starts, experts, n, k, act); \
    } while (0)
    if (bm == 16) XB_GO(16, 128); else if (bm == 64) XB_GO(64, 128); else XB_GO(128, 256);
#undef XB_GO
    HB_LAUNCH_CHECK("expert_linear_bf16");
    return 0;
}
