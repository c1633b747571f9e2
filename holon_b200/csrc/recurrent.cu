// Mixers whose memory is a matrix per head instead of a cache of keys: S [key channel, value channel] in 32-bit per
// request slot and head (kept column by column: state [slots, heads, vdim, dim], so that the key channels a thread owns
// lie side by side), updated token by token,
//     S <- diag(g_t) S                      (g_t: a decay per key channel and token, one per head and token, or one fixed
//                                            decay per head)
//     u  = beta_t (v_t - S^T k_t)           (the delta rule; without beta: u = v_t)
//     S <- S + k_t u^T,      o_t = S^T q_t  (the read-out sees the token's own write)
// or, with a removal rate r_t per key channel (the generalized delta rule, both terms on the old S),
//     S <- diag(g_t) S - (r_t o k_t)(k_t^T S) + k_t v_t^T,      o_t = S^T q_t
// and the kernels around that scan: what turns a layer's first product into q, k, v, decays and gates (a short causal
// convolution over time with its carried inputs, activations, unit vectors, rotation), and the per-head norm with the
// output gate behind the scan. Everything that enters the recurrence is 32-bit here, whatever the engine's dtype.
#include "common.cuh"

// The row b with query_start[b] <= t < query_start[b + 1].
__device__ __forceinline__ int row_of_token(const int32_t* __restrict__ query_start, int rows, int t) {
    int lo = 0, hi = rows;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (query_start[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------- the scan
// grid (rows, heads, column tiles); a thread owns DPT key channels of one value column, in groups of four that lie
// side by side (group i4 of thread p: channels (i4 P + p) 4 .. + 3), and the P threads of a column are neighbouring lanes
// that read a token's k, q and decays as 16-byte pieces without bank conflicts. With P = 32 a warp is a column, and the
// many warps of an SM hide one another's waits: a token is a chain of multiply-adds and two sums over P lanes that no
// width shortens. Tokens are staged in shared memory `tb` at a time by cp.async, a stage ahead of the one in work, so
// the loop over a stage's tokens has no block-wide barrier and no wait for global memory.
#define SC_TB 16

__device__ __forceinline__ void cp_async_f32(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_f32x4(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// TOKEN: `head_decay` holds one decay per token and head [tokens, heads]; it rides in the stage's beta column (no delta rule then).
// GENERAL (with PER_CHANNEL, without DELTA): `rate` [tokens, heads, dim] is the removal rate per key channel; a fourth
// array of the stage holds it, and a token's step is S_i <- g_i S_i + k_i (v - r_i (k . S_old)).
template <int DPT, int P, bool PER_CHANNEL, bool DELTA, bool TOKEN = false, bool GENERAL = false>
__global__ void recurrent_scan_kernel(float* __restrict__ out, const float* __restrict__ qk, const float* __restrict__ v,
                                      const float* __restrict__ decay, const float* __restrict__ head_decay,
                                      const float* __restrict__ beta, const float* __restrict__ rate, float* __restrict__ state,
                                      const int32_t* __restrict__ query_start, const int32_t* __restrict__ row_slot,
                                      int heads, int kv_heads, int dim, int vdim, int VT, int tb) {
    extern __shared__ __align__(16) float sm[];
    constexpr int DP = P * DPT;
    const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * VT;
    const int hk = h / (heads / kv_heads);
    const int p = threadIdx.x % P, cl = threadIdx.x / P, c = c0 + cl;
    const bool col = cl < VT && c < vdim;
    const int t0 = query_start[b], n = query_start[b + 1] - t0;
    float* S_g = state + (((size_t)row_slot[b] * heads + h) * vdim + (col ? c : 0)) * dim;   // this thread's column
    // a stage: q [tb][DP], k [tb][DP], decays [tb][DP] (per-channel decays only), v [tb][VT], beta [tb]; two of them
    float S[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = ((i >> 2) * P + p) * 4 + (i & 3);
        S[i] = col && d < dim ? S_g[d] : 0.f;
    }
    float fixed = head_decay && !TOKEN ? head_decay[h] : 1.f;
    const bool vec = (dim & 3) == 0;
    if (n == 1) {                            // a row of one token (a decode step): no stage, no barrier; every thread reads
        const size_t t = (size_t)t0;         // its own channels of k, q and the decays straight from global memory
        if (TOKEN) fixed = head_decay[t * heads + h];
        auto four = [&](const float* base, int d, float fill) -> float4 {
            if (vec && d + 3 < dim) return *(const float4*)(base + d);
            return make_float4(d < dim ? base[d] : fill, d + 1 < dim ? base[d + 1] : fill, d + 2 < dim ? base[d + 2] : fill,
                               d + 3 < dim ? base[d + 3] : fill);
        };
        const float* q_g = qk + ((t * 2) * kv_heads + hk) * dim;
        const float* k_g = qk + ((t * 2 + 1) * kv_heads + hk) * dim;
        float u = col ? v[(t * heads + h) * vdim + c] : 0.f;
        float4 k4[DPT / 4], q4[DPT / 4];
        if (GENERAL) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) {
                k4[i] = four(k_g, (i * P + p) * 4, 0.f);
                a += S[4 * i] * k4[i].x + S[4 * i + 1] * k4[i].y + S[4 * i + 2] * k4[i].z + S[4 * i + 3] * k4[i].w;
            }
#pragma unroll
            for (int o = 1; o < P; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) {
                const int d = (i * P + p) * 4;
                const float4 g = four(decay + (t * heads + h) * dim, d, 1.f), r = four(rate + (t * heads + h) * dim, d, 0.f);
                const float4 q = four(q_g, d, 0.f);
                S[4 * i] = fmaf(g.x, S[4 * i], k4[i].x * fmaf(-r.x, a, u));
                S[4 * i + 1] = fmaf(g.y, S[4 * i + 1], k4[i].y * fmaf(-r.y, a, u));
                S[4 * i + 2] = fmaf(g.z, S[4 * i + 2], k4[i].z * fmaf(-r.z, a, u));
                S[4 * i + 3] = fmaf(g.w, S[4 * i + 3], k4[i].w * fmaf(-r.w, a, u));
                o += S[4 * i] * q.x + S[4 * i + 1] * q.y + S[4 * i + 2] * q.z + S[4 * i + 3] * q.w;
            }
#pragma unroll
            for (int x = 1; x < P; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
            if (p == 0 && col) out[(t * heads + h) * vdim + c] = o;
#pragma unroll
            for (int i = 0; i < DPT; ++i) {
                const int d = ((i >> 2) * P + p) * 4 + (i & 3);
                if (col && d < dim) S_g[d] = S[i];
            }
            return;
        }
#pragma unroll
        for (int i = 0; i < DPT / 4; ++i) {
            const int d = (i * P + p) * 4;
            k4[i] = four(k_g, d, 0.f);
            q4[i] = four(q_g, d, 0.f);
            if (PER_CHANNEL) {
                const float4 g = four(decay + (t * heads + h) * dim, d, 1.f);
                S[4 * i] *= g.x; S[4 * i + 1] *= g.y; S[4 * i + 2] *= g.z; S[4 * i + 3] *= g.w;
            } else {
                S[4 * i] *= fixed; S[4 * i + 1] *= fixed; S[4 * i + 2] *= fixed; S[4 * i + 3] *= fixed;
            }
        }
        if (DELTA) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i)
                a += S[4 * i] * k4[i].x + S[4 * i + 1] * k4[i].y + S[4 * i + 2] * k4[i].z + S[4 * i + 3] * k4[i].w;
#pragma unroll
            for (int o = 1; o < P; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            u = beta[t * heads + h] * (u - a);
        }
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < DPT / 4; ++i) {
            S[4 * i] = fmaf(k4[i].x, u, S[4 * i]);
            S[4 * i + 1] = fmaf(k4[i].y, u, S[4 * i + 1]);
            S[4 * i + 2] = fmaf(k4[i].z, u, S[4 * i + 2]);
            S[4 * i + 3] = fmaf(k4[i].w, u, S[4 * i + 3]);
            o += S[4 * i] * q4[i].x + S[4 * i + 1] * q4[i].y + S[4 * i + 2] * q4[i].z + S[4 * i + 3] * q4[i].w;
        }
#pragma unroll
        for (int x = 1; x < P; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
        if (p == 0 && col) out[(t * heads + h) * vdim + c] = o;
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = ((i >> 2) * P + p) * 4 + (i & 3);
            if (col && d < dim) S_g[d] = S[i];
        }
        return;
    }
    constexpr int ARRAYS = PER_CHANNEL ? (GENERAL ? 4 : 3) : 2;       // q, k, decays, removal rates
    const int used = tb * (ARRAYS * DP + VT + 1), per_stage = (used + 3) & ~3;   // (stages start on 16-byte boundaries)
    for (int e = threadIdx.x; e < 2 * per_stage; e += blockDim.x) {      // what no copy fills stays neutral: k = q = v = 0,
        const int at = e % per_stage;                                    // decay = beta = 1
        const bool one = (PER_CHANNEL && at >= 2 * tb * DP && at < 3 * tb * DP) || (at >= used - tb && at < used);
        sm[e] = one ? 1.f : 0.f;
    }
    const int width = min(VT, vdim - c0);
    __syncthreads();

    auto fetch = [&](int j0, int which) {
        float* sq = sm + which * per_stage;
        float* sk = sq + tb * DP;
        float* sg = sk + tb * DP;
        float* sr = sg + tb * DP;
        float* sv = sk + (ARRAYS - 1) * tb * DP;
        float* sb = sv + tb * VT;
        const int m = min(tb, n - j0);
        if (vec) {
            const int quads = dim >> 2;
            for (int e = threadIdx.x; e < m * quads; e += blockDim.x) {
                const int j = e / quads, d = (e - j * quads) * 4;
                const size_t t = (size_t)(t0 + j0 + j);
                cp_async_f32x4(sq + j * DP + d, qk + ((t * 2) * kv_heads + hk) * dim + d);
                cp_async_f32x4(sk + j * DP + d, qk + ((t * 2 + 1) * kv_heads + hk) * dim + d);
                if (PER_CHANNEL) cp_async_f32x4(sg + j * DP + d, decay + (t * heads + h) * dim + d);
                if (GENERAL) cp_async_f32x4(sr + j * DP + d, rate + (t * heads + h) * dim + d);
            }
        } else {
            for (int e = threadIdx.x; e < m * dim; e += blockDim.x) {
                const int j = e / dim, d = e - j * dim;
                const size_t t = (size_t)(t0 + j0 + j);
                cp_async_f32(sq + j * DP + d, qk + ((t * 2) * kv_heads + hk) * dim + d);
                cp_async_f32(sk + j * DP + d, qk + ((t * 2 + 1) * kv_heads + hk) * dim + d);
                if (PER_CHANNEL) cp_async_f32(sg + j * DP + d, decay + (t * heads + h) * dim + d);
                if (GENERAL) cp_async_f32(sr + j * DP + d, rate + (t * heads + h) * dim + d);
            }
        }
        for (int e = threadIdx.x; e < m * width; e += blockDim.x) {
            const int j = e / width, x = e - j * width;
            cp_async_f32(sv + j * VT + x, v + ((size_t)(t0 + j0 + j) * heads + h) * vdim + c0 + x);
        }
        if ((DELTA || TOKEN) && (int)threadIdx.x < m)
            cp_async_f32(sb + threadIdx.x, (TOKEN ? head_decay : beta) + (size_t)(t0 + j0 + threadIdx.x) * heads + h);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    fetch(0, 0);
    int which = 0;
    float o_before = 0.f;                    // the token before's read-out, not yet summed over the column's lanes: its
    long at_before = -1;                     // sum rides along with this token's S^T k sum, so the two waits overlap
    for (int j0 = 0; j0 < n; j0 += tb, which ^= 1) {
        const int m = min(tb, n - j0);
        if (j0 + tb < n) {
            fetch(j0 + tb, which ^ 1);                                  // (that buffer was read a stage ago: barrier below)
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        const float* sq = sm + which * per_stage;
        const float* sk = sq + tb * DP;
        const float* sg = sk + tb * DP;
        const float* sr = sg + tb * DP;
        const float* sv = sk + (ARRAYS - 1) * tb * DP;
        const float* sb = sv + tb * VT;
#pragma unroll 2
        for (int j = 0; j < m; ++j) {
            const float4* kj = (const float4*)(sk + j * DP) + p;    // group i4 of this thread: kj[i4 * P]
            const float4* qj = (const float4*)(sq + j * DP) + p;
            float u = cl < VT ? sv[j * VT + cl] : 0.f;               // (threads past the tile carry zeros: the sums below are warp-wide)
            float4 k4[DPT / 4];
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) k4[i] = kj[i * P];
            if (GENERAL) {                                           // k . S on the state as it was, then decay, removal and write
                float a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int i = 0; i < DPT / 4; ++i) {
                    a0 = fmaf(S[4 * i], k4[i].x, a0); a1 = fmaf(S[4 * i + 1], k4[i].y, a1);
                    a0 = fmaf(S[4 * i + 2], k4[i].z, a0); a1 = fmaf(S[4 * i + 3], k4[i].w, a1);
                }
                float a = a0 + a1;
#pragma unroll
                for (int o = 1; o < P; o <<= 1) {
                    a += __shfl_xor_sync(0xffffffffu, a, o);
                    o_before += __shfl_xor_sync(0xffffffffu, o_before, o);
                }
                if (at_before >= 0 && p == 0 && col) out[((size_t)at_before * heads + h) * vdim + c] = o_before;
                const float4* gj = (const float4*)(sg + j * DP) + p;
                const float4* rj = (const float4*)(sr + j * DP) + p;
                float o0 = 0.f, o1 = 0.f;
#pragma unroll
                for (int i = 0; i < DPT / 4; ++i) {
                    const float4 g = gj[i * P], r = rj[i * P], q4 = qj[i * P];
                    S[4 * i] = fmaf(g.x, S[4 * i], k4[i].x * fmaf(-r.x, a, u));
                    S[4 * i + 1] = fmaf(g.y, S[4 * i + 1], k4[i].y * fmaf(-r.y, a, u));
                    S[4 * i + 2] = fmaf(g.z, S[4 * i + 2], k4[i].z * fmaf(-r.z, a, u));
                    S[4 * i + 3] = fmaf(g.w, S[4 * i + 3], k4[i].w * fmaf(-r.w, a, u));
                    o0 = fmaf(S[4 * i], q4.x, o0); o1 = fmaf(S[4 * i + 1], q4.y, o1);
                    o0 = fmaf(S[4 * i + 2], q4.z, o0); o1 = fmaf(S[4 * i + 3], q4.w, o1);
                }
                o_before = o0 + o1;
                at_before = t0 + j0 + j;
                continue;
            }
            if (PER_CHANNEL) {
                const float4* gj = (const float4*)(sg + j * DP) + p;
#pragma unroll
                for (int i = 0; i < DPT / 4; ++i) {
                    const float4 g = gj[i * P];
                    S[4 * i] *= g.x; S[4 * i + 1] *= g.y; S[4 * i + 2] *= g.z; S[4 * i + 3] *= g.w;
                }
            } else {
                if (TOKEN) fixed = sb[j];
#pragma unroll
                for (int i = 0; i < DPT; ++i) S[i] *= fixed;
            }
            if (DELTA) {
                float a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int i = 0; i < DPT / 4; ++i) {
                    a0 = fmaf(S[4 * i], k4[i].x, a0); a1 = fmaf(S[4 * i + 1], k4[i].y, a1);
                    a0 = fmaf(S[4 * i + 2], k4[i].z, a0); a1 = fmaf(S[4 * i + 3], k4[i].w, a1);
                }
                float a = a0 + a1;
#pragma unroll
                for (int o = 1; o < P; o <<= 1) {
                    a += __shfl_xor_sync(0xffffffffu, a, o);
                    o_before += __shfl_xor_sync(0xffffffffu, o_before, o);
                }
                u = sb[j] * (u - a);
            } else {
#pragma unroll
                for (int o = 1; o < P; o <<= 1) o_before += __shfl_xor_sync(0xffffffffu, o_before, o);
            }
            if (at_before >= 0 && p == 0 && col) out[((size_t)at_before * heads + h) * vdim + c] = o_before;
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int i = 0; i < DPT / 4; ++i) {
                const float4 q4 = qj[i * P];
                S[4 * i] = fmaf(k4[i].x, u, S[4 * i]);
                S[4 * i + 1] = fmaf(k4[i].y, u, S[4 * i + 1]);
                S[4 * i + 2] = fmaf(k4[i].z, u, S[4 * i + 2]);
                S[4 * i + 3] = fmaf(k4[i].w, u, S[4 * i + 3]);
                o0 = fmaf(S[4 * i], q4.x, o0); o1 = fmaf(S[4 * i + 1], q4.y, o1);
                o0 = fmaf(S[4 * i + 2], q4.z, o0); o1 = fmaf(S[4 * i + 3], q4.w, o1);
            }
            o_before = o0 + o1;
            at_before = t0 + j0 + j;
        }
        __syncthreads();                                            // this stage is read: the next fetch may fill it
    }
#pragma unroll
    for (int x = 1; x < P; x <<= 1) o_before += __shfl_xor_sync(0xffffffffu, o_before, x);
    if (at_before >= 0 && p == 0 && col) out[((size_t)at_before * heads + h) * vdim + c] = o_before;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = ((i >> 2) * P + p) * 4 + (i & 3);
        if (col && d < dim) S_g[d] = S[i];
    }
}

template <int DPT, int P>
static int launch_scan(float* out, const float* qk, const float* v, const float* decay, const float* head_decay,
                       const float* token_decay, const float* beta, const float* rate, float* state, const int32_t* query_start, const int32_t* row_slot, int rows,
                       int heads, int kv_heads, int dim, int vdim, int most, cudaStream_t s) {
    const int unit = 32 / P > 1 ? 32 / P : 1;                         // columns a warp holds
    int VT = vdim < 256 / P ? vdim : 256 / P;
    if (VT < 1) VT = 1;
    const int threads = ((VT + unit - 1) / unit) * unit * P;
    const int tiles = (vdim + VT - 1) / VT;
    const int per_token = (decay ? (rate ? 4 : 3) : 2) * P * DPT + VT + 1;
    int tb = 96 * 1024 / 8 / per_token;                               // two stages in at most 96 KB
    if (tb > SC_TB) tb = SC_TB;
    if (tb < 1) HB_REFUSE("recurrent_scan: key size %d needs more shared memory than a block has", dim);
    if (tb > threads) tb = threads;
    if (most > 0 && tb > most) tb = most;                             // (no row brings more tokens than that)
    const size_t smem = (size_t)2 * ((tb * per_token + 3) & ~3) * sizeof(float);
    auto kernel = decay ? (beta ? recurrent_scan_kernel<DPT, P, true, true> : recurrent_scan_kernel<DPT, P, true, false>)
                        : (beta ? recurrent_scan_kernel<DPT, P, false, true> : recurrent_scan_kernel<DPT, P, false, false>);
    if (token_decay) { kernel = recurrent_scan_kernel<DPT, P, false, false, true>; head_decay = token_decay; }
    if (rate) kernel = recurrent_scan_kernel<DPT, P, true, false, false, true>;
    if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<dim3(rows, heads, tiles), threads, smem, s>>>(out, qk, v, decay, head_decay, beta, rate, state, query_start, row_slot,
                                                          heads, kv_heads, dim, vdim, VT, tb);
    HB_LAUNCH_CHECK("recurrent_scan");
    return 0;
}

extern "C" int hb_recurrent_scan(float* out, const float* qk, const float* v, const float* decay, const float* head_decay,
                                 const float* token_decay, const float* beta, const float* rate, float* state, const int32_t* query_start, const int32_t* row_slot,
                                 int rows, int heads, int kv_heads, int dim, int vdim, int most, hb_stream stream) {
    if (rows == 0) return 0;
    if (kv_heads < 1 || heads % kv_heads) HB_REFUSE("recurrent_scan: %d heads are no multiple of %d key heads", heads, kv_heads);
    if (dim < 1 || dim > 1024 || vdim < 1) HB_REFUSE("recurrent_scan: key size %d (1 to 1024), value size %d", dim, vdim);
    if ((decay != nullptr) + (head_decay != nullptr) + (token_decay != nullptr) != 1) HB_REFUSE("recurrent_scan: give decays per channel and token, per head and token, or one per head");
    if (token_decay && beta) HB_REFUSE("recurrent_scan: the delta rule does not go with a decay per head and token");
    if (rate && (!decay || beta)) HB_REFUSE("recurrent_scan: removal rates per key channel go with decays per key channel and without beta");
    if (rows > 65535 * 32 || heads > 65535 || (vdim + 7) / 8 > 65535) HB_REFUSE("recurrent_scan: %d rows, %d heads, value size %d", rows, heads, vdim);
    if ((((uintptr_t)qk | (uintptr_t)decay | (uintptr_t)rate) & 15) != 0) HB_REFUSE("recurrent_scan: qk, decay and rate must lie on 16-byte boundaries");
    cudaStream_t s = (cudaStream_t)stream;
#define HB_SCAN(D, PP) return launch_scan<D, PP>(out, qk, v, decay, head_decay, token_decay, beta, rate, state, query_start, row_slot, rows, heads, \
                                                 kv_heads, dim, vdim, most, s)
    // Four channels a thread up to a key size of 64, then more channels a thread. (Key size 128, 2,048 tokens of 16 heads,
    // microseconds a token with the delta rule: 16 lanes of 8 channels 0.37, 32 lanes of 4 0.40, 8 lanes of 16 0.40, 4 lanes of
    // 32 0.51: a token is one chain of dependent steps whatever the lanes, and the warps of an SM fill one another's gaps.)
    if (dim <= 4) HB_SCAN(4, 1);
    if (dim <= 8) HB_SCAN(4, 2);
    if (dim <= 16) HB_SCAN(4, 4);
    if (dim <= 32) HB_SCAN(4, 8);
    if (dim <= 64) HB_SCAN(4, 16);
    if (dim <= 128) HB_SCAN(8, 16);
    if (dim <= 256) HB_SCAN(8, 32);
    if (dim <= 512) HB_SCAN(16, 32);
    HB_SCAN(32, 32);
#undef HB_SCAN
}

// ---------------------------------------------------------------- what the delta-rule mixer's first product becomes
// A token's row of `first` holds [q (kv_heads dim) | k (kv_heads dim) | v (heads vdim) | b (heads)], its row of `low2`
// (32-bit) the outputs of the two low-rank projections [a (heads dim) | g (heads vdim)].
// q, k, v pass a causal convolution over time (weights conv [channels, taps], the last tap the token's own; inputs
// before the step's first token of the row come from conv_state [slots, taps - 1, channels], oldest first) and silu;
// q and k become unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times q_scale. beta = sigmoid(b).
// decay[h, d] = exp(-exp(rate_log[h]) softplus(a[h dim + d] + dt_bias[h dim + d])), gate = sigmoid(g).
// grid (tokens, segments): the first segments take the q and k heads, a warp a head (the convolution twice: once for the
// sum of squares, once for the values); the others an element a thread of v, beta, the decays and the gate. No thread
// waits for another, so a step of a few tokens still spreads over many blocks.
template <typename T>
__global__ void delta_prepare_kernel(float* __restrict__ qk, float* __restrict__ v, float* __restrict__ beta,
                                     float* __restrict__ decay, float* __restrict__ gate, const T* __restrict__ first,
                                     int ld, const T* __restrict__ conv, int taps, const T* __restrict__ conv_state,
                                     const float* __restrict__ low2, const float* __restrict__ dt_bias,
                                     const float* __restrict__ rate_log, const int32_t* __restrict__ query_start,
                                     const int32_t* __restrict__ row_slot, int rows, int heads, int kv_heads, int dim,
                                     int vdim, float q_scale, float unit_eps) {
    const int t = blockIdx.x, seg = blockIdx.y;
    const int b = row_of_token(query_start, rows, t);
    const int t0 = query_start[b];
    const int nq = kv_heads * dim, nv = heads * vdim, C = 2 * nq + nv;
    const T* st = conv_state ? conv_state + (size_t)row_slot[b] * (taps - 1) * C : nullptr;
    auto channel = [&](int c) -> float {                               // convolution over time and silu of channel c
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int at = t - (taps - 1 - j);                           // the token this tap weighs
            const float x = at >= t0 ? to_f32(first[(size_t)at * ld + c]) : to_f32(st[(size_t)(taps - 1 + (at - t0)) * C + c]);
            acc = fmaf(to_f32(conv[(size_t)c * taps + j]), x, acc);
        }
        return silu_f(acc);
    };
    const int head_segments = (2 * kv_heads + 7) / 8;
    if (seg < head_segments) {                                          // unit vectors: q heads, then k heads
        const int g = seg * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
        if (g >= 2 * kv_heads) return;
        float ss = 0.f;
        for (int d = lane; d < dim; d += 32) { const float x = channel(g * dim + d); ss = fmaf(x, x, ss); }
        const float f = rsqrtf(warp_sum(ss) + unit_eps) * (g < kv_heads ? q_scale : 1.f);
        for (int d = lane; d < dim; d += 32) qk[((size_t)t * 2 * kv_heads + g) * dim + d] = channel(g * dim + d) * f;
        return;
    }
    int e = (seg - head_segments) * blockDim.x + threadIdx.x;
    if (e < nv) { v[(size_t)t * nv + e] = channel(2 * nq + e); return; }
    e -= nv;
    if (e < heads) { beta[(size_t)t * heads + e] = sigmoid_f(to_f32(first[(size_t)t * ld + C + e])); return; }
    e -= heads;
    const float* z = low2 + (size_t)t * (heads * dim + nv);
    if (e < heads * dim) {
        decay[(size_t)t * heads * dim + e] = expf(-expf(rate_log[e / dim]) * softplus_f(z[e] + dt_bias[e]));
        return;
    }
    e -= heads * dim;
    if (e < nv) gate[(size_t)t * nv + e] = sigmoid_f(z[heads * dim + e]);
}

extern "C" int hb_delta_prepare(float* qk, float* v, float* beta, float* decay, float* gate, const void* first, int dtype,
                                int ld, const void* conv, int taps, const void* conv_state, const float* low2,
                                const float* dt_bias, const float* rate_log, const int32_t* query_start,
                                const int32_t* row_slot, int rows, int tokens, int heads, int kv_heads, int dim, int vdim,
                                float q_scale, float unit_eps, hb_stream stream) {
    if (tokens == 0) return 0;
    if (taps < 1 || (taps > 1 && !conv_state)) HB_REFUSE("delta_prepare: %d taps need the carried inputs", taps);
    const long elements = 2L * heads * vdim + heads + (long)heads * dim;
    const long segments = (2 * kv_heads + 7) / 8 + (elements + 255) / 256;
    if (segments > 65535) HB_REFUSE("delta_prepare: %ld segments a token are above 65535", segments);
    dim3 grid(tokens, (unsigned)segments);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_ARGS(T) (const T*)first, ld, (const T*)conv, taps, (const T*)conv_state, low2, dt_bias, rate_log, \
    query_start, row_slot, rows, heads, kv_heads, dim, vdim, q_scale, unit_eps
    if (dtype == HB_F32) delta_prepare_kernel<float><<<grid, 256, 0, s>>>(qk, v, beta, decay, gate, HB_ARGS(float));
    else if (dtype == HB_BF16) delta_prepare_kernel<bf16><<<grid, 256, 0, s>>>(qk, v, beta, decay, gate, HB_ARGS(bf16));
    else HB_REFUSE("delta_prepare: dtype %d", dtype);
#undef HB_ARGS
    HB_LAUNCH_CHECK("delta_prepare");
    return 0;
}

// The carried inputs of the convolution after a step: the last taps - 1 inputs of (what was carried, the row's tokens).
// A thread per (row, channel); entry i takes what lies n places further on, so ascending i reads nothing written.
template <typename T>
__global__ void conv_carry_kernel(T* __restrict__ conv_state, const T* __restrict__ first, int ld, int C, int keep,
                                  const int32_t* __restrict__ query_start, const int32_t* __restrict__ row_slot) {
    const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int t0 = query_start[b], n = query_start[b + 1] - t0;
    T* st = conv_state + (size_t)row_slot[b] * keep * C;
    for (int i = 0; i < keep; ++i) {
        const int src = n - keep + i;                                // among the row's tokens; negative: carried before
        st[(size_t)i * C + c] = src >= 0 ? first[(size_t)(t0 + src) * ld + c] : st[(size_t)(keep + src) * C + c];
    }
}

extern "C" int hb_conv_carry(void* conv_state, const void* first, int dtype, int ld, int channels, int taps,
                             const int32_t* query_start, const int32_t* row_slot, int rows, hb_stream stream) {
    if (rows == 0 || taps <= 1) return 0;
    if (rows > 65535) HB_REFUSE("conv_carry: %d rows are above 65535", rows);
    dim3 grid((channels + 127) / 128, rows);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_F32) conv_carry_kernel<float><<<grid, 128, 0, s>>>((float*)conv_state, (const float*)first, ld, channels, taps - 1, query_start, row_slot);
    else if (dtype == HB_BF16) conv_carry_kernel<bf16><<<grid, 128, 0, s>>>((bf16*)conv_state, (const bf16*)first, ld, channels, taps - 1, query_start, row_slot);
    else HB_REFUSE("conv_carry: dtype %d", dtype);
    HB_LAUNCH_CHECK("conv_carry");
    return 0;
}

// ---------------------------------------------------------------- what the retention mixer's first product becomes
// A token's row of `first` holds [q (heads dim) | k (heads dim) | v (heads vdim) | ...]. q and k turn by the token's
// position (the first rot_dims channels of a head, half-split pairs, table [positions, rot_dims]: cosines then sines),
// k is then scaled. grid (tokens, segments of 256 elements).
template <typename T>
__global__ void retention_prepare_kernel(float* __restrict__ qk, float* __restrict__ v, const T* __restrict__ first, int ld,
                                         const int32_t* __restrict__ positions, const float* __restrict__ table,
                                         int rot_dims, int max_positions, int heads, int dim, int vdim, float k_scale) {
    const size_t t = blockIdx.x;
    const T* row = first + t * ld;
    const int pos = min(max(positions[t], 0), max_positions > 0 ? max_positions - 1 : 0);
    const float* cs = table ? table + (size_t)pos * rot_dims : nullptr;
    const int half = rot_dims >> 1, nq = heads * dim;
    int e = blockIdx.y * blockDim.x + threadIdx.x;                       // an element a thread: q and k, then v
    if (e < 2 * nq) {
        const int d = e % dim;
        float x = to_f32(row[e]);
        if (d < half) x = x * cs[d] - to_f32(row[e + half]) * cs[half + d];
        else if (d < rot_dims) x = x * cs[d - half] + to_f32(row[e - half]) * cs[d];
        qk[t * 2 * nq + e] = e >= nq ? x * k_scale : x;
        return;
    }
    e -= 2 * nq;
    if (e < heads * vdim) v[t * heads * vdim + e] = to_f32(row[2 * nq + e]);
}

extern "C" int hb_retention_prepare(float* qk, float* v, const void* first, int dtype, int ld, const int32_t* positions,
                                    const float* table, int rot_dims, int max_positions, int tokens, int heads, int dim,
                                    int vdim, float k_scale, hb_stream stream) {
    if (tokens == 0) return 0;
    if (rot_dims % 2 || rot_dims < 0 || rot_dims > dim) HB_REFUSE("retention_prepare: %d rotated channels of %d", rot_dims, dim);
    if (rot_dims && !table) HB_REFUSE("retention_prepare: a rotation needs its table");
    cudaStream_t s = (cudaStream_t)stream;
    const long segments = (2L * heads * dim + (long)heads * vdim + 255) / 256;
    if (segments > 65535) HB_REFUSE("retention_prepare: %ld segments a token are above 65535", segments);
    const dim3 tokens_by_segments(tokens, (unsigned)segments);
    if (dtype == HB_F32) retention_prepare_kernel<float><<<tokens_by_segments, 256, 0, s>>>(qk, v, (const float*)first, ld, positions, table, rot_dims, max_positions, heads, dim, vdim, k_scale);
    else if (dtype == HB_BF16) retention_prepare_kernel<bf16><<<tokens_by_segments, 256, 0, s>>>(qk, v, (const bf16*)first, ld, positions, table, rot_dims, max_positions, heads, dim, vdim, k_scale);
    else HB_REFUSE("retention_prepare: dtype %d", dtype);
    HB_LAUNCH_CHECK("retention_prepare");
    return 0;
}

// ---------------------------------------------------------------- per-head norm and output gate behind the scan
// out[t, h, :] = o / sqrt(mean(o^2) + eps) * weight * gate. `weight` [vdim], [heads vdim] (`weight_heads`) or null; the
// gate is either a ready multiplier in 32-bit (gate_mul [tokens, heads vdim]) or silu (`gate_sigmoid`: sigmoid) of a
// pre-activation in the engine's dtype (gate_pre, rows `ld` apart). One warp per (token, head).
template <typename T>
__global__ void head_norm_gate_kernel(T* __restrict__ out, const float* __restrict__ o, const float* __restrict__ weight,
                                      const float* __restrict__ gate_mul, const T* __restrict__ gate_pre, long ld,
                                      float eps, long items, int heads, int vdim, int weight_heads, int gate_sigmoid) {
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int lane = threadIdx.x & 31;
    const long t = item / heads;
    const int h = (int)(item - t * heads);
    const float* x = o + item * vdim;
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) ss += x[d] * x[d];
    const float f = rsqrtf(warp_sum(ss) / vdim + eps);
    for (int d = lane; d < vdim; d += 32) {
        float y = x[d] * f;
        if (weight) y *= weight[weight_heads ? h * vdim + d : d];
        if (gate_mul) y *= gate_mul[item * vdim + d];
        else if (gate_pre) {
            const float g = to_f32(gate_pre[t * ld + (long)h * vdim + d]);
            y *= gate_sigmoid ? sigmoid_f(g) : silu_f(g);
        }
        out[item * vdim + d] = from_f32<T>(y);
    }
}

extern "C" int hb_head_norm_gate(void* out, const float* o, int dtype, const float* weight, const float* gate_mul,
                                 const void* gate_pre, long ld, float eps, int tokens, int heads, int vdim,
                                 int weight_heads, int gate_sigmoid, hb_stream stream) {
    const long items = (long)tokens * heads;
    if (items == 0) return 0;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_F32) head_norm_gate_kernel<float><<<blocks, 128, 0, s>>>((float*)out, o, weight, gate_mul, (const float*)gate_pre, ld, eps, items, heads, vdim, weight_heads, gate_sigmoid);
    else if (dtype == HB_BF16) head_norm_gate_kernel<bf16><<<blocks, 128, 0, s>>>((bf16*)out, o, weight, gate_mul, (const bf16*)gate_pre, ld, eps, items, heads, vdim, weight_heads, gate_sigmoid);
    else HB_REFUSE("head_norm_gate: dtype %d", dtype);
    HB_LAUNCH_CHECK("head_norm_gate");
    return 0;
}

// ---------------------------------------------------------------- what the generalized delta rule's first product becomes
// A token's row of `first` holds [r | k | v | g | a], each heads dim wide, `ld` apart; `pre` (32-bit) [tokens, heads dim] is
// the low-rank pair's output. qk = (r, k) and v in 32-bit; decay = exp(-decay_scale sigmoid(pre + decay_bias));
// rate = sigmoid(a + rate_bias) / (sum over the head of k^2 + unit_eps): the removal along the unit key, as a factor on k.
// One warp per (token, head).
template <typename T>
__global__ void gdelta_prepare_kernel(float* __restrict__ qk, float* __restrict__ v, float* __restrict__ decay,
                                      float* __restrict__ rate, const T* __restrict__ first, long ld,
                                      const float* __restrict__ pre, const float* __restrict__ decay_bias,
                                      const float* __restrict__ rate_bias, long items, int heads, int dim,
                                      float decay_scale, float unit_eps) {
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int lane = threadIdx.x & 31;
    const long t = item / heads;
    const int h = (int)(item - t * heads);
    const long n = (long)heads * dim;
    const T* row = first + t * ld + (long)h * dim;
    float ss = 0.f;
    for (int d = lane; d < dim; d += 32) { const float k = to_f32(row[n + d]); ss = fmaf(k, k, ss); }
    const float inv = 1.f / (warp_sum(ss) + unit_eps);
    float* q_out = qk + ((t * 2) * heads + h) * dim;
    float* k_out = qk + ((t * 2 + 1) * heads + h) * dim;
    for (int d = lane; d < dim; d += 32) {
        const long at = item * dim + d;
        q_out[d] = to_f32(row[d]);
        k_out[d] = to_f32(row[n + d]);
        v[at] = to_f32(row[2 * n + d]);
        decay[at] = expf(-decay_scale * sigmoid_f(pre[at] + decay_bias[h * dim + d]));
        rate[at] = sigmoid_f(to_f32(row[4 * n + d]) + rate_bias[h * dim + d]) * inv;
    }
}

extern "C" int hb_gdelta_prepare(float* qk, float* v, float* decay, float* rate, const void* first, int dtype, long ld,
                                 const float* pre, const float* decay_bias, const float* rate_bias, int tokens, int heads,
                                 int dim, float decay_scale, float unit_eps, hb_stream stream) {
    const long items = (long)tokens * heads;
    if (items == 0) return 0;
    if (heads < 1 || dim < 1 || ld < 5L * heads * dim) HB_REFUSE("gdelta_prepare: %d heads of %d in rows of %ld", heads, dim, ld);
    const unsigned blocks = (unsigned)((items + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_F32) gdelta_prepare_kernel<float><<<blocks, 128, 0, s>>>(qk, v, decay, rate, (const float*)first, ld, pre, decay_bias, rate_bias, items, heads, dim, decay_scale, unit_eps);
    else if (dtype == HB_BF16) gdelta_prepare_kernel<bf16><<<blocks, 128, 0, s>>>(qk, v, decay, rate, (const bf16*)first, ld, pre, decay_bias, rate_bias, items, heads, dim, decay_scale, unit_eps);
    else HB_REFUSE("gdelta_prepare: dtype %d", dtype);
    HB_LAUNCH_CHECK("gdelta_prepare");
    return 0;
}
