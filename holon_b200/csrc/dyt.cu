// A norm without statistics, N(x) = tanh(alpha x) w + b element by element (alpha one number; alpha, w, b in 32-bit), the
// residual sums around it, and the blend of a token's normed row with the row of the token before it.
//
// hb_dyt_add_norm   h += N_post(y);  out = N_pre(h)          (either half may be left out; rows may be gathered)
// hb_dyt_shift      x_t = h_t + N_post(y_t);  n_t = N_pre(x_t);  out_t = n_t + (n_(t-1) - n_t) mix
//                   with n_(t-1) of a row's first token carried per request slot, and the row's last n written there
// Nothing here sums over a row, so the grid is flat: a thread four neighbouring columns of one token (in the blend
// kernel, for prompts, of four tokens one after the other). 32-bit arithmetic,
// one rounding where the output is stored.
#include "common.cuh"

struct DytNorm {                    // null alpha: no such norm
    const float* alpha;
    const float* w;
    const float* b;
};

__device__ __forceinline__ float dyt_one(float x, float alpha, float w, float b) { return fmaf(tanhf(alpha * x), w, b); }

template <typename T>
__device__ __forceinline__ void load4(const T* p, bool vec, int left, float (&f)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, bool vec, int left, float (&f)[4]) {
    if (vec) { const float4 v = *(const float4*)p; f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; return; }
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = i < left ? p[i] : 0.f;
}
template <>
__device__ __forceinline__ void load4<bf16>(const bf16* p, bool vec, int left, float (&f)[4]) {
    if (vec) {
        const uint2 v = *(const uint2*)p;
        const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&v.x), c = __bfloat1622float2(*(const __nv_bfloat162*)&v.y);
        f[0] = a.x; f[1] = a.y; f[2] = c.x; f[3] = c.y;
        return;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = i < left ? __bfloat162float(p[i]) : 0.f;
}
__device__ __forceinline__ void store4(float* p, bool vec, int left, const float (&f)[4]) {
    if (vec) { *(float4*)p = make_float4(f[0], f[1], f[2], f[3]); return; }
#pragma unroll
    for (int i = 0; i < 4; ++i) if (i < left) p[i] = f[i];
}
__device__ __forceinline__ void store4(bf16* p, bool vec, int left, const float (&f)[4]) {
    if (vec) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), c = __floats2bfloat162_rn(f[2], f[3]);
        *(uint2*)p = make_uint2(*(const uint32_t*)&a, *(const uint32_t*)&c);
        return;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) if (i < left) p[i] = __float2bfloat16_rn(f[i]);
}

// x = (h ? h[src row] : 0) + (y ? N_post(y[src row]) or, without h, y itself : 0); out[r] = N_pre(x).
// TY: the type of y; TO: the type of out.
template <typename TY, typename TO>
__global__ void dyt_add_norm_kernel(float* __restrict__ h, const TY* __restrict__ y, DytNorm post, TO* __restrict__ out,
                                    DytNorm pre, const int32_t* __restrict__ index, int dim, int vec) {
    const size_t r = blockIdx.x;
    const int d = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (d >= dim) return;
    const int left = dim - d;
    const size_t src = index ? (size_t)index[r] : r;
    float x[4] = {0.f, 0.f, 0.f, 0.f}, w[4], b[4];
    if (h) load4<float>(h + src * dim + d, vec, left, x);
    if (y) {
        float z[4];
        load4<TY>(y + src * dim + d, vec, left, z);
        if (post.alpha) {
            const float a = *post.alpha;
            load4<float>(post.w + d, vec, left, w);
            load4<float>(post.b + d, vec, left, b);
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] += dyt_one(z[i], a, w[i], b[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] += z[i];
        }
        if (h && !index) store4(h + src * dim + d, vec, left, x);
    }
    if (out) {
        const float a = *pre.alpha;
        load4<float>(pre.w + d, vec, left, w);
        load4<float>(pre.b + d, vec, left, b);
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = dyt_one(x[i], a, w[i], b[i]);
        store4(out + r * dim + d, vec, left, x);
    }
}

extern "C" int hb_dyt_add_norm(float* h, const void* y, int y_dtype, const float* post_alpha, const float* post_w,
                               const float* post_b, void* out, int out_dtype, const float* pre_alpha, const float* pre_w,
                               const float* pre_b, const int32_t* index, int rows, int dim, hb_stream stream) {
    if (rows == 0 || dim == 0) return 0;
    if (!h && !y) HB_REFUSE("dyt_add_norm: neither a stream nor an input");
    if (out && !pre_alpha) HB_REFUSE("dyt_add_norm: an output without its norm");
    if (!y) y_dtype = HB_F32;
    if (!out) out_dtype = HB_F32;
    const int vec = dim % 4 == 0 && (((uintptr_t)h | (uintptr_t)y | (uintptr_t)out | (uintptr_t)post_w | (uintptr_t)post_b |
                                      (uintptr_t)pre_w | (uintptr_t)pre_b) & 15) == 0;
    const int quads = (dim + 3) / 4, threads = quads >= 256 ? 256 : ((quads + 31) / 32) * 32;
    const dim3 grid(rows, (quads + threads - 1) / threads);
    const DytNorm post{post_alpha, post_w, post_b}, pre{pre_alpha, pre_w, pre_b};
    cudaStream_t s = (cudaStream_t)stream;
#define HB_RUN(TY, TO) dyt_add_norm_kernel<TY, TO><<<grid, threads, 0, s>>>(h, (const TY*)y, post, (TO*)out, pre, index, dim, vec)
    if (y_dtype == HB_F32 && out_dtype == HB_F32) HB_RUN(float, float);
    else if (y_dtype == HB_BF16 && out_dtype == HB_BF16) HB_RUN(bf16, bf16);
    else if (y_dtype == HB_F32 && out_dtype == HB_BF16) HB_RUN(float, bf16);
    else if (y_dtype == HB_BF16 && out_dtype == HB_F32) HB_RUN(bf16, float);
    else HB_REFUSE("dyt_add_norm: dtypes %d, %d", y_dtype, out_dtype);
#undef HB_RUN
    HB_LAUNCH_CHECK("dyt_add_norm");
    return 0;
}

// The row b with query_start[b] <= t < query_start[b + 1].
__device__ __forceinline__ int dyt_row_of_token(const int32_t* __restrict__ query_start, int rows, int t) {
    int lo = 0, hi = rows;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (query_start[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

// grid (groups of `walk` tokens, column segments): a thread walks the tokens of its group for its four columns and keeps
// the normed row it made for the next token (the group's first token recomputes the row before it, unless it is a row's
// first). The thread that meets a row's first token reads what the slot carries and then, alone, writes the row's last
// normed row there (which it computes itself): no other thread touches those four numbers.
template <typename TY, typename TO>
__global__ void dyt_shift_kernel(TO* __restrict__ out, float* __restrict__ into, const float* __restrict__ h,
                                 const TY* __restrict__ y, DytNorm post, DytNorm pre, const float* __restrict__ mix,
                                 float* __restrict__ carried, const int32_t* __restrict__ query_start,
                                 const int32_t* __restrict__ row_slot, int rows, int tokens, int dim, int vec, int walk) {
    const int first_token = blockIdx.x * walk, end = min(tokens, first_token + walk);
    const int d = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (d >= dim) return;
    const int left = dim - d;
    float wq[4], bq[4], wp[4], bp[4], mu[4];
    const float ap = *pre.alpha, aq = post.alpha ? *post.alpha : 0.f;
    load4<float>(pre.w + d, vec, left, wp);
    load4<float>(pre.b + d, vec, left, bp);
    load4<float>(mix + d, vec, left, mu);
    if (y && post.alpha) { load4<float>(post.w + d, vec, left, wq); load4<float>(post.b + d, vec, left, bq); }
    auto summed = [&](int at, float (&x)[4]) {                       // the stream's row of token `at` with what is pending
        load4<float>(h + (size_t)at * dim + d, vec, left, x);
        if (y) {
            float z[4];
            load4<TY>(y + (size_t)at * dim + d, vec, left, z);
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] += post.alpha ? dyt_one(z[i], aq, wq[i], bq[i]) : z[i];
        }
    };
    int b = dyt_row_of_token(query_start, rows, first_token);
    float before[4];
    bool have = false;                                               // `before` holds the normed row of token t - 1
    for (int t = first_token; t < end; ++t) {
        while (t >= query_start[b + 1]) ++b;                         // (rows without tokens are passed over)
        const int t0 = query_start[b], t1 = query_start[b + 1];
        float x[4], n[4];
        summed(t, x);
        if (y || into != h) store4(into + (size_t)t * dim + d, vec, left, x);
#pragma unroll
        for (int i = 0; i < 4; ++i) n[i] = dyt_one(x[i], ap, wp[i], bp[i]);
        if (t == t0) {
            float* kept = carried + (size_t)row_slot[b] * dim + d;
            load4<float>(kept, vec, left, before);
            if (t1 - 1 == t) {
                store4(kept, vec, left, n);
            } else {
                float xl[4];
                summed(t1 - 1, xl);
#pragma unroll
                for (int i = 0; i < 4; ++i) xl[i] = dyt_one(xl[i], ap, wp[i], bp[i]);
                store4(kept, vec, left, xl);
            }
        } else if (!have) {
            summed(t - 1, before);
#pragma unroll
            for (int i = 0; i < 4; ++i) before[i] = dyt_one(before[i], ap, wp[i], bp[i]);
        }
        float o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { o[i] = fmaf(before[i] - n[i], mu[i], n[i]); before[i] = n[i]; }
        have = true;
        store4(out + (size_t)t * dim + d, vec, left, o);
    }
}

extern "C" int hb_dyt_shift(void* out, int out_dtype, float* into, const float* h, const void* y, int y_dtype,
                            const float* post_alpha, const float* post_w, const float* post_b, const float* pre_alpha,
                            const float* pre_w, const float* pre_b, const float* mix, float* carried,
                            const int32_t* query_start, const int32_t* row_slot, int rows, int tokens, int dim,
                            hb_stream stream) {
    if (tokens == 0 || dim == 0 || rows == 0) return 0;
    if (y && into == h) HB_REFUSE("dyt_shift: with a pending output the sums need a tensor of their own");
    if (!y) y_dtype = HB_F32;
    const int vec = dim % 4 == 0 && (((uintptr_t)h | (uintptr_t)into | (uintptr_t)y | (uintptr_t)out | (uintptr_t)post_w |
                                      (uintptr_t)post_b | (uintptr_t)pre_w | (uintptr_t)pre_b | (uintptr_t)mix |
                                      (uintptr_t)carried) & 15) == 0;
    const int quads = (dim + 3) / 4, threads = quads >= 256 ? 256 : ((quads + 31) / 32) * 32;
    const int walk = tokens >= 1024 ? 4 : 1;            // prompts: a thread four tokens; the few rows of a decode step: one each
    const dim3 grid((tokens + walk - 1) / walk, (quads + threads - 1) / threads);
    const DytNorm post{post_alpha, post_w, post_b}, pre{pre_alpha, pre_w, pre_b};
    cudaStream_t s = (cudaStream_t)stream;
#define HB_RUN(TY, TO) dyt_shift_kernel<TY, TO><<<grid, threads, 0, s>>>((TO*)out, into, h, (const TY*)y, post, pre, mix, carried, \
                                                                         query_start, row_slot, rows, tokens, dim, vec, walk)
    if (y_dtype == HB_F32 && out_dtype == HB_F32) HB_RUN(float, float);
    else if (y_dtype == HB_BF16 && out_dtype == HB_BF16) HB_RUN(bf16, bf16);
    else if (y_dtype == HB_F32 && out_dtype == HB_BF16) HB_RUN(float, bf16);
    else HB_REFUSE("dyt_shift: dtypes %d, %d", y_dtype, out_dtype);
#undef HB_RUN
    HB_LAUNCH_CHECK("dyt_shift");
    return 0;
}
