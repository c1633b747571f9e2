// Embedding gather, RMSNorm with the residual sum folded in, SwiGLU's activation.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512] = "";
void hb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}
extern "C" const char* hb_last_error(void) { return g_error; }
extern "C" int hb_version(void) { return 1; }

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table, const int32_t* __restrict__ ids,
                             int hidden, int vocab) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* row = table + (size_t)(ok ? id : 0) * hidden;
    float* o = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = ok ? to_f32(row[i]) : 0.f;
}
// The same for a bfloat16 table whose rows are a multiple of 8 wide: 16 bytes a load, all of a thread's loads in flight
// before the first is used (a row of 4,096 is two loads a thread instead of sixteen in a row).
__global__ void embed_bf16x8_kernel(float* __restrict__ out, const bf16* __restrict__ table, const int32_t* __restrict__ ids,
                                    int hidden, int vocab) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const uint4* row = (const uint4*)(table + (size_t)(ok ? id : 0) * hidden);
    float4* o = (float4*)(out + (size_t)t * hidden);
    const int pieces = hidden >> 3;
    for (int i0 = threadIdx.x; i0 < pieces; i0 += 4 * blockDim.x) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * blockDim.x;
            v[u] = ok && i < pieces ? __ldg(row + i) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * blockDim.x;
            if (i < pieces) {
                const __nv_bfloat162* h = (const __nv_bfloat162*)&v[u];
                const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), c = __bfloat1622float2(h[2]), d = __bfloat1622float2(h[3]);
                o[2 * i] = make_float4(a.x, a.y, b.x, b.y);
                o[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
            }
        }
    }
}

extern "C" int hb_embed(float* out, const void* table, int table_dtype, const int32_t* ids, int tokens, int hidden,
                        int vocab, hb_stream stream) {
    if (tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == HB_F32) embed_kernel<float><<<tokens, threads, 0, s>>>(out, (const float*)table, ids, hidden, vocab);
    else if (table_dtype == HB_BF16 && hidden % 8 == 0 && (((uintptr_t)table | (uintptr_t)out) % 16) == 0)
        embed_bf16x8_kernel<<<tokens, threads, 0, s>>>(out, (const bf16*)table, ids, hidden, vocab);
    else if (table_dtype == HB_BF16) embed_kernel<bf16><<<tokens, threads, 0, s>>>(out, (const bf16*)table, ids, hidden, vocab);
    else HB_REFUSE("embed: table dtype %d", table_dtype);
    HB_LAUNCH_CHECK("embed");
    return 0;
}

// ---------------------------------------------------------------- (add +) RMSNorm
// One block per output row. The row is kept in shared memory as 32-bit between the two passes.
// VEC: dim is a multiple of 4 and every pointer is 16-byte aligned per row, so a thread moves 4 values at a time.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) { const float4 x = *(const float4*)p; v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) { *(float4*)p = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
        const uint2 x = *(const uint2*)p;
        const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&x.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&x.y);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 x; x.x = *(uint32_t*)&a; x.y = *(uint32_t*)&b;
        *(uint2*)p = x;
    }
};

template <typename TH, typename TD, typename TW, bool VEC>
__global__ void add_rmsnorm_kernel(TD* __restrict__ out, TH* h, const TD* __restrict__ delta,
                                   const TW* __restrict__ weight, float eps, float offset,
                                   const int32_t* __restrict__ index, int dim) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t t = index ? (size_t)index[r] : (size_t)r;
    TH* hr = h + t * dim;
    const TD* dr = delta ? delta + t * dim : nullptr;
    const bool write_back = delta != nullptr && index == nullptr;
    float ss = 0.f;
    if (VEC && dim <= (int)blockDim.x * 4) {
        // A thread holds its (at most) four values in registers and reads the weight before the block-wide sum, so
        // that load's latency passes while the sum is formed; the values and their order are those of the loops below.
        const int i = threadIdx.x * 4;
        float v[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
        if (i < dim) {
            float d[4];
            Vec4<TH>::load(hr + i, v);
            if (dr) {
                Vec4<TD>::load(dr + i, d);
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] += d[k];
            }
            Vec4<TW>::load(weight + i, w);
            if (write_back) Vec4<TH>::store(hr + i, v);
            ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        }
        const float rstd = rsqrtf(block_sum(ss, scratch) / (float)dim + eps);
        if (i < dim) {
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = v[k] * rstd * (w[k] + offset);
            Vec4<TD>::store(out + (size_t)r * dim + i, v);
        }
        return;
    }
    if (VEC) {
        for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
            float v[4], d[4];
            Vec4<TH>::load(hr + i, v);
            if (dr) {
                Vec4<TD>::load(dr + i, d);
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] += d[k];
            }
            if (write_back) Vec4<TH>::store(hr + i, v);
            *(float4*)(row + i) = make_float4(v[0], v[1], v[2], v[3]);
            ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            float v = to_f32(hr[i]);
            if (dr) v += to_f32(dr[i]);
            if (write_back) hr[i] = from_f32<TH>(v);
            row[i] = v;
            ss += v * v;
        }
    }
    const float total = block_sum(ss, scratch);
    const float rstd = rsqrtf(total / (float)dim + eps);
    TD* o = out + (size_t)r * dim;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
            float w[4], v[4];
            Vec4<TW>::load(weight + i, w);
            const float4 x = *(const float4*)(row + i);
            v[0] = x.x * rstd * (w[0] + offset); v[1] = x.y * rstd * (w[1] + offset);
            v[2] = x.z * rstd * (w[2] + offset); v[3] = x.w * rstd * (w[3] + offset);
            Vec4<TD>::store(o + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x)
            o[i] = from_f32<TD>(row[i] * rstd * (to_f32(weight[i]) + offset));
    }
}

template <typename TH, typename TD, typename TW>
static int launch_add_rmsnorm(void* out, void* h, const void* delta, const void* weight, float eps, float offset,
                              const int32_t* index, int rows, int dim, cudaStream_t s) {
    const size_t smem = (size_t)dim * sizeof(float);
    if (smem > 200 * 1024) HB_REFUSE("rmsnorm: a row of %d values does not fit shared memory (limit 51200)", dim);
    const bool vec = dim % 4 == 0 && (((uintptr_t)out | (uintptr_t)h | (uintptr_t)delta | (uintptr_t)weight) % 16 == 0);
    auto kernel = vec ? add_rmsnorm_kernel<TH, TD, TW, true> : add_rmsnorm_kernel<TH, TD, TW, false>;
    if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int per = vec ? 4 : 1;
    int threads = dim >= 4096 * per ? 1024 : (dim >= 1024 * per ? 512 : (dim >= 256 * per ? 256 : 128));
    if (vec && dim <= 4096 && rows <= 256) threads = (dim / 4 + 31) / 32 * 32;   // few rows (latency counts): a row in one pass, four values a thread in registers
    kernel<<<rows, threads, smem, s>>>((TD*)out, (TH*)h, (const TD*)delta, (const TW*)weight, eps, offset, index, dim);
    HB_LAUNCH_CHECK("add_rmsnorm");
    return 0;
}

extern "C" int hb_add_rmsnorm(void* out, int out_dtype, void* h, int h_dtype, const void* delta, const void* weight,
                              int weight_dtype, float eps, float offset, const int32_t* index, int rows, int dim,
                              hb_stream stream) {
    if (rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (h_dtype != HB_F32 && delta) HB_REFUSE("add_rmsnorm: the residual stream must be float32 when a delta is added");
#define HB_CASE(H, D, W, TH, TD, TW) if (h_dtype == H && out_dtype == D && weight_dtype == W) \
    return launch_add_rmsnorm<TH, TD, TW>(out, h, delta, weight, eps, offset, index, rows, dim, s);
    HB_CASE(HB_F32, HB_F32, HB_F32, float, float, float)
    HB_CASE(HB_F32, HB_BF16, HB_BF16, float, bf16, bf16)
    HB_CASE(HB_F32, HB_BF16, HB_F32, float, bf16, float)
    HB_CASE(HB_BF16, HB_BF16, HB_BF16, bf16, bf16, bf16)
    HB_CASE(HB_BF16, HB_BF16, HB_F32, bf16, bf16, float)
#undef HB_CASE
    HB_REFUSE("add_rmsnorm: no kernel for dtypes h=%d out=%d weight=%d", h_dtype, out_dtype, weight_dtype);
}

// ---------------------------------------------------------------- silu(gate) * up
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, c = i % inter;
        const float g = to_f32(gate_up[t * 2 * inter + c]), u = to_f32(gate_up[t * 2 * inter + inter + c]);
        out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
    }
}

// bfloat16 with inter a multiple of 8: a thread takes 8 gates and 8 ups as two 16-byte loads.
__global__ void silu_mul_bf16x8_kernel(bf16* __restrict__ out, const bf16* __restrict__ gate_up, int inter, size_t groups) {
    const int per_row = inter >> 3;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / per_row, c = (i % per_row) << 3;
        const uint4 g4 = *(const uint4*)(gate_up + t * 2 * inter + c), u4 = *(const uint4*)(gate_up + t * 2 * inter + inter + c);
        const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 g = __bfloat1622float2(*(const __nv_bfloat162*)&gw[k]), u = __bfloat1622float2(*(const __nv_bfloat162*)&uw[k]);
            __nv_bfloat162 r = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y);
            ow[k] = *(uint32_t*)&r;
        }
        *(uint4*)(out + t * inter + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

extern "C" int hb_silu_mul(void* out, const void* gate_up, int dtype, int tokens, int inter, hb_stream stream) {
    const size_t total = (size_t)tokens * inter;
    if (total == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    if (dtype == HB_BF16 && inter % 8 == 0 && (((uintptr_t)out | (uintptr_t)gate_up) % 16 == 0)) {
        const size_t groups = total / 8;
        const int blocks = (int)((groups + threads - 1) / threads < 148 * 32 ? (groups + threads - 1) / threads : 148 * 32);
        silu_mul_bf16x8_kernel<<<blocks, threads, 0, s>>>((bf16*)out, (const bf16*)gate_up, inter, groups);
        HB_LAUNCH_CHECK("silu_mul");
        return 0;
    }
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == HB_F32) silu_mul_kernel<float><<<blocks, threads, 0, s>>>((float*)out, (const float*)gate_up, inter, total);
    else if (dtype == HB_BF16) silu_mul_kernel<bf16><<<blocks, threads, 0, s>>>((bf16*)out, (const bf16*)gate_up, inter, total);
    else HB_REFUSE("silu_mul: dtype %d", dtype);
    HB_LAUNCH_CHECK("silu_mul");
    return 0;
}

// ---------------------------------------------------------------- embedding with a scale and a table of token pairs
// out[t] = table[id] * scale + pair[r], r = (previous id * mul_prev + id * mul_cur) mod buckets, or `buckets` (the pair
// table's last row) for a sequence's first token (position 0). The previous id is the step's token before, or, for a
// row's first token in this step, what `prev` [slots] holds for the row's slot; the block of a row's first token then
// stores the row's last id there for the next step (it alone reads and writes that cell in this launch).
template <typename T>
__global__ void embed_pair_kernel(float* __restrict__ out, const T* __restrict__ table, float scale,
                                  const T* __restrict__ pair, const int32_t* __restrict__ ids,
                                  const int32_t* __restrict__ positions, const int32_t* __restrict__ query_start,
                                  const int32_t* __restrict__ row_slot, int32_t* __restrict__ prev, int rows, int hidden,
                                  int vocab, long mul_prev, long mul_cur, int buckets) {
    const int t = blockIdx.x;
    __shared__ int s_before;
    if (threadIdx.x == 0) {
        int lo = 0, hi = rows;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (query_start[mid] <= t) lo = mid; else hi = mid;
        }
        int before;
        if (t > query_start[lo]) before = ids[t - 1];
        else {
            before = prev[row_slot[lo]];
            prev[row_slot[lo]] = ids[query_start[lo + 1] - 1];
        }
        s_before = before;
    }
    __syncthreads();
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* row = table + (size_t)(ok ? id : 0) * hidden;
    const T* extra = nullptr;
    if (pair && ok) {
        long r = buckets;
        if (positions[t] > 0) {
            r = ((long)s_before * mul_prev + (long)id * mul_cur) % buckets;
            if (r < 0) r += buckets;
        }
        extra = pair + (size_t)r * hidden;
    }
    float* o = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        o[i] = ok ? to_f32(row[i]) * scale + (extra ? to_f32(extra[i]) : 0.f) : 0.f;
}

extern "C" int hb_embed_pair(float* out, const void* table, int table_dtype, float scale, const void* pair,
                             const int32_t* ids, const int32_t* positions, const int32_t* query_start,
                             const int32_t* row_slot, int32_t* prev, int rows, int tokens, int hidden, int vocab,
                             long mul_prev, long mul_cur, int buckets, hb_stream stream) {
    if (tokens == 0) return 0;
    if (pair && (buckets < 1 || !prev)) HB_REFUSE("embed_pair: a pair table needs buckets >= 1 and the slots' previous ids");
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 1024 ? 256 : 128;
#define HB_ARGS(T) out, (const T*)table, scale, (const T*)pair, ids, positions, query_start, row_slot, prev, rows, hidden, \
    vocab, mul_prev, mul_cur, buckets
    if (table_dtype == HB_F32) embed_pair_kernel<float><<<tokens, threads, 0, s>>>(HB_ARGS(float));
    else if (table_dtype == HB_BF16) embed_pair_kernel<bf16><<<tokens, threads, 0, s>>>(HB_ARGS(bf16));
    else HB_REFUSE("embed_pair: table dtype %d", table_dtype);
#undef HB_ARGS
    HB_LAUNCH_CHECK("embed_pair");
    return 0;
}

// ---------------------------------------------------------------- the residual sum of a block whose parts run side by side
// h[t, :] += sum_i scale_i x_i[t, :] + bias, in 32-bit; up to four terms of the engine's dtype, bias [hidden] or null.
template <typename T>
__global__ void sum_into_kernel(float* __restrict__ h, const T* __restrict__ x0, const T* __restrict__ x1,
                                const T* __restrict__ x2, const T* __restrict__ x3, float s0, float s1, float s2, float s3,
                                const T* __restrict__ bias, long count, int hidden) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float a = h[i];
    if (x0) a = fmaf(s0, to_f32(x0[i]), a);
    if (x1) a = fmaf(s1, to_f32(x1[i]), a);
    if (x2) a = fmaf(s2, to_f32(x2[i]), a);
    if (x3) a = fmaf(s3, to_f32(x3[i]), a);
    if (bias) a += to_f32(bias[i % hidden]);
    h[i] = a;
}

// The same, four neighbouring values a thread (hidden a multiple of 4, pointers on 16-byte boundaries).
template <typename T>
__global__ void sum_into4_kernel(float* __restrict__ h, const T* __restrict__ x0, const T* __restrict__ x1,
                                 const T* __restrict__ x2, const T* __restrict__ x3, float s0, float s1, float s2, float s3,
                                 const T* __restrict__ bias, long quads, int hidden) {
    const long q = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= quads) return;
    const long i = q * 4;
    float a[4], x[4];
    Vec4<float>::load(h + i, a);
    const T* terms[4] = {x0, x1, x2, x3};
    const float scales[4] = {s0, s1, s2, s3};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (terms[k]) {
            Vec4<T>::load(terms[k] + i, x);
#pragma unroll
            for (int e = 0; e < 4; ++e) a[e] = fmaf(scales[k], x[e], a[e]);
        }
    }
    if (bias) {
        Vec4<T>::load(bias + i % hidden, x);
#pragma unroll
        for (int e = 0; e < 4; ++e) a[e] += x[e];
    }
    Vec4<float>::store(h + i, a);
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

extern "C" int hb_sum_into(float* h, const void* x0, const void* x1, const void* x2, const void* x3, float s0, float s1,
                           float s2, float s3, const void* bias, int dtype, int tokens, int hidden, hb_stream stream) {
    const long count = (long)tokens * hidden;
    if (count == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (hidden % 4 == 0 && aligned16(h) && aligned16(x0) && aligned16(x1) && aligned16(x2) && aligned16(x3) && aligned16(bias)
        && (dtype == HB_F32 || dtype == HB_BF16)) {
        const long quads = count / 4;
        const unsigned blocks4 = (unsigned)((quads + 255) / 256);
        if (dtype == HB_F32) sum_into4_kernel<float><<<blocks4, 256, 0, s>>>(h, (const float*)x0, (const float*)x1, (const float*)x2, (const float*)x3, s0, s1, s2, s3, (const float*)bias, quads, hidden);
        else sum_into4_kernel<bf16><<<blocks4, 256, 0, s>>>(h, (const bf16*)x0, (const bf16*)x1, (const bf16*)x2, (const bf16*)x3, s0, s1, s2, s3, (const bf16*)bias, quads, hidden);
        HB_LAUNCH_CHECK("sum_into");
        return 0;
    }
    const unsigned blocks = (unsigned)((count + 255) / 256);
    if (dtype == HB_F32) sum_into_kernel<float><<<blocks, 256, 0, s>>>(h, (const float*)x0, (const float*)x1, (const float*)x2, (const float*)x3, s0, s1, s2, s3, (const float*)bias, count, hidden);
    else if (dtype == HB_BF16) sum_into_kernel<bf16><<<blocks, 256, 0, s>>>(h, (const bf16*)x0, (const bf16*)x1, (const bf16*)x2, (const bf16*)x3, s0, s1, s2, s3, (const bf16*)bias, count, hidden);
    else HB_REFUSE("sum_into: dtype %d", dtype);
    HB_LAUNCH_CHECK("sum_into");
    return 0;
}

// ---------------------------------------------------------------- a gated unit with clamped inputs
// gate_up [tokens, 2 inter] (gate columns first), bias [2 inter] or null: g = min(gate + b, limit),
// u = clamp(up + b, -limit, limit), out = g sigmoid(alpha g) (u + 1), in 32-bit with one rounding.
template <typename T>
__global__ void glu_clamped_kernel(T* __restrict__ out, const T* __restrict__ gate_up, const T* __restrict__ bias,
                                   float limit, float alpha, int inter) {
    const size_t t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    float g = to_f32(gate_up[t * 2 * inter + i]), u = to_f32(gate_up[t * 2 * inter + inter + i]);
    if (bias) { g += to_f32(bias[i]); u += to_f32(bias[inter + i]); }
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    out[t * inter + i] = from_f32<T>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
}

// The same, four neighbouring values a thread (inter a multiple of 4, pointers on 16-byte boundaries).
template <typename T>
__global__ void glu_clamped4_kernel(T* __restrict__ out, const T* __restrict__ gate_up, const T* __restrict__ bias,
                                    float limit, float alpha, int inter) {
    const size_t t = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= inter) return;
    float g[4], u[4], b[4], y[4];
    Vec4<T>::load(gate_up + t * 2 * inter + i, g);
    Vec4<T>::load(gate_up + t * 2 * inter + inter + i, u);
    if (bias) {
        Vec4<T>::load(bias + i, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) g[e] += b[e];
        Vec4<T>::load(bias + inter + i, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) u[e] += b[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float ge = fminf(g[e], limit), ue = fminf(fmaxf(u[e], -limit), limit);
        y[e] = ge / (1.f + expf(-alpha * ge)) * (ue + 1.f);
    }
    Vec4<T>::store(out + t * inter + i, y);
}

extern "C" int hb_glu_clamped(void* out, const void* gate_up, const void* bias, int dtype, float limit, float alpha,
                              int tokens, int inter, hb_stream stream) {
    if (tokens == 0 || inter == 0) return 0;
    if (tokens > 65535) HB_REFUSE("glu_clamped: %d rows are above 65535", tokens);
    cudaStream_t s = (cudaStream_t)stream;
    if (inter % 4 == 0 && aligned16(out) && aligned16(gate_up) && aligned16(bias) && (dtype == HB_F32 || dtype == HB_BF16)) {
        dim3 grid4((inter / 4 + 255) / 256, tokens);
        if (dtype == HB_F32) glu_clamped4_kernel<float><<<grid4, 256, 0, s>>>((float*)out, (const float*)gate_up, (const float*)bias, limit, alpha, inter);
        else glu_clamped4_kernel<bf16><<<grid4, 256, 0, s>>>((bf16*)out, (const bf16*)gate_up, (const bf16*)bias, limit, alpha, inter);
        HB_LAUNCH_CHECK("glu_clamped");
        return 0;
    }
    dim3 grid((inter + 255) / 256, tokens);
    if (dtype == HB_F32) glu_clamped_kernel<float><<<grid, 256, 0, s>>>((float*)out, (const float*)gate_up, (const float*)bias, limit, alpha, inter);
    else if (dtype == HB_BF16) glu_clamped_kernel<bf16><<<grid, 256, 0, s>>>((bf16*)out, (const bf16*)gate_up, (const bf16*)bias, limit, alpha, inter);
    else HB_REFUSE("glu_clamped: dtype %d", dtype);
    HB_LAUNCH_CHECK("glu_clamped");
    return 0;
}

// ---------------------------------------------------------------- the block's sum and the next block's norm in one
// h[t, :] += sum_i scale_i x_i[t, :] + bias as hb_sum_into, and out[t, :] = h[t, :] rsqrt(mean(h[t, :]^2) + eps)
// (weight + offset): one block a row, the summed row kept in shared memory between the two passes.
template <typename T, typename TW, bool VEC>
__global__ void sum_norm_kernel(float* __restrict__ h, const T* __restrict__ x0, const T* __restrict__ x1,
                                const T* __restrict__ x2, const T* __restrict__ x3, float s0, float s1, float s2, float s3,
                                const T* __restrict__ bias, T* __restrict__ out, const TW* __restrict__ weight, float eps,
                                float offset, int hidden) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * hidden;
    float ss = 0.f;
    if constexpr (VEC) {                          // four neighbouring values a thread and turn, every load of a turn in flight at once
        const T* terms[4] = {x0, x1, x2, x3};
        const float scales[4] = {s0, s1, s2, s3};
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float a[4], x[4][4], b[4] = {0.f, 0.f, 0.f, 0.f};
            Vec4<float>::load(h + base + i, a);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (terms[k]) Vec4<T>::load(terms[k] + base + i, x[k]);
            if (bias) Vec4<T>::load(bias + i, b);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (terms[k]) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) a[e] = fmaf(scales[k], x[k][e], a[e]);
                }
#pragma unroll
            for (int e = 0; e < 4; ++e) { a[e] += b[e]; ss = fmaf(a[e], a[e], ss); }
            Vec4<float>::store(h + base + i, a);
            Vec4<float>::store(row + i, a);
        }
        const float f = rsqrtf(block_sum(ss, scratch) / hidden + eps);
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float a[4], w[4];
            Vec4<float>::load(row + i, a);
            Vec4<TW>::load(weight + i, w);
#pragma unroll
            for (int e = 0; e < 4; ++e) a[e] = a[e] * f * (w[e] + offset);
            Vec4<T>::store(out + base + i, a);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float a = h[base + i];
            if (x0) a = fmaf(s0, to_f32(x0[base + i]), a);
            if (x1) a = fmaf(s1, to_f32(x1[base + i]), a);
            if (x2) a = fmaf(s2, to_f32(x2[base + i]), a);
            if (x3) a = fmaf(s3, to_f32(x3[base + i]), a);
            if (bias) a += to_f32(bias[i]);
            h[base + i] = a;
            row[i] = a;
            ss = fmaf(a, a, ss);
        }
        const float f = rsqrtf(block_sum(ss, scratch) / hidden + eps);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x)
            out[base + i] = from_f32<T>(row[i] * f * (to_f32(weight[i]) + offset));
    }
}

extern "C" int hb_sum_norm(float* h, const void* x0, const void* x1, const void* x2, const void* x3, float s0, float s1,
                           float s2, float s3, const void* bias, int dtype, void* out, const void* weight, int weight_dtype,
                           float eps, float offset, int tokens, int hidden, hb_stream stream) {
    if (tokens == 0 || hidden == 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) HB_REFUSE("sum_norm: rows of %d values are more than a block's shared memory holds", hidden);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = hidden >= 2048 ? 512 : 256;
    const bool vec = hidden % 4 == 0 && aligned16(h) && aligned16(x0) && aligned16(x1) && aligned16(x2) && aligned16(x3)
        && aligned16(bias) && aligned16(out) && aligned16(weight);
#define HB_RUN(T, TW) do { \
        auto kernel = vec ? sum_norm_kernel<T, TW, true> : sum_norm_kernel<T, TW, false>; \
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kernel<<<tokens, threads, smem, s>>>(h, (const T*)x0, (const T*)x1, (const T*)x2, (const T*)x3, s0, s1, s2, s3, \
                                            (const T*)bias, (T*)out, (const TW*)weight, eps, offset, hidden); } while (0)
    if (dtype == HB_F32 && weight_dtype == HB_F32) HB_RUN(float, float);
    else if (dtype == HB_BF16 && weight_dtype == HB_BF16) HB_RUN(bf16, bf16);
    else if (dtype == HB_BF16 && weight_dtype == HB_F32) HB_RUN(bf16, float);
    else HB_REFUSE("sum_norm: no kernel for dtype %d with weight dtype %d", dtype, weight_dtype);
#undef HB_RUN
    HB_LAUNCH_CHECK("sum_norm");
    return 0;
}

// ---------------------------------------------------------------- a norm on a sublayer's OUTPUT, and the depth average
// dst[r] = src[r] + N(y[r] + bias), N(z) = z * rsqrt(mean(z^2) + eps) * (weight + offset): the block "x <- x + norm(f(x))",
// whose sublayers read the stream itself. y null: dst[r] = src[r] (nothing is normed). With `hist` (n_hist tensors
// [rows, dim], hist_stride elements apart, of which dst is the last): avg[r] = sum_j coef[j] hist[j][r] in the order of j,
// the average over everything earlier layers and the embedding have left. `cast` (or null) gets the rows that go on
// (avg with hist, else dst) in the storage type `cast_dtype`: what the next sublayer's products read. 32-bit throughout.
// One block per row; the row waits in shared memory between the two passes.
template <typename T>
__device__ __forceinline__ void out_norm_row(float* __restrict__ dst, const float* __restrict__ src, const T* __restrict__ y,
                                             const void* __restrict__ bias, int bias_f32, const void* __restrict__ weight,
                                             int weight_f32, float eps, float offset, const float* __restrict__ hist,
                                             long hist_stride, int n_hist, const float* __restrict__ coef,
                                             float* __restrict__ avg, void* __restrict__ cast, int cast_dtype, int dim,
                                             float* row, float* scratch) {
    const size_t r = blockIdx.x;
    float ss = 0.f;
    if (y) {
        for (int d = threadIdx.x; d < dim; d += blockDim.x) {
            float z = to_f32(y[r * dim + d]);
            if (bias) z += bias_f32 ? ((const float*)bias)[d] : to_f32(((const bf16*)bias)[d]);
            row[d] = z;
            ss += z * z;
        }
        ss = block_sum(ss, scratch);
    }
    const float scale = rsqrtf(ss / (float)dim + eps);
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float x = src[r * dim + d];
        if (y) {
            const float w = (weight_f32 ? ((const float*)weight)[d] : to_f32(((const bf16*)weight)[d])) + offset;
            x += row[d] * scale * w;
        }
        if (y || dst != src) dst[r * dim + d] = x;
        float go = x;
        if (hist) {
            go = 0.f;
            for (int j = 0; j + 1 < n_hist; ++j) go = fmaf(coef[j], hist[(size_t)j * hist_stride + r * dim + d], go);
            go = fmaf(coef[n_hist - 1], x, go);
            avg[r * dim + d] = go;
        }
        if (cast) {
            if (cast_dtype == HB_F32) ((float*)cast)[r * dim + d] = go;
            else ((bf16*)cast)[r * dim + d] = __float2bfloat16_rn(go);
        }
    }
}

template <typename T>
__global__ void out_norm_add_kernel(float* dst, const float* src, const T* y, const void* bias, int bias_f32,
                                    const void* weight, int weight_f32, float eps, float offset, const float* hist,
                                    long hist_stride, int n_hist, const float* coef, float* avg, void* cast, int cast_dtype,
                                    int dim) {
    extern __shared__ float on_row[];
    __shared__ float scratch[33];
    out_norm_row<T>(dst, src, y, bias, bias_f32, weight, weight_f32, eps, offset, hist, hist_stride, n_hist, coef, avg, cast,
                    cast_dtype, dim, on_row, scratch);
}

extern "C" int hb_out_norm_add(float* dst, const float* src, const void* y, int y_dtype, const void* bias, int bias_dtype,
                               const void* weight, int weight_dtype, float eps, float offset, const float* hist,
                               long hist_stride, int n_hist, const float* coef, float* avg, void* cast, int cast_dtype,
                               int rows, int dim, hb_stream stream) {
    if (rows == 0) return 0;
    if (dim < 1 || (size_t)dim * sizeof(float) > 200 * 1024) HB_REFUSE("out_norm_add: rows of %d numbers", dim);
    if (y && !weight) HB_REFUSE("out_norm_add: a norm needs its weight");
    if (hist && (n_hist < 1 || !coef || !avg)) HB_REFUSE("out_norm_add: the depth average needs its coefficients and a place for the result");
    if (hist && dst != hist + (size_t)(n_hist - 1) * hist_stride) HB_REFUSE("out_norm_add: the layer's result is the last of the kept ones");
    const size_t smem = (size_t)dim * sizeof(float);
    const int threads = dim >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (y_dtype == HB_F32 || !y) {
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(out_norm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        out_norm_add_kernel<float><<<rows, threads, smem, s>>>(dst, src, (const float*)y, bias, bias_dtype == HB_F32, weight,
            weight_dtype == HB_F32, eps, offset, hist, hist_stride, n_hist, coef, avg, cast, cast_dtype, dim);
    } else if (y_dtype == HB_BF16) {
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(out_norm_add_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        out_norm_add_kernel<bf16><<<rows, threads, smem, s>>>(dst, src, (const bf16*)y, bias, bias_dtype == HB_F32, weight,
            weight_dtype == HB_F32, eps, offset, hist, hist_stride, n_hist, coef, avg, cast, cast_dtype, dim);
    } else HB_REFUSE("out_norm_add: dtype %d", y_dtype);
    HB_LAUNCH_CHECK("out_norm_add");
    return 0;
}
