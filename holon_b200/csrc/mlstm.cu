// The matrix memory with exponential gates (mLSTM): per head a state S [key channel, value channel] and a normaliser n
// [key channel], both scaled by exp(-m) for a running maximum m of the gates' logarithms, so that neither overflows:
//
//     i_t = cap tanh(a_t / cap),   f_t = logsigmoid(cap tanh(b_t / cap))        (a, b: the gates' pre-activations + bias)
//     m_t = max(f_t + m_(t-1), i_t)                                            (m starts at 0)
//     keep_t = exp(f_t + m_(t-1) - m_t),   take_t = exp(i_t - m_t)
//     S_t = keep_t S_(t-1) + take_t k_t v_t^T,   n_t = keep_t n_(t-1) + take_t k_t
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// n is kept as one more value column of S (the value row gets a 1 behind its last number), so the update is the scan of
// csrc/recurrent.cu with a decay per token and head (keep_t), keys take_t k_t and vdim + 1 value columns; its last output
// column is n_t . q_t. The kernels here make the scan's inputs and finish its outputs. Everything is 32-bit.
//
// hb_mlstm_gates     the gates' pre-activations -> keep, take, exp(-m) per token and head; m carried per slot and head
// hb_mlstm_prepare   a first product's rows [q | k | v | ...] -> q dim^(-1/2), take k, [v | 1] in 32-bit
// hb_mlstm_read_out  the scan's rows [S^T q | n . q] -> the quotient, each head divided by its root mean square, times a
//                    weight over all heads' channels, times sigmoid of the output gate's pre-activation
#include "common.cuh"

#define MG_CHUNK 1024
// One block per (row, head). A row's tokens pass in chunks of MG_CHUNK: all threads make i and f (the transcendental part),
// one thread walks the chain m_t = max(f_t + m_(t-1), i_t) (two dependent operations a token), all threads make the
// exponentials. out [3][tokens, heads]: keep, take, exp(-m).
__global__ void mlstm_gates_kernel(float* __restrict__ out, const float* __restrict__ pre, int ld,
                                   const void* __restrict__ bias, int bias_f32, float cap, float* __restrict__ m_state,
                                   const int32_t* __restrict__ query_start, const int32_t* __restrict__ row_slot,
                                   long tokens, int heads) {
    __shared__ float si[MG_CHUNK], sf[MG_CHUNK], sm[MG_CHUNK + 1];
    const int b = blockIdx.x, h = blockIdx.y;
    const int t0 = query_start[b], n = query_start[b + 1] - t0;
    float* m_g = m_state + (size_t)row_slot[b] * heads + h;
    const float bi = bias ? (bias_f32 ? ((const float*)bias)[h] : to_f32(((const bf16*)bias)[h])) : 0.f;
    const float bf = bias ? (bias_f32 ? ((const float*)bias)[heads + h] : to_f32(((const bf16*)bias)[heads + h])) : 0.f;
    const float inv_cap = 1.f / cap;
    float* keep = out;
    float* take = out + tokens * heads;
    float* floor_ = out + 2 * tokens * heads;
    if (threadIdx.x == 0) sm[0] = *m_g;
    for (int j0 = 0; j0 < n; j0 += MG_CHUNK) {
        const int m = min(MG_CHUNK, n - j0);
        for (int j = threadIdx.x; j < m; j += blockDim.x) {
            const float* row = pre + (size_t)(t0 + j0 + j) * ld;
            const float a = row[h] + bi, c = row[heads + h] + bf;
            si[j] = cap * tanhf(a * inv_cap);
            const float z = cap * tanhf(c * inv_cap);
            sf[j] = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));          // log sigmoid(z)
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float mx = sm[0];
#pragma unroll 8
            for (int j = 0; j < m; ++j) { mx = fmaxf(sf[j] + mx, si[j]); sm[j + 1] = mx; }    // (loads run ahead of the chain)
        }
        __syncthreads();
        for (int j = threadIdx.x; j < m; j += blockDim.x) {
            const size_t at = (size_t)(t0 + j0 + j) * heads + h;
            keep[at] = expf(sf[j] + sm[j] - sm[j + 1]);
            take[at] = expf(si[j] - sm[j + 1]);
            floor_[at] = expf(-sm[j + 1]);
        }
        __syncthreads();
        if (threadIdx.x == 0) sm[0] = sm[m];
    }
    __syncthreads();
    if (threadIdx.x == 0) *m_g = sm[0];
}

extern "C" int hb_mlstm_gates(float* out, const float* pre, int ld, const void* bias, int bias_dtype, float cap,
                              float* m_state, const int32_t* query_start, const int32_t* row_slot, int rows, int tokens,
                              int heads, hb_stream stream) {
    if (rows == 0 || tokens == 0) return 0;
    if (heads < 1 || heads > 65535 || ld < 2 * heads) HB_REFUSE("mlstm_gates: %d heads in rows of %d", heads, ld);
    if (!(cap > 0.f)) HB_REFUSE("mlstm_gates: the gates' cap must be positive");
    mlstm_gates_kernel<<<dim3(rows, heads), 128, 0, (cudaStream_t)stream>>>(out, pre, ld, bias, bias_dtype == HB_F32, cap, m_state,
                                                                           query_start, row_slot, (long)tokens, heads);
    HB_LAUNCH_CHECK("mlstm_gates");
    return 0;
}

// grid (tokens, segments of 256 of a token's 2 heads dim + heads (vdim + 1) numbers)
template <typename T>
__global__ void mlstm_prepare_kernel(float* __restrict__ qk, float* __restrict__ v1, const float* __restrict__ take,
                                     const T* __restrict__ first, int ld, int heads, int dim, int vdim, float q_scale) {
    const size_t t = blockIdx.x;
    const int e = blockIdx.y * blockDim.x + threadIdx.x;
    const int nq = heads * dim, nv = heads * (vdim + 1);
    const T* row = first + t * ld;
    if (e < nq) {
        qk[t * 2 * nq + e] = to_f32(row[e]) * q_scale;
    } else if (e < 2 * nq) {
        const int x = e - nq;
        qk[t * 2 * nq + e] = to_f32(row[e]) * take[t * heads + x / dim];
    } else if (e < 2 * nq + nv) {
        const int x = e - 2 * nq, h = x / (vdim + 1), d = x - h * (vdim + 1);
        v1[t * nv + x] = d < vdim ? to_f32(row[2 * nq + h * vdim + d]) : 1.f;
    }
}

extern "C" int hb_mlstm_prepare(float* qk, float* v1, const float* take, const void* first, int dtype, int ld, int tokens,
                                int heads, int dim, int vdim, float q_scale, hb_stream stream) {
    if (tokens == 0) return 0;
    const long per = 2L * heads * dim + (long)heads * (vdim + 1);
    const long segments = (per + 255) / 256;
    if (segments > 65535 || ld < 2 * heads * dim + heads * vdim) HB_REFUSE("mlstm_prepare: %ld numbers a token, rows of %d", per, ld);
    const dim3 grid(tokens, (unsigned)segments);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_F32) mlstm_prepare_kernel<float><<<grid, 256, 0, s>>>(qk, v1, take, (const float*)first, ld, heads, dim, vdim, q_scale);
    else if (dtype == HB_BF16) mlstm_prepare_kernel<bf16><<<grid, 256, 0, s>>>(qk, v1, take, (const bf16*)first, ld, heads, dim, vdim, q_scale);
    else HB_REFUSE("mlstm_prepare: dtype %d", dtype);
    HB_LAUNCH_CHECK("mlstm_prepare");
    return 0;
}

// One warp per (token, head). o1 [tokens, heads, vdim + 1]; floor_ [tokens, heads] = exp(-m); weight [heads vdim];
// gate_pre rows `ld` apart (sigmoid of it is the gate).
template <typename T>
__global__ void mlstm_read_out_kernel(T* __restrict__ out, const float* __restrict__ o1, const float* __restrict__ floor_,
                                      const void* __restrict__ weight, int weight_f32, const T* __restrict__ gate_pre,
                                      long ld, float eps, float tiny, long items, int heads, int vdim) {
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const int lane = threadIdx.x & 31;
    const long t = item / heads;
    const int h = (int)(item - t * heads);
    const float* x = o1 + item * (vdim + 1);
    const float inv = 1.f / (fmaxf(fabsf(x[vdim]), floor_[item]) + tiny);
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) { const float y = x[d] * inv; ss += y * y; }
    const float f = rsqrtf(warp_sum(ss) / vdim + eps);
    for (int d = lane; d < vdim; d += 32) {
        float y = x[d] * inv * f;
        const int c = h * vdim + d;
        y *= weight_f32 ? ((const float*)weight)[c] : to_f32(((const bf16*)weight)[c]);
        const float g = to_f32(gate_pre[t * ld + c]);
        y *= 1.f / (1.f + expf(-g));
        out[item * vdim + d] = from_f32<T>(y);
    }
}

extern "C" int hb_mlstm_read_out(void* out, const float* o1, const float* floor_, int dtype, const void* weight,
                                 int weight_dtype, const void* gate_pre, long ld, float eps, float tiny, int tokens, int heads,
                                 int vdim, hb_stream stream) {
    const long items = (long)tokens * heads;
    if (items == 0) return 0;
    if (!weight || !gate_pre) HB_REFUSE("mlstm_read_out: the weight and the gate's rows are needed");
    const unsigned blocks = (unsigned)((items + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_F32) mlstm_read_out_kernel<float><<<blocks, 128, 0, s>>>((float*)out, o1, floor_, weight, weight_dtype == HB_F32, (const float*)gate_pre, ld, eps, tiny, items, heads, vdim);
    else if (dtype == HB_BF16) mlstm_read_out_kernel<bf16><<<blocks, 128, 0, s>>>((bf16*)out, o1, floor_, weight, weight_dtype == HB_F32, (const bf16*)gate_pre, ld, eps, tiny, items, heads, vdim);
    else HB_REFUSE("mlstm_read_out: dtype %d", dtype);
    HB_LAUNCH_CHECK("mlstm_read_out");
    return 0;
}
