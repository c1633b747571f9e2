// Attention whose heads share their softmax weights after the softmax ("talking heads"), over a paged cache that keeps a
// token's key and value of one kv head side by side in one row (key_dim + value_dim numbers, the two sizes free of one
// another): cache [pages, kv_heads, page_size, key_dim + value_dim].
//
//   p_g(i, j)   = softmax_j(q_g(i) . k_kv(g)(j) * scale * head_scale[g]) over the keys j that i may see
//   out_h(i)    = sum_j (sum_g talk[h, g] p_g(i, j)) v_kv(h)(j)  =  sum_g talk[h, g] (sum_j p_g(i, j) v_kv(h)(j))
//
// so a query head's weights are applied to the values of EVERY kv head, normalised by that head's own denominator, and
// the mixing matrix then takes what each output head needs: no weight ever leaves its kernel. Which keys a query at
// position i sees: j <= i, with `chunk` C > 0 only those of its own block (j >= floor(i / C) C, blocks counted from the
// sequence's first token), with `window` W > 0 only j > i - W. Scores, weights and sums are 32-bit whatever the storage.
//
// hb_qkv_talking_prepare  a first product's rows [q | k | v] -> bias, per-head RMSNorm of q and k, rotation, the value
//                         blend with an earlier layer's values, q rows and the cache's [k | v] rows
// hb_attention_talking    any sizes on CUDA cores, 32-bit arithmetic: the float32 engine's kernel, and the bfloat16
//                         engine's for one-token rows and for sizes the tensor-core kernel refuses. With `splits` > 1 a
//                         token's keys are cut into that many parts, a block each, and a second kernel merges the
//                         parts (running maxima, sums, weighted values) and mixes the heads: rows of one token then
//                         fill the GPU. Where every row has one token and the sizes allow, the parts run on a kernel
//                         that stages the keys and values in shared memory once for all heads (talking_rows1_kernel).
// hb_talking_mix          the mixing alone, for rows whose per-(query head, kv head) results the tensor-core prompt
//                         kernel (csrc/attention_tcgen05.cu, value_heads = kv_heads) has left
#include "common.cuh"

__device__ __forceinline__ float load_any(const void* p, int f32, size_t i) {
    return f32 ? ((const float*)p)[i] : to_f32(((const bf16*)p)[i]);
}

// ---------------------------------------------------------------- from the first product to q rows and cache rows
// One warp per (token, head slot): heads query slots, kv_heads key slots, kv_heads value slots. A q or k head: x + bias,
// x / sqrt(mean(x^2) + eps) * weight (if a weight is given), the first rot_dims channels turned by the token's position:
// in neighbouring pairs (2c, 2c + 1) if `interleaved`, else in half-split pairs (c, c + rot_dims / 2); `table` holds, per
// position, the rot_dims / 2 cosines and then the sines. One rounding, at the end. A value head: x + bias; with `blend`,
// (1 - blend[0]) x + blend[0] first[t, slot, :]; with `keep`, the 32-bit value is also left there for later layers.
#define TP_WARPS 4
#define TP_PER_LANE 16            // head sizes up to 512
template <typename T>
__global__ void talking_prepare_kernel(T* __restrict__ q_out, T* __restrict__ kv, float* __restrict__ keep,
                                       const T* __restrict__ qkv, const void* __restrict__ bias, int bias_f32,
                                       const void* __restrict__ q_weight, const void* __restrict__ k_weight, int weight_f32,
                                       float eps, const int32_t* __restrict__ positions, const float* __restrict__ table,
                                       int rot_dims, int table_rows, int interleaved, const float* __restrict__ first,
                                       const float* __restrict__ blend, const int32_t* __restrict__ write_index,
                                       int pages, int page_size, int tokens, int heads, int kv_heads, int kd, int vd) {
    extern __shared__ float tp_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slots = heads + 2 * kv_heads;
    const long item = (long)blockIdx.x * TP_WARPS + warp;
    if (item >= (long)tokens * slots) return;
    const int t = (int)(item / slots), slot = (int)(item % slots);
    const int width = heads * kd + kv_heads * (kd + vd);
    const T* row = qkv + (size_t)t * width;
    const long w = write_index ? write_index[t] : -1;
    const bool stored = w >= 0 && w < (long)pages * page_size;
    const int rowlen = kd + vd;
    if (slot >= heads + kv_heads) {                                   // a value head
        const int c = slot - heads - kv_heads, at = heads * kd + kv_heads * kd + c * vd;
        const float lam = blend ? blend[0] : 0.f;
        T* dst = stored ? kv + (((size_t)(w / page_size) * kv_heads + c) * page_size + w % page_size) * rowlen + kd : nullptr;
        for (int d = lane; d < vd; d += 32) {
            float x = to_f32(row[at + d]) + (bias ? load_any(bias, bias_f32, at + d) : 0.f);
            if (keep) keep[((size_t)t * kv_heads + c) * vd + d] = x;
            if (blend) x = (1.f - lam) * x + lam * first[((size_t)t * kv_heads + c) * vd + d];
            if (dst) dst[d] = from_f32<T>(x);
        }
        return;
    }
    const bool is_q = slot < heads;
    const int head = is_q ? slot : slot - heads, at = is_q ? head * kd : heads * kd + head * kd;
    const void* weight = is_q ? q_weight : k_weight;
    float* ys = tp_smem + (size_t)warp * kd;
    float x[TP_PER_LANE], ss = 0.f;
#pragma unroll
    for (int i = 0; i < TP_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        x[i] = d < kd ? to_f32(row[at + d]) + (bias ? load_any(bias, bias_f32, at + d) : 0.f) : 0.f;
        ss += x[i] * x[i];
    }
    const float r = weight ? rsqrtf(warp_sum(ss) / (float)kd + eps) : 1.f;
#pragma unroll
    for (int i = 0; i < TP_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < kd) ys[d] = weight ? x[i] * r * load_any(weight, weight_f32, d) : x[i];
    }
    __syncwarp();
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= table_rows && table_rows > 0 ? table_rows - 1 : pos);
    const float* cs = table ? table + (size_t)pos * rot_dims : nullptr;
    const int half = rot_dims >> 1;
    T* dst = is_q ? q_out + ((size_t)t * heads + head) * kd
                  : (stored ? kv + (((size_t)(w / page_size) * kv_heads + head) * page_size + w % page_size) * rowlen : nullptr);
    if (!dst) return;
    for (int d = lane; d < kd; d += 32) {
        float y = ys[d];
        if (cs && d < rot_dims) {
            int c, partner; bool lead;                                // lead: the pair's first member (u of (u, v))
            if (interleaved) { c = d >> 1; partner = d ^ 1; lead = (d & 1) == 0; }
            else { lead = d < half; c = lead ? d : d - half; partner = lead ? d + half : d - half; }
            const float co = cs[c], si = cs[half + c], o = ys[partner];
            y = lead ? y * co - o * si : y * co + o * si;
        }
        dst[d] = from_f32<T>(y);
    }
}

extern "C" int hb_qkv_talking_prepare(void* q_out, void* kv, float* keep, const void* qkv, int dtype, const void* bias,
                                      int bias_dtype, const void* q_weight, const void* k_weight, int weight_dtype, float eps,
                                      const int32_t* positions, const float* table, int rot_dims, int table_rows,
                                      int interleaved, const float* first, const float* blend, const int32_t* write_index,
                                      int pages, int page_size, int tokens, int heads, int kv_heads, int key_dim,
                                      int value_dim, hb_stream stream) {
    if (tokens == 0) return 0;
    if (key_dim < 1 || key_dim > 32 * TP_PER_LANE || value_dim < 1) HB_REFUSE("qkv_talking_prepare: key size %d (1 to %d), value size %d", key_dim, 32 * TP_PER_LANE, value_dim);
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > key_dim) HB_REFUSE("qkv_talking_prepare: %d rotated channels of %d", rot_dims, key_dim);
    if (rot_dims && !table) HB_REFUSE("qkv_talking_prepare: a rotation needs its table");
    if ((q_weight == nullptr) != (k_weight == nullptr)) HB_REFUSE("qkv_talking_prepare: give both norm weights or none");
    if (blend && !first) HB_REFUSE("qkv_talking_prepare: a blend needs the first layer's values");
    const long items = (long)tokens * (heads + 2 * kv_heads);
    const unsigned blocks = (unsigned)((items + TP_WARPS - 1) / TP_WARPS);
    const size_t smem = (size_t)TP_WARPS * key_dim * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (!rot_dims) table = nullptr;
    if (dtype == HB_F32)
        talking_prepare_kernel<float><<<blocks, TP_WARPS * 32, smem, s>>>(
            (float*)q_out, (float*)kv, keep, (const float*)qkv, bias, bias_dtype == HB_F32, q_weight, k_weight,
            weight_dtype == HB_F32, eps, positions, table, rot_dims, table_rows, interleaved, first, blend, write_index, pages,
            page_size, tokens, heads, kv_heads, key_dim, value_dim);
    else if (dtype == HB_BF16)
        talking_prepare_kernel<bf16><<<blocks, TP_WARPS * 32, smem, s>>>(
            (bf16*)q_out, (bf16*)kv, keep, (const bf16*)qkv, bias, bias_dtype == HB_F32, q_weight, k_weight,
            weight_dtype == HB_F32, eps, positions, table, rot_dims, table_rows, interleaved, first, blend, write_index, pages,
            page_size, tokens, heads, kv_heads, key_dim, value_dim);
    else HB_REFUSE("qkv_talking_prepare: dtype %d", dtype);
    HB_LAUNCH_CHECK("qkv_talking_prepare");
    return 0;
}

// ---------------------------------------------------------------- the attention, any sizes, CUDA cores
// One block per query token, a warp per query head (a warp takes several heads in turn where there are more than
// TK_WARPS). A lane scores one key of a block of 32 (q in shared memory), the block's weights then sweep the value rows
// of all kv heads: a lane owns every 32nd of the kv_heads * value_dim output numbers of its head (EPL of them). The
// normalised results of all heads wait in shared memory, wide [heads][kv_heads * value_dim], and the block's threads then
// mix them: out[h, d] = sum_g talk[h, g] wide[g][kv(h) value_dim + d] (talk null: the head's own result).
#define TK_WARPS 16
// out[h, d] = sum_g talk[h, g] wide[g][kv(h) value_dim + d] for one token, by all threads of the block.
template <typename T>
__device__ __forceinline__ void talking_mix_store(T* __restrict__ out, const float* wide, const float* __restrict__ talk,
                                                  size_t t, int heads, int kv_heads, int vd) {
    const int group = heads / kv_heads, all = kv_heads * vd;
    for (int e = threadIdx.x; e < heads * vd; e += blockDim.x) {
        const int h = e / vd, d = e - h * vd, at = (h / group) * vd + d;
        float o;
        if (talk) {
            o = 0.f;
            for (int g = 0; g < heads; ++g) o = fmaf(talk[h * heads + g], wide[(size_t)g * all + at], o);
        } else {
            o = wide[(size_t)h * all + at];
        }
        out[(t * heads + h) * vd + d] = from_f32<T>(o);
    }
}

// SPLIT: block (t, s) takes the s-th part of token t's keys and leaves, per head, its maximum, its sum and its weighted
// values (not normalised) in partial [tokens, splits, heads, kv_heads value_dim + 2]; hb_talking_merge finishes.
// VEC: a lane owns runs of four neighbouring numbers (4 lane + 128 i .. + 3) and loads each run at once; the sizes must
// then be multiples of four and the pool aligned (the launcher sees to it). Else it owns every 32nd number.
__device__ __forceinline__ void load_run4(const bf16* p, float v[4]) {
    const uint2 w = *(const uint2*)p;                        // (a bfloat16 is the upper half of the float32 of the same value)
    v[0] = __uint_as_float(w.x << 16); v[1] = __uint_as_float(w.x & 0xffff0000u);
    v[2] = __uint_as_float(w.y << 16); v[3] = __uint_as_float(w.y & 0xffff0000u);
}
__device__ __forceinline__ void load_run4(const float* p, float v[4]) {
    const float4 w = *(const float4*)p;
    v[0] = w.x; v[1] = w.y; v[2] = w.z; v[3] = w.w;
}

template <typename T, int EPL, bool SPLIT, bool VEC>
__global__ void __launch_bounds__(TK_WARPS * 32) attention_talking_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ kv,
                                         const int32_t* __restrict__ block_table, int table_stride,
                                         const int32_t* __restrict__ row_slot, const int32_t* __restrict__ query_start,
                                         const int32_t* __restrict__ kv_len, int rows, int heads, int kv_heads, int kd,
                                         int vd, int pages, int page_size, float scale,
                                         const float* __restrict__ head_scale, int chunk, int window,
                                         const float* __restrict__ talk, float* __restrict__ partial) {
    extern __shared__ float tk_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int t = blockIdx.x;
    const int all = kv_heads * vd, rowlen = kd + vd;
    float* wide = tk_smem;                                   // [heads][all] (not with SPLIT)
    float* qs = wide + (SPLIT ? 0 : (size_t)heads * all) + (size_t)warp * kd;

    int lo = 0, hi = rows;                                   // the row b with query_start[b] <= t < query_start[b + 1]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (query_start[mid] <= t) lo = mid; else hi = mid;
    }
    const int b = lo;
    const int n = kv_len[b];
    const int pos = n - query_start[b + 1] + t;              // the query's position in its sequence
    const bool live = n > 0 && pos >= 0;
    const int32_t* table = block_table + (size_t)row_slot[b] * table_stride;
    int first = 0;
    if (live && chunk > 0) first = (pos / chunk) * chunk;
    if (live && window > 0) first = max(first, pos - window + 1);
    int last = pos;                                          // this block's keys: first .. last
    if (SPLIT && live) {
        const int splits = gridDim.y, per = (((pos - first + splits) / splits) + 31) & ~31;
        first += (int)blockIdx.y * per;
        last = min(pos, first + per - 1);
    }
    const long head_shift = (long)page_size * rowlen;        // from a kv head's row to the next kv head's row of the token
    const bool vec16 = (kd & 7) == 0 && (rowlen & 7) == 0 && ((uintptr_t)kv & 15) == 0;

    long off[EPL];                                           // element e = lane + 32 i of [kv head][value]: where it lies
#pragma unroll                                               // relative to the token's row of kv head 0
    for (int i = 0; i < EPL; ++i) {
        const int e = VEC ? 4 * lane + 128 * (i >> 2) + (i & 3) : lane + 32 * i;
        off[i] = e < all ? (long)(e / vd) * head_shift + kd + e % vd : -1;
    }
    for (int g = warp; g < heads; g += warps) {
        float acc[EPL];
#pragma unroll
        for (int i = 0; i < EPL; ++i) acc[i] = 0.f;
        float m = -INFINITY, l = 0.f;
        if (live) {
            const float sc = scale * (head_scale ? head_scale[g] : 1.f);
            const T* qr = q + ((size_t)t * heads + g) * kd;
            __syncwarp();
            for (int d = lane; d < kd; d += 32) qs[d] = to_f32(qr[d]);
            __syncwarp();
            const int hk = g / (heads / kv_heads);
            for (int j0 = first; j0 <= last; j0 += 32) {
                const int j = j0 + lane;
                long base = -1;                              // element offset of key j's row of kv head 0
                if (j <= last) {
                    const int page = table[j / page_size];
                    if (page >= 0 && page < pages) base = (((long)page * kv_heads) * page_size + j % page_size) * rowlen;
                }
                float s = -INFINITY;
                if (base >= 0) {
                    const T* kr = kv + base + hk * head_shift;
                    float dot = 0.f;
                    if (sizeof(T) == 2 && vec16) {           // a row of bfloat16 in pieces of 16 bytes
                        const uint4* k4 = (const uint4*)kr;
                        float d4[4] = {0.f, 0.f, 0.f, 0.f};
                        for (int c = 0; c < (kd >> 3); ++c) {
                            const uint4 w = k4[c];
                            const uint32_t u[4] = {w.x, w.y, w.z, w.w};
                            const float* qc = qs + 8 * c;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {    // (a bfloat16 is the upper half of the float32 of the same value)
                                d4[i] = fmaf(qc[2 * i], __uint_as_float(u[i] << 16), d4[i]);
                                d4[i] = fmaf(qc[2 * i + 1], __uint_as_float(u[i] & 0xffff0000u), d4[i]);
                            }
                        }
                        dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
                    } else {
                        for (int d = 0; d < kd; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
                    }
                    s = dot * sc;
                }
                const float m_new = fmaxf(m, warp_max(s));
                const float corr = m_new == -INFINITY ? 1.f : expf(m - m_new);
                const float p = base >= 0 ? expf(s - m_new) : 0.f;
                l = l * corr + warp_sum(p);
                m = m_new;
#pragma unroll
                for (int i = 0; i < EPL; ++i) acc[i] *= corr;
                const int count = min(32, last - j0 + 1);
#pragma unroll 4
                for (int jj = 0; jj < count; ++jj) {         // (no branch inside: the loads of several keys fly together)
                    const float pj = __shfl_sync(0xffffffffu, p, jj);
                    long bj = __shfl_sync(0xffffffffu, base, jj);
                    bj = bj < 0 ? 0 : bj;                    // (a key without a page has weight 0: any row of finite numbers serves)
                    if (VEC) {
#pragma unroll
                        for (int r = 0; r < EPL / 4; ++r) {  // (a run past the row's end reads the row's start: its sums are dropped)
                            float v[4];
                            load_run4(kv + bj + (off[4 * r] >= 0 ? off[4 * r] : 0), v);
#pragma unroll
                            for (int k = 0; k < 4; ++k) acc[4 * r + k] = fmaf(pj, v[k], acc[4 * r + k]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < EPL; ++i)
                            if (off[i] >= 0) acc[i] = fmaf(pj, to_f32(kv[bj + off[i]]), acc[i]);
                    }
                }
            }
        }
        if (SPLIT) {
            float* part = partial + (((size_t)t * gridDim.y + blockIdx.y) * heads + g) * (all + 2);
            if (lane == 0) { part[0] = m; part[1] = l; }
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                const int e = VEC ? 4 * lane + 128 * (i >> 2) + (i & 3) : lane + 32 * i;
                if (e < all) part[2 + e] = acc[i];
            }
            continue;
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int e = VEC ? 4 * lane + 128 * (i >> 2) + (i & 3) : lane + 32 * i;
            if (e < all) wide[(size_t)g * all + e] = acc[i] * inv;
        }
    }
    if (SPLIT) return;
    __syncthreads();
    talking_mix_store<T>(out, wide, talk, (size_t)t, heads, kv_heads, vd);
}

// Rows of one token, staged: block (t, s) brings tiles of R1_KEYS keys of its part, the rows [key | value] of every kv
// head, into shared memory once (16 bytes a load, rows padded against bank conflicts), and all heads work on them:
// a thread a (head, key) pair for the scores, a warp a head for the running maximum and sum, and for the values a thread
// owns a run of four numbers of the kv_heads * value_dim wide row under HPT heads (their weights come from shared memory
// four at a time). Leaves the same partial results as the kernel above with SPLIT; hb's merge kernel finishes.
#define R1_KEYS 32
#define R1_THREADS 512
template <typename T, int HPT>
__global__ void __launch_bounds__(R1_THREADS) talking_rows1_kernel(
        const T* __restrict__ q, const T* __restrict__ kv, const int32_t* __restrict__ block_table, int table_stride,
        const int32_t* __restrict__ row_slot, const int32_t* __restrict__ kv_len, int heads, int kv_heads, int kd, int vd,
        int pages, int page_size, float scale, const float* __restrict__ head_scale, int chunk, int window,
        float* __restrict__ partial) {
    extern __shared__ __align__(16) unsigned char r1_smem[];
    constexpr int PER16 = 16 / (int)sizeof(T);               // numbers in 16 bytes
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t = blockIdx.x, splits = gridDim.y;
    const int all = kv_heads * vd, rowlen = kd + vd, rowpad = rowlen + PER16, group = heads / kv_heads;
    float* qs = (float*)r1_smem;                             // [heads][kd]
    float* sc = qs + (size_t)heads * kd;                     // [R1_KEYS][heads]: scores, then weights
    float* st = sc + R1_KEYS * heads;                        // [3][heads]: maximum, sum, this tile's correction
    T* tile = (T*)(qs + (((size_t)heads * (kd + R1_KEYS + 3) + 3) & ~(size_t)3));   // [kv_heads][R1_KEYS][rowpad], 16-byte aligned
    const int n = kv_len[t], pos = n - 1;                    // (row t holds one token: the last of its n)
    const bool live = n > 0;
    int first = 0, last = pos;
    if (live && chunk > 0) first = (pos / chunk) * chunk;
    if (live && window > 0) first = max(first, pos - window + 1);
    if (live) {
        const int per = (((pos - first + splits) / splits) + 31) & ~31;
        first += (int)blockIdx.y * per;
        last = min(pos, first + per - 1);
    }
    for (int i = tid; i < heads * kd; i += R1_THREADS) qs[i] = to_f32(q[(size_t)t * heads * kd + i]);
    for (int i = tid; i < heads; i += R1_THREADS) { st[i] = -INFINITY; st[heads + i] = 0.f; }
    const int runs = all >> 2;                               // threads a head group
    const int r = tid % runs, g0 = (tid / runs) * HPT;       // this thread's run of values and its first head
    const int e0 = 4 * r, c = e0 / vd;                       // the run's first number in the wide row, its kv head
    const bool owner = g0 + HPT <= heads;
    float acc[HPT][4];
#pragma unroll
    for (int h = 0; h < HPT; ++h)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[h][k] = 0.f;
    const int32_t* table = block_table + (size_t)row_slot[t] * table_stride;
    const int chunks16 = rowlen / PER16;                     // 16-byte pieces a row
    for (int j0 = first; live && j0 <= last; j0 += R1_KEYS) {
        __syncthreads();                                     // (the tile before is read; first pass: qs and st are written)
        for (int i = tid; i < kv_heads * R1_KEYS * chunks16; i += R1_THREADS) {
            const int piece = i % chunks16, j = (i / chunks16) % R1_KEYS, ck = i / (chunks16 * R1_KEYS);
            const int key = j0 + j;
            uint4 w = make_uint4(0u, 0u, 0u, 0u);            // keys past the part, or without a page: zeros
            if (key <= last) {
                const int page = table[key / page_size];
                if (page >= 0 && page < pages)
                    w = *(const uint4*)(kv + (((size_t)page * kv_heads + ck) * page_size + key % page_size) * rowlen + piece * PER16);
            }
            *(uint4*)(tile + ((size_t)ck * R1_KEYS + j) * rowpad + piece * PER16) = w;
        }
        __syncthreads();
        for (int pair = tid; pair < heads * R1_KEYS; pair += R1_THREADS) {      // scores: a warp a head, a lane a key
            const int g = pair / R1_KEYS, j = pair % R1_KEYS;
            const T* kr = tile + ((size_t)(g / group) * R1_KEYS + j) * rowpad;
            const float* qg = qs + (size_t)g * kd;
            float d4[4] = {0.f, 0.f, 0.f, 0.f};
            for (int x = 0; x < kd; x += 4) {
                float v[4];
                load_run4(kr + x, v);
#pragma unroll
                for (int k = 0; k < 4; ++k) d4[k] = fmaf(qg[x + k], v[k], d4[k]);
            }
            const float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
            sc[j * heads + g] = j0 + j <= last ? dot * scale * (head_scale ? head_scale[g] : 1.f) : -INFINITY;
        }
        __syncthreads();
        for (int g = warp; g < heads; g += R1_THREADS / 32) {                    // maximum and sum: a warp a head
            const float sv = sc[lane * heads + g];
            const float m_old = st[g], m_new = fmaxf(m_old, warp_max(sv));
            const float corr = m_new == -INFINITY ? 1.f : expf(m_old - m_new);
            const float pv = sv > -INFINITY ? expf(sv - m_new) : 0.f;
            const float sum = warp_sum(pv);
            sc[lane * heads + g] = pv;
            if (lane == 0) { st[g] = m_new; st[heads + g] = st[heads + g] * corr + sum; st[2 * heads + g] = corr; }
        }
        __syncthreads();
        if (owner) {
#pragma unroll
            for (int h = 0; h < HPT; ++h) {
                const float corr = st[2 * heads + g0 + h];
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[h][k] *= corr;
            }
            const T* vr = tile + (size_t)c * R1_KEYS * rowpad + kd + (e0 - c * vd);
#pragma unroll 4
            for (int j = 0; j < R1_KEYS; ++j) {
                float v[4];
                load_run4(vr + (size_t)j * rowpad, v);
                const float* pj = sc + j * heads + g0;
#pragma unroll
                for (int h = 0; h < HPT; ++h) {
                    const float w = pj[h];
#pragma unroll
                    for (int k = 0; k < 4; ++k) acc[h][k] = fmaf(w, v[k], acc[h][k]);
                }
            }
        }
    }
    __syncthreads();
    if (owner) {
#pragma unroll
        for (int h = 0; h < HPT; ++h) {
            float* part = partial + (((size_t)t * splits + blockIdx.y) * heads + g0 + h) * (all + 2);
            if (r == 0) { part[0] = st[g0 + h]; part[1] = st[heads + g0 + h]; }
            *(float2*)(part + 2 + e0) = make_float2(acc[h][0], acc[h][1]);          // (rows of all + 2 numbers: 8-byte aligned)
            *(float2*)(part + 4 + e0) = make_float2(acc[h][2], acc[h][3]);
        }
    }
}

// One block per (token, output head h): out[h, d] = sum over query heads g and parts s of
// talk[h, g] exp(m_gs - m_g) / l_g * part_gs[kv(h) value_dim + d], m_g and l_g the merged maximum and sum of head g.
// The factors of all (g, s) are made first (a thread a head, its parts in order), then the threads share the pairs
// (g, s) out in slices, a value channel each, and the slices are added in order: loads that do not wait for one another.
#define TM_THREADS 1024
template <typename T>
__global__ void __launch_bounds__(TM_THREADS) talking_merge_kernel(T* __restrict__ out, const float* __restrict__ partial, int splits, int heads,
                                     int kv_heads, int vd, const float* __restrict__ talk) {
    extern __shared__ float tk_smem[];
    const size_t t = blockIdx.x;
    const int h = blockIdx.y, tid = threadIdx.x;
    const int all = kv_heads * vd, c = h / (heads / kv_heads), pairs = heads * splits;
    float* w = tk_smem;                                      // [splits][heads]: sums, then factors
    float* mm = w + pairs;                                   // [splits][heads]: maxima, then exp(m_gs - m_g)
    float* red = mm + pairs;                                 // [slices][vd]
    const float* mine = partial + t * (size_t)pairs * (all + 2);
    for (int i = tid; i < pairs; i += TM_THREADS) { mm[i] = mine[(size_t)i * (all + 2)]; w[i] = mine[(size_t)i * (all + 2) + 1]; }
    __syncthreads();
    for (int g = tid; g < heads; g += TM_THREADS) {
        float m = -INFINITY, l = 0.f;
        for (int s = 0; s < splits; ++s) m = fmaxf(m, mm[s * heads + g]);
        for (int s = 0; s < splits; ++s) {
            const float ms = mm[s * heads + g], e = ms > -INFINITY ? expf(ms - m) : 0.f;
            l = fmaf(w[s * heads + g], e, l);
            mm[s * heads + g] = e;
        }
        const float f = (talk ? talk[h * heads + g] : (g == h ? 1.f : 0.f)) * (l > 0.f ? 1.f / l : 0.f);
        for (int s = 0; s < splits; ++s) w[s * heads + g] = mm[s * heads + g] * f;
    }
    __syncthreads();
    const int slices = vd >= TM_THREADS ? 1 : TM_THREADS / vd;
    const int slice = vd >= TM_THREADS ? 0 : tid / vd;
    if (slice < slices) {
        for (int d = vd >= TM_THREADS ? tid : tid - slice * vd; d < vd; d += TM_THREADS) {
            const float* col = mine + 2 + c * vd + d;
            float a = 0.f;
#pragma unroll 16
            for (int i = slice; i < pairs; i += slices) a = fmaf(col[(size_t)i * (all + 2)], w[i], a);
            red[slice * vd + d] = a;
        }
    }
    __syncthreads();
    for (int d = tid; d < vd; d += TM_THREADS) {
        float a = 0.f;
        for (int k = 0; k < slices; ++k) a += red[k * vd + d];
        out[(t * heads + h) * vd + d] = from_f32<T>(a);
    }
}

// One block per token: wide_in [tokens, heads, value_heads, vd] (value_heads = kv_heads: every kv head's values under every
// query head's weights; 1: one kv head in all) -> out[t, h, :] = sum_g talk[h, g] wide_in[t, g, kv(h), :].
template <typename T>
__global__ void talking_mix_kernel(T* __restrict__ out, const T* __restrict__ wide_in, int token0, int heads, int kv_heads,
                                   int vd, const float* __restrict__ talk) {
    extern __shared__ float tk_smem[];
    const size_t t = (size_t)token0 + blockIdx.x;
    const int n = heads * kv_heads * vd;
    const T* src = wide_in + t * n;
    float* mix = tk_smem + n;                                // the mixing matrix beside the token's rows
    if (sizeof(T) == 2 && (n & 7) == 0 && ((uintptr_t)wide_in & 15) == 0) {      // bfloat16 rows in pieces of 16 bytes
        for (int e = threadIdx.x; e < (n >> 3); e += blockDim.x) {
            const uint4 w = ((const uint4*)src)[e];
            const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                tk_smem[8 * e + 2 * i] = __uint_as_float(u[i] << 16);
                tk_smem[8 * e + 2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
            }
        }
    } else {
        for (int e = threadIdx.x; e < n; e += blockDim.x) tk_smem[e] = to_f32(src[e]);
    }
    if (talk) for (int e = threadIdx.x; e < heads * heads; e += blockDim.x) mix[e] = talk[e];
    __syncthreads();
    talking_mix_store<T>(out, tk_smem, talk ? mix : nullptr, t, heads, kv_heads, vd);
}

template <typename T>
static int launch_talking_merge(void* out, const float* partial, int splits, int tokens, int heads, int kv_heads, int vd,
                                const float* talk, cudaStream_t s) {
    const int slices = vd >= TM_THREADS ? 1 : TM_THREADS / vd;
    const size_t merge_bytes = ((size_t)2 * heads * splits + (size_t)slices * vd) * sizeof(float);
    if (merge_bytes > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(talking_merge_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)merge_bytes));
    talking_merge_kernel<T><<<dim3(tokens, heads), TM_THREADS, merge_bytes, s>>>((T*)out, partial, splits, heads, kv_heads, vd, talk);
    HB_LAUNCH_CHECK("talking_merge");
    return 0;
}

template <typename T>
static int launch_talking(void* out, const void* q, const void* kv, const int32_t* block_table, int table_stride,
                          const int32_t* row_slot, const int32_t* query_start, const int32_t* kv_len, int rows, int tokens,
                          int heads, int kv_heads, int kd, int vd, int pages, int page_size, float scale,
                          const float* head_scale, int chunk, int window, const float* talk, float* partial, int splits,
                          cudaStream_t s) {
    const int all = kv_heads * vd;
    const int warps = heads < TK_WARPS ? heads : TK_WARPS;
    const size_t wide_bytes = (size_t)heads * all * sizeof(float);
    const size_t smem = (splits > 1 ? 0 : wide_bytes) + (size_t)warps * kd * sizeof(float);
    if (wide_bytes + (size_t)warps * kd * sizeof(float) > 200 * 1024) HB_REFUSE("attention_talking: %d heads over %d kv heads of %d values need %zu bytes of shared memory", heads, kv_heads, vd, smem);
    const bool vec = vd % 4 == 0 && kd % 4 == 0 && ((uintptr_t)kv % (4 * sizeof(T))) == 0;   // runs of four never cross a kv head
    {   // rows of one token whose sizes the staged kernel takes
        const int per16 = 16 / (int)sizeof(T), runs = all / 4;
        const int ng = runs > 0 && runs <= R1_THREADS && R1_THREADS % runs == 0 ? R1_THREADS / runs : 0;
        const int hpt = !ng ? 0 : heads % ng == 0 ? heads / ng : heads < ng ? 1 : 0;    // (fewer heads than groups: some threads idle)
        const size_t bytes = (((size_t)heads * (kd + R1_KEYS + 3) + 3) & ~(size_t)3) * sizeof(float)
                             + (size_t)kv_heads * R1_KEYS * (kd + vd + per16) * sizeof(T);
        if (splits > 1 && tokens == rows && vec && (kd + vd) % per16 == 0 && ((uintptr_t)kv % 16) == 0 && bytes <= 200 * 1024
                && (hpt == 1 || hpt == 2 || hpt == 4 || hpt == 8 || hpt == 16)) {
#define HB_ROWS1(H) do { \
                auto kernel = talking_rows1_kernel<T, H>; \
                if (bytes > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes)); \
                kernel<<<dim3(tokens, splits), R1_THREADS, bytes, s>>>((const T*)q, (const T*)kv, block_table, table_stride, row_slot, \
                    kv_len, heads, kv_heads, kd, vd, pages, page_size, scale, head_scale, chunk, window, partial); \
            } while (0)
            if (hpt == 1) HB_ROWS1(1); else if (hpt == 2) HB_ROWS1(2); else if (hpt == 4) HB_ROWS1(4);
            else if (hpt == 8) HB_ROWS1(8); else HB_ROWS1(16);
#undef HB_ROWS1
            HB_LAUNCH_CHECK("talking_rows1");
            return launch_talking_merge<T>(out, partial, splits, tokens, heads, kv_heads, vd, talk, s);
        }
    }
#define HB_TALK(E) do { \
        auto kernel = splits > 1 ? (vec && E >= 4 ? attention_talking_kernel<T, E, true, (E >= 4)> : attention_talking_kernel<T, E, true, false>) \
                                 : (vec && E >= 4 ? attention_talking_kernel<T, E, false, (E >= 4)> : attention_talking_kernel<T, E, false, false>); \
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kernel<<<dim3(tokens, splits > 1 ? splits : 1), warps * 32, smem, s>>>((T*)out, (const T*)q, (const T*)kv, block_table, \
            table_stride, row_slot, query_start, kv_len, rows, heads, kv_heads, kd, vd, pages, page_size, scale, head_scale, \
            chunk, window, talk, partial); \
    } while (0)
    if (all <= 32) HB_TALK(1);
    else if (all <= 64) HB_TALK(2);
    else if (all <= 128) HB_TALK(4);
    else if (all <= 256) HB_TALK(8);
    else if (all <= 512) HB_TALK(16);
    else if (all <= 1024) HB_TALK(32);
    else HB_REFUSE("attention_talking: %d kv heads of %d values are above 1024 numbers a head", kv_heads, vd);
#undef HB_TALK
    HB_LAUNCH_CHECK("attention_talking");
    if (splits > 1) return launch_talking_merge<T>(out, partial, splits, tokens, heads, kv_heads, vd, talk, s);
    return 0;
}

extern "C" int hb_attention_talking(void* out, const void* q, const void* kv, int dtype, const int32_t* block_table,
                                    int table_stride, const int32_t* row_slot, const int32_t* query_start,
                                    const int32_t* kv_len, int rows, int tokens, int heads, int kv_heads, int key_dim,
                                    int value_dim, int pages, int page_size, float scale, const float* head_scale, int chunk,
                                    int window, const float* talk, float* partial, int splits, hb_stream stream) {
    if (tokens == 0 || rows == 0) return 0;
    if (splits > 1 && !partial) HB_REFUSE("attention_talking: %d parts need their scratch", splits);
    if (splits > 65535) HB_REFUSE("attention_talking: %d parts", splits);
    if (kv_heads < 1 || heads % kv_heads) HB_REFUSE("attention_talking: %d heads are no multiple of %d kv heads", heads, kv_heads);
    if (key_dim < 1 || value_dim < 1 || chunk < 0 || window < 0) HB_REFUSE("attention_talking: key size %d, value size %d, chunk %d, window %d", key_dim, value_dim, chunk, window);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_F32)
        return launch_talking<float>(out, q, kv, block_table, table_stride, row_slot, query_start, kv_len, rows, tokens, heads,
                                     kv_heads, key_dim, value_dim, pages, page_size, scale, head_scale, chunk, window, talk, partial, splits, s);
    if (dtype == HB_BF16)
        return launch_talking<bf16>(out, q, kv, block_table, table_stride, row_slot, query_start, kv_len, rows, tokens, heads,
                                    kv_heads, key_dim, value_dim, pages, page_size, scale, head_scale, chunk, window, talk, partial, splits, s);
    HB_REFUSE("attention_talking: dtype %d", dtype);
}

// out [tokens, heads, value_dim] for tokens token0 .. token0 + count - 1 from wide [tokens, heads, value_heads, value_dim]
// (value_heads: kv_heads, or 1 with one kv head).
extern "C" int hb_talking_mix(void* out, const void* wide, int dtype, int token0, int count, int heads, int kv_heads,
                              int value_dim, const float* talk, hb_stream stream) {
    if (count <= 0) return 0;
    if (kv_heads < 1 || heads % kv_heads || value_dim < 1) HB_REFUSE("talking_mix: %d heads, %d kv heads, value size %d", heads, kv_heads, value_dim);
    const size_t smem = ((size_t)heads * kv_heads * value_dim + (size_t)heads * heads) * sizeof(float);
    if (smem > 200 * 1024) HB_REFUSE("talking_mix: %zu bytes of shared memory a token", smem);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == HB_BF16) {
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(talking_mix_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        talking_mix_kernel<bf16><<<count, 256, smem, s>>>((bf16*)out, (const bf16*)wide, token0, heads, kv_heads, value_dim, talk);
    } else if (dtype == HB_F32) {
        if (smem > 48 * 1024) HB_CUDA(cudaFuncSetAttribute(talking_mix_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        talking_mix_kernel<float><<<count, 256, smem, s>>>((float*)out, (const float*)wide, token0, heads, kv_heads, value_dim, talk);
    } else HB_REFUSE("talking_mix: dtype %d", dtype);
    HB_LAUNCH_CHECK("talking_mix");
    return 0;
}
