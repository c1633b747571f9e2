// The C interface of the kernel library. Every function enqueues work on `stream` and returns at once:
// 0 on success, HB_ERR_REFUSED for sizes or types a kernel does not take (hb_last_error() says which),
// HB_ERR_CUDA when the launch itself failed. Pointers are device pointers unless a comment says otherwise.
// dtype codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HB_F32 0
#define HB_BF16 1
#define HB_ERR_REFUSED 1
#define HB_ERR_CUDA 2

typedef void* hb_stream;

const char* hb_last_error(void);
int hb_version(void);

// out[t, :] = float(table[ids[t], :]); ids outside [0, vocab) give a row of zeros.
int hb_embed(float* out, const void* table, int table_dtype, const int32_t* ids, int tokens, int hidden, int vocab,
             hb_stream stream);

// Row r reads row t = index ? index[r] : r of h (and of delta when given): v = h[t] + delta[t];
// out[r] = v * rsqrt(mean(v^2) + eps) * (weight + offset), rounded once. With delta and without index, h[t] = v is
// written back (h must then be float32). h_dtype may be bfloat16 only without delta (a plain norm).
int hb_add_rmsnorm(void* out, int out_dtype, void* h, int h_dtype, const void* delta, const void* weight,
                   int weight_dtype, float eps, float offset, const int32_t* index, int rows, int dim,
                   hb_stream stream);

// out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i], in 32-bit, rounded once.
int hb_silu_mul(void* out, const void* gate_up, int dtype, int tokens, int inter, hb_stream stream);

// Per token and head: RMSNorm over the head (if weights are given), rounding, rotation of the first rotary_dim
// dimensions in half-split pairs with cos|sin rows of `table` [max_positions, rotary_dim], rounding. q goes to q_out
// [tokens, heads, head_dim]; k and v go to kv [pages, 2, kv_heads, page_size, head_dim] at write_index = page *
// page_size + offset (a negative or out-of-range index skips the token). kv may be null (q only). `bias` (or null): one
// vector [(heads + 2 kv_heads) head_dim] of `dtype` that is added to q, k and v first.
int hb_qk_norm_rope_kv_write(void* q_out, const void* qkv, int dtype, const int32_t* positions, const float* table,
                             int rotary_dim, int max_positions, const void* q_weight, const void* k_weight,
                             int weight_dtype, float eps, float offset, void* kv, const int32_t* write_index,
                             int pages, int page_size, int tokens, int heads, int kv_heads, int head_dim,
                             const void* bias, hb_stream stream);

// Attention of the step's new rows over the paged cache, any sizes, on CUDA cores with 32-bit arithmetic.
// Row b owns query rows query_start[b] .. query_start[b+1], the last ones of its kv_len[b] tokens; a query at position
// p sees keys j <= p, with window > 0 only p - j < window. `sinks` (float [heads], or null): each head's softmax
// denominator also holds exp(sinks[h]), a weight without key or value that is not scaled; the bfloat16 kernels below that
// take `sinks` mean the same.
int hb_attention_generic(void* out, const void* q, const void* kv, int dtype, const int32_t* block_table,
                         int table_stride, const int32_t* row_slot, const int32_t* query_start,
                         const int32_t* kv_len, int rows, int tokens, int heads, int kv_heads, int head_dim,
                         int pages, int page_size, float scale, int window, const float* sinks, hb_stream stream);

// bfloat16 attention on tensor cores for rows that bring one token each (rows 0 .. rows - 1 of the batch). The keys of
// a row are cut into `splits` parts that run side by side; with more than one split, `scratch` must hold
// hb_attention_decode_scratch_floats(...) floats: the parts' partial results, merged by a second kernel.
// head_dim: a multiple of 16 up to 256.
size_t hb_attention_decode_scratch_floats(int rows, int heads, int head_dim, int splits);
int hb_attention_decode_bf16(void* out, float* scratch, const void* q, const void* kv, const int32_t* block_table,
                             int table_stride, const int32_t* row_slot, const int32_t* query_start,
                             const int32_t* kv_len, int rows, int heads, int kv_heads, int head_dim, int pages,
                             int page_size, float scale, int window, int splits, const float* sinks, hb_stream stream);

// The same rows with 2 to 16 splits whose CTAs form a thread-block cluster and merge through distributed shared memory
// inside the kernel: no scratch, no second kernel. hb_attention_decode_cluster_capacity: clusters of that many CTAs
// that the GPU runs at once for this head size (0: none).
int hb_attention_decode_cluster_capacity(int head_dim, int splits);
int hb_attention_decode_bf16_cluster(void* out, const void* q, const void* kv, const int32_t* block_table,
                                     int table_stride, const int32_t* row_slot, const int32_t* query_start,
                                     const int32_t* kv_len, int rows, int heads, int kv_heads, int head_dim, int pages,
                                     int page_size, float scale, int window, int splits, const float* sinks,
                                     hb_stream stream);

// The same rows with the keys of all of them shared out evenly over `ctas` CTAs (one wave that fills the GPU): each
// takes the same number of 64-key tiles, across rows and heads where its stretch crosses them, so rows of any lengths
// cost what their sum costs. At most 256 rows. `scratch`: hb_attention_decode_balanced_scratch_floats(...) floats.
size_t hb_attention_decode_balanced_scratch_floats(int rows, int heads, int kv_heads, int head_dim, int ctas);
int hb_attention_decode_bf16_balanced(void* out, float* scratch, const void* q, const void* kv,
                                      const int32_t* block_table, int table_stride, const int32_t* row_slot,
                                      const int32_t* query_start, const int32_t* kv_len, int rows, int heads,
                                      int kv_heads, int head_dim, int pages, int page_size, float scale, int window,
                                      int ctas, hb_stream stream);

// bfloat16 attention on tensor cores for rows row0 .. rows - 1, each bringing any number of tokens. q_tiles: at least
// the sum over these rows of ceil(tokens / 64).
int hb_attention_prefill_bf16(void* out, const void* q, const void* kv, const int32_t* block_table, int table_stride,
                              const int32_t* row_slot, const int32_t* query_start, const int32_t* kv_len, int row0,
                              int rows, int q_tiles, int heads, int kv_heads, int head_dim, int pages, int page_size,
                              float scale, int window, const float* sinks, hb_stream stream);

// The same rows on tcgen05 tensor cores (scores and output in tensor memory, operands by TMA): head_dim 128, page
// sizes that are multiples of 64. q_tiles: the sum over the rows of ceil(tokens / tile_q); tokens: all tokens of the
// step; tile_q: 256, or 128 for twice the CTAs at half the work each (steps with few query tiles).
// hb_attention_tcgen05_status synchronises the device and returns (and clears) the kernel's bounded-wait status word.
int hb_attention_prefill_tcgen05(void* out, const void* q, const void* kv, const int32_t* block_table, int table_stride,
                                 const int32_t* row_slot, const int32_t* query_start, const int32_t* kv_len, int row0,
                                 int rows, int q_tiles, int tokens, int heads, int kv_heads, int head_dim, int pages,
                                 int page_size, float scale, int window, int tile_q, const float* sinks, hb_stream stream);
// The same kernel with its other forms as parameters. planes: 2 for a cache [pages, 2, kv_heads, page, 128], 1 for one whose
// rows hold a token's key and value side by side [pages, kv_heads, page, 256]. value_heads: 1 (a query head weighs the
// values of its own kv head; out [tokens, heads, 128]) or kv_heads (those of every kv head; out [tokens, heads * kv_heads,
// 128], row h * kv_heads + c for query head h and kv head c). chunk > 0: a query at position i sees only keys
// j >= floor(i / chunk) * chunk. head_scale (float [heads] without zeros, or null): a factor per head on the scores.
int hb_attention_prefill_tcgen05_rows(void* out, const void* q, const void* kv, const int32_t* block_table, int table_stride,
                                      const int32_t* row_slot, const int32_t* query_start, const int32_t* kv_len, int row0,
                                      int rows, int q_tiles, int tokens, int heads, int kv_heads, int head_dim, int pages,
                                      int page_size, float scale, int window, int tile_q, const float* sinks, int planes,
                                      int value_heads, int chunk, const float* head_scale, hb_stream stream);
int hb_attention_tcgen05_status(unsigned int* status);

// out[m, n] = sum_k x[m, k] * w[n, k], all float32, sums in a fixed order that does not depend on m's neighbours.
int hb_gemm_f32(float* out, const float* x, const float* w, int m, int n, int k, hb_stream stream);

// `batch` float32 products at once, one per head: out[t, b, :] = x[t, b, :] · w[b]ᵀ with w [batch, n, k]; row t of
// product b starts at x + t * ldx + b * x_batch and at out + t * ldo + b * o_batch (elements).
int hb_gemm_f32_heads(float* out, const float* x, const float* w, int m, int n, int k, int batch, long ldx, long x_batch,
                      long ldo, long o_batch, hb_stream stream);

// Hyper-connections (csrc/hyper.cu). Row r reads token t = index ? index[r] : r. Old streams: xs [tokens, streams,
// dim] (32-bit), or, with src [tokens, dim], that row for every stream. With y [tokens, dim] (out's dtype):
// new_q = sum_s mix[s * streams + q] old_s + outc[q] y, else new = old. Without index the new streams are written to
// xs. out [rows, dim] = RMSNorm(sum_q inc[q] new_q) (inc null: ones) · (weight + offset). 1 to 16 streams.
int hb_hyper_mix_norm(void* out, int out_dtype, float* xs, const float* src, const void* y, const float* mix,
                      const float* outc, const float* inc, const void* weight, int weight_dtype, float eps, float offset,
                      const int32_t* index, int rows, int dim, int streams, hb_stream stream);

// Latent attention (csrc/latent.cu, csrc/latent_bf16.cu). The cache holds one row per token, [latent (rank) | rotated
// key part (rot)], in pages [pages, page_size, rank + rot]; queries are folded per head: qa [tokens, heads, rank + rot].
// hb_latent_prepare: `first` [tokens, ld] holds per head [dim unrotated | rot rotated] query entries from column 0 and,
// from column dkv_at (< 0: none), the down-projection's rank + rot outputs. Writes the rotated query parts into
// qa[:, :, rank:] (the first rot_dims entries turn, half-split pairs, angles from table [max_positions, rot_dims],
// cosines then sines) and, with dkv_at >= 0, [RMSNorm(latent) · norm_weight | rotated key part] into cache row
// write_index[t] (negative or out of range: skipped).
int hb_latent_prepare(void* qa, const void* first, int dtype, int ld, int tokens, int heads, int dim, int rot, int rank,
                      int dkv_at, const int32_t* positions, const float* table, int rot_dims, int max_positions,
                      const void* norm_weight, int weight_dtype, float eps, void* cache, const int32_t* write_index,
                      int pages, int page_size, hb_stream stream);
// out [tokens, heads, rank] = softmax_j(scale · qa · row_j) · latent_j over the keys a query sees (as hb_attention_generic).
int hb_latent_attention_generic(void* out, const void* qa, const void* cache, int dtype, const int32_t* block_table,
                                int table_stride, const int32_t* row_slot, const int32_t* query_start,
                                const int32_t* kv_len, int rows, int tokens, int heads, int rank, int rot, int pages,
                                int page_size, float scale, int window, hb_stream stream);

// The same on tensor cores in bfloat16 (csrc/latent_bf16.cu) for rows row0 .. row1 - 1 of the batch, which bring `tokens`
// tokens in all, the first of them token `first_token` of the step; rank and rot multiples of 16, rank up to 512.
// splits > 1: the keys of every row are cut into that many parts whose partial results go to scratch
// (hb_latent_attention_scratch_floats(first_token + tokens, ...) floats) and are merged by a second kernel.
size_t hb_latent_attention_scratch_floats(int tokens, int heads, int rank, int splits);
int hb_latent_attention_bf16(void* out, float* scratch, const void* qa, const void* cache, const int32_t* block_table,
                             int table_stride, const int32_t* row_slot, const int32_t* query_start, const int32_t* kv_len,
                             int row0, int row1, int first_token, int tokens, int heads, int rank, int rot, int pages,
                             int page_size, float scale, int window, int splits, hb_stream stream);

// Routed experts (csrc/experts.cu). z [tokens, ld]: 32-bit router logits in columns 0 .. experts - 1. chosen / weight
// [tokens, top]: the experts with the largest softmax scores (equal ones by ascending expert) and score · scale
// (renormalize: divided by the chosen scores' sum first); counts[e] += 1 per choice. hb_expert_rows: counts
// [2 experts + 1] -> counts[experts + e] = first row of expert e (and the end); place[token * top + k] = the pair's
// row, token_of[row] = its token. hb_expert_linear: out [rows, n] = act(x[token_of ? token_of[row] : row] · w[e]ᵀ) for
// the rows of expert e, w [experts, n, k]; act 0 none, 1 relu squared, 2 silu. hb_expert_combine: out [tokens, hidden] =
// sum_k weight[t, k] · y[place[t, k]] + (shared ? sigmoid(z[t, gate_at]) · shared[t] : 0) (z null: the shared rows are
// added as they are); with `x` [tokens, hidden] and `identity_from` (one int32 on the device) a pair whose row is
// *identity_from or later belongs to an identity expert and reads x[t] in place of y.
// The choice may run on other numbers than the weights: `correction` (float [experts] or null) is added to the softmax
// scores for the choice alone; with `groups` > 1 the experts form that many equal groups of neighbours, a group counts by
// its best choice score and only experts of the `keep` best groups can be chosen; `tiny` is added to the chosen scores'
// sum before `renormalize` divides by it.
int hb_route_top(int32_t* chosen, float* weight, int32_t* counts, const float* z, const float* bias, int ld, int tokens, int experts,
                 int top, float scale, int renormalize, const float* correction, int groups, int keep, float tiny, hb_stream stream);
int hb_expert_rows(int32_t* place, int32_t* token_of, int32_t* counts, const int32_t* chosen, int tokens, int top,
                   int experts, hb_stream stream);
// hb_route_top and hb_expert_rows as one call (one launch for up to 256 tokens and 1,024 experts). counts [2 experts + 3]
// need not be zeroed; afterwards counts[2 experts + 1 ..] = (0, tokens): the `starts` of one expert that takes every token.
int hb_route_rows(int32_t* chosen, float* weight, int32_t* counts, int32_t* place, int32_t* token_of, const float* z,
                  const float* bias, int ld, int tokens, int experts, int top, float scale, int renormalize,
                  const float* correction, int groups, int keep, float tiny, hb_stream stream);
int hb_expert_linear(void* out, const void* x, int dtype, const int32_t* token_of, const void* w, const int32_t* starts,
                     int rows, int experts, int n, int k, int act, hb_stream stream);
int hb_expert_combine(void* out, const void* y, int dtype, const int32_t* place, const float* weight, const void* shared,
                      const float* z, int ldz, int gate_at, int tokens, int top, int hidden, const void* x,
                      const int32_t* identity_from, hb_stream stream);
// hb_expert_linear in bfloat16 on tensor cores: k and n multiples of 8; tile_rows 8 (on CUDA cores, for a row or two an expert), 16, 64 or 128 rows a tile (0: chosen
// from the rows an expert gets on average).
int hb_expert_linear_bf16(void* out, const void* x, const int32_t* token_of, const void* w, const int32_t* starts, int rows,
                          int experts, int n, int k, int act, int tile_rows, hb_stream stream);
// The same for prompts on tcgen05 tensor cores (csrc/experts_tcgen05.cu: tiles of 128 rows x 256 columns, TMA, tensor
// memory). token_of given: x is first gathered into `gathered` [rows, k]. table: 3 * hb_expert_linear_tcgen05_tiles(rows,
// experts) int32 of scratch. hb_experts_tcgen05_status synchronises the device and returns (and clears) the kernel's
// bounded-wait status word.
int hb_expert_linear_tcgen05_tiles(int rows, int experts);
int hb_expert_linear_tcgen05(void* out, const void* x, const int32_t* token_of, void* gathered, const void* w,
                             const int32_t* starts, int32_t* table, int rows, int experts, int n, int k, int act,
                             hb_stream stream);
int hb_experts_tcgen05_status(unsigned int* status);
// x = act(x) in place (act as above, 3 the tanh form of gelu, 4 xielu with the two numbers `numbers`, 5 tanh);
// o [tokens, n] *= sigmoid(g[t * ld + i]).
int hb_activation(void* x, int dtype, long count, int act, const float* numbers, hb_stream stream);
int hb_sigmoid_gate(void* o, const void* g, int dtype, int tokens, int n, long ld, hb_stream stream);
// A norm without statistics, N(x) = tanh(alpha x) w + b (alpha one number on the device; alpha, w, b 32-bit), csrc/dyt.cu.
// hb_dyt_add_norm: x = (h ? h[row] : 0) + (y ? N_post(y[row]) : 0) (post_alpha null: y as it is); without `index` and
// with y the sum is stored in h; out[r] = N_pre(x) where out is given; index (int32 [rows]) gathers rows.
int hb_dyt_add_norm(float* h, const void* y, int y_dtype, const float* post_alpha, const float* post_w, const float* post_b,
                    void* out, int out_dtype, const float* pre_alpha, const float* pre_w, const float* pre_b,
                    const int32_t* index, int rows, int dim, hb_stream stream);
// hb_dyt_shift: x_t = h_t + N_post(y_t) -> into (which may be h itself only without y); n_t = N_pre(x_t);
// out_t = n_t + (n_(t-1) - n_t) mix, where a row's first token takes n_(t-1) from carried [slots, dim] (32-bit) and the
// row's last n is written there.
int hb_dyt_shift(void* out, int out_dtype, float* into, const float* h, const void* y, int y_dtype, const float* post_alpha,
                 const float* post_w, const float* post_b, const float* pre_alpha, const float* pre_w, const float* pre_b,
                 const float* mix, float* carried, const int32_t* query_start, const int32_t* row_slot, int rows, int tokens,
                 int dim, hb_stream stream);

// bfloat16 product for at most 16 rows of x, bound by reading w once. mode 0: out [m, n] (bfloat16, or float32 when
// out_f32) = x [m, k] · w [n, k]ᵀ. mode 1: w is [2 inter, k], gate rows first; out [m, inter] = silu(x · gateᵀ) ·
// (x · upᵀ). k a multiple of 8; pointers 16-byte aligned.
int hb_gemm_bf16_skinny(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode, int inter,
                        hb_stream stream);

// The same kernel with the norms around the product folded in. mode 3: h [m, n] (float32) += bfloat16(x · wᵀ),
// out [m, n] = bfloat16(h · (next_weight + next_offset)), ss_out [ceil(n / 16), 16] = sums of squares of the new h
// per 16 columns and token. ss_in (any mode; null: none): x is such an `out` and lacks its row scale
// rsqrt(sum of ss_in [parts_in, 16] over parts / dim_in + eps_in), which is applied to the product's sums.
int hb_gemm_bf16_skinny_linked(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode,
                               int inter, float* h, const void* next_weight, int next_weight_f32, float next_offset,
                               float* ss_out, const float* ss_in, int parts_in, float eps_in, int dim_in,
                               hb_stream stream);

// The attention's first product for up to 16 tokens with what follows it in one kernel: x [m, k] times
// w [(heads + 2 kv_heads) * head_dim, k], then per head the q/k RMSNorm (weights bfloat16 or, with weight_f32, float32;
// null: no norm), the rotation of the whole head by the token's position (table [max_positions, head_dim], cosines
// then sines) and the write of queries to q_out [m, heads, head_dim] and of keys and values into their cache pages.
// head_dim 32, 64 or 128. The head_dim / 16 CTAs of a head are a thread-block cluster.
int hb_qkv_rope_skinny(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions,
                       const float* table, int max_positions, const void* q_weight, const void* k_weight, int weight_f32,
                       float eps, float offset, void* kv, const int32_t* write_index, int pages, int page_size, int heads,
                       int kv_heads, int head_dim, hb_stream stream);
int hb_qkv_rope_skinny_linked(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions,
                              const float* table, int max_positions, const void* q_weight, const void* k_weight,
                              int weight_f32, float eps, float offset, void* kv, const int32_t* write_index, int pages,
                              int page_size, int heads, int kv_heads, int head_dim, const float* ss_in, int parts_in,
                              float eps_in, int dim_in, hb_stream stream);
// The same link for a norm without statistics, N(y) = tanh(alpha y) weight + bias (alpha one number on the device, weights
// and biases float32 [n]): h [m, n] (float32) += N_post(bfloat16(x · wᵀ)); out (bfloat16 [m, n], or null) = N_pre(h).
int hb_gemm_bf16_skinny_dyt(void* out, const void* x, const void* w, int m, int n, int k, float* h, const float* post_alpha,
                            const float* post_w, const float* post_b, const float* pre_alpha, const float* pre_w,
                            const float* pre_b, hb_stream stream);
// The same two for up to 32 rows (four 8-row tiles of x a warp; meant for 17 to 32 rows and weights of a few MB, where a
// product is its launch): ss_in and ss_out hold 32 tokens a part.
int hb_gemm_bf16_skinny32(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode, int inter,
                          float* h, const void* next_weight, int next_weight_f32, float next_offset, float* ss_out,
                          const float* ss_in, int parts_in, float eps_in, int dim_in, hb_stream stream);
int hb_qkv_rope_skinny32(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions,
                         const float* table, int max_positions, const void* q_weight, const void* k_weight, int weight_f32,
                         float eps, float offset, void* kv, const int32_t* write_index, int pages, int page_size, int heads,
                         int kv_heads, int head_dim, const float* ss_in, int parts_in, float eps_in, int dim_in,
                         hb_stream stream);

// Several products of the same few rows, one after the other, as phases of ONE persistent kernel (csrc/gemm_chain.cu):
// the weight stream keeps running across them. A phase is a product of hb_gemm_bf16_skinny_linked (modes 0, 1, 3, same
// meanings of the fields); a phase may read what an earlier phase wrote. sync: two words, zero before the first
// launch; scratch: `slots` x 512 floats; flags: `slots` words, zero before the first launch; none of them may be
// shared with a launch that runs at the same time. hb_gemm_chain_capacity: the most CTAs a launch can have.
typedef struct {
    const void* w; const void* x; void* out; float* h; const void* next_weight; float* ss_out; const float* ss_in;
    int n, k, mode, inter, out_f32, next_weight_f32, parts_in, dim_in;
    float next_offset, eps_in;
} hb_chain_phase;
int hb_gemm_chain_capacity(void);
int hb_gemm_chain(const hb_chain_phase* phases, int n_phases, int m, unsigned int* sync, float* scratch,
                  unsigned int* flags, int slots, int cooperative, hb_stream stream);
int hb_gemm_chain_status(unsigned int* status);

// The same products in one launch whose CTAs each take one tile of one product, in the products' order (tickets drawn
// at the start; csrc/gemm_tickets.cu): a product's CTAs start while the one before ends, ask for their weights and
// wait for its last tile. Up to 4 products; state: 6 words, zero before the first launch.
int hb_gemm_tickets(const hb_chain_phase* phases, int n_phases, int m, unsigned int* state, hb_stream stream);
int hb_gemm_tickets_status(unsigned int* status);

// bfloat16 product on tcgen05 tensor cores with TMA loads and the accumulator in tensor memory (128 x 256 tiles).
// Same arguments and modes as hb_gemm_bf16_skinny, any m. hb_gemm_tcgen05_status synchronises the device and
// returns (and clears) a status word that is non-zero if a bounded wait inside the kernel ever gave up.
int hb_gemm_bf16_tcgen05(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode, int inter,
                         hb_stream stream);
int hb_gemm_tcgen05_status(unsigned int* status);

// The same product by pairs of CTAs on neighbouring SMs (tcgen05 cta_group::2: 256 x 256 tiles, each CTA loading half
// of both operands); same arguments and modes, its own status word.
int hb_gemm_bf16_tcgen05_pair(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode,
                              int inter, hb_stream stream);
int hb_gemm_tcgen05_pair_status(unsigned int* status);
int hb_gemm_tcgen05_pair_width(int bn);             // tests: fix the tile width (0: chosen per launch)

// bfloat16 products of 1 to 64 rows with the following work in their epilogue (csrc/gemm_mid.cu): weight tiles of
// 256 rows on tcgen05, a tile's k range split over a thread-block cluster of `split` CTAs (0: chosen; 1 to 8) that
// sum their partial results through distributed shared memory. mode 0 plain, 1 SwiGLU (w [2 inter, k], gate rows
// first; out [m, inter]), 3 residual sum and next norm (h [m, n] float32 += product; out = bfloat16(h (next_weight +
// next_offset)); ss_out [ceil(n / 256), 64] partial sums of squares of the new h). ss_in [parts_in, stride_in] (null:
// none): x lacks its norm's row scale rsqrt(sum over parts / dim_in + eps_in). hb_qkv_rope_mid: the attention's first
// product with q/k norm, rotation and cache write (arguments as hb_qkv_rope_skinny_linked).
int hb_gemm_bf16_mid(void* out, int out_f32, const void* x, const void* w, int m, int n, int k, int mode, int inter,
                     float* h, const void* next_weight, int next_weight_f32, float next_offset, float* ss_out,
                     const float* ss_in, int parts_in, int stride_in, float eps_in, int dim_in, int split,
                     hb_stream stream);
int hb_qkv_rope_mid(void* q_out, const void* x, const void* w, int m, int k, const int32_t* positions, const float* table,
                    int max_positions, const void* q_weight, const void* k_weight, int weight_f32, float eps, float offset,
                    void* kv, const int32_t* write_index, int pages, int page_size, int heads, int kv_heads, int head_dim,
                    const float* ss_in, int parts_in, int stride_in, float eps_in, int dim_in, int split, hb_stream stream);
int hb_gemm_mid_status(unsigned int* status);

// The waits inside the tcgen05 kernels are bounded; one that gives up records (place << 28) | (block + 1) in its
// kernel file's status word (the *_status functions above read those, synchronising) and in one word of page-locked
// host memory that hb_status_word hands out: the host reads it without a copy or a synchronisation, after a step's
// completion event, and may write 0 to it. hb_status_selftest enqueues a wait of `polls` polls on a barrier nobody
// arrives at (place 15): it runs out within microseconds and lets tests see what the host does then.
int hb_status_word(unsigned int** host);
int hb_status_word_device(unsigned int** device);   // the same word as the device addresses it (for a part's own kernel files)
int hb_status_selftest(int polls, hb_stream stream);

// The token each request sampled last, kept on the device by slot. feed: for every row r with from_last[r] != 0,
// token_ids[query_start[r]] = last_tokens[row_slot[r]]. store: last_tokens[slots[i]] = tokens[i] for i < n.
int hb_feed_tokens(int32_t* token_ids, const int32_t* last_tokens, const int32_t* row_slot, const int32_t* query_start,
                   const int32_t* from_last, int rows, hb_stream stream);
int hb_store_tokens(int32_t* last_tokens, const int32_t* slots, const int32_t* tokens, int n, hb_stream stream);

// Block-table rows that changed on the host, uploaded packed: table[slots[i], :] = rows[i, :] for i < n.
int hb_scatter_rows(int32_t* table, const int32_t* slots, const int32_t* rows, int n, int width, int table_rows,
                    hb_stream stream);

// One token per logits row: arg max where temperature is 0, else a draw from softmax(logits / temperature) after the
// filters (when `filtered`), by inverse CDF in vocabulary order with the uniform of (seed, position).
int hb_sample(int32_t* tokens, const float* logits, const float* temperature, const int32_t* top_k,
              const float* top_p, const float* min_p, const int32_t* seed_lo, const int32_t* seed_hi,
              const int32_t* position, int filtered, int rows, int vocab, hb_stream stream);

// Log-probabilities of the raw logits per row: chosen[r] of tokens[r], and the k most likely tokens ranked (equal
// logits by ascending id) as top_ids / top [rows, k]; places beyond the row's finite entries hold id -1 and -inf.
int hb_logprobs(float* chosen, int32_t* top_ids, float* top, const float* logits, const int32_t* tokens, int rows,
                int vocab, int k, hb_stream stream);

// Embedding rows times `scale`, plus a row of `pair` [buckets + 1, hidden] chosen by (previous id, id): row
// (previous * mul_prev + id * mul_cur) mod buckets, or row `buckets` at position 0. `prev` [slots] carries each slot's
// last id from step to step (read for a row's first token, then set to the row's last id). pair null: none is added.
int hb_embed_pair(float* out, const void* table, int table_dtype, float scale, const void* pair, const int32_t* ids,
                  const int32_t* positions, const int32_t* query_start, const int32_t* row_slot, int32_t* prev, int rows,
                  int tokens, int hidden, int vocab, long mul_prev, long mul_cur, int buckets, hb_stream stream);
// h [tokens, hidden] (32-bit) += s0 x0 + s1 x1 + s2 x2 + s3 x3 + bias; terms of `dtype`, any of them null.
int hb_sum_into(float* h, const void* x0, const void* x1, const void* x2, const void* x3, float s0, float s1, float s2,
                float s3, const void* bias, int dtype, int tokens, int hidden, hb_stream stream);
// hb_sum_into, and out [tokens, hidden] (`dtype`) = RMSNorm of the summed rows with `weight` (+ offset): the sum that ends one
// block and the norm that starts the next in one kernel.
int hb_sum_norm(float* h, const void* x0, const void* x1, const void* x2, const void* x3, float s0, float s1, float s2,
                float s3, const void* bias, int dtype, void* out, const void* weight, int weight_dtype, float eps,
                float offset, int tokens, int hidden, hb_stream stream);
// out [tokens, inter] = g sigmoid(alpha g) (u + 1), g = min(gate + b, limit), u = clamp(up + b, -limit, limit), from
// gate_up [tokens, 2 inter] (gate first) and bias [2 inter] (or null).
int hb_glu_clamped(void* out, const void* gate_up, const void* bias, int dtype, float limit, float alpha, int tokens,
                   int inter, hb_stream stream);

// ---- mixers with a matrix state per head (csrc/recurrent.cu). Rows as for attention: row b brings tokens
// query_start[b] .. query_start[b + 1] and lives in slot row_slot[b].
// The scan. qk [tokens, 2, kv_heads, dim] (queries, then keys), v [tokens, heads, vdim], state [slots, heads, vdim, dim]
// (S column by column), all 32-bit; head h reads key head h / (heads / kv_heads). Per token: S <- g S with g = decay[t, h, :] (per key channel)
// or head_decay[h] or token_decay[t, h] (give exactly one of the three; no beta with the last); u = beta[t, h] (v - S^T k) (beta null: u = v); S <- S + k u^T;
// out[t, h, :] = S^T q. The state is read at the start of a row and written back at its end. `most`: no row brings more
// tokens than this (0: unknown); it bounds the stage of tokens a block keeps in shared memory.
int hb_recurrent_scan(float* out, const float* qk, const float* v, const float* decay, const float* head_decay,
                      const float* token_decay, const float* beta, const float* rate, float* state, const int32_t* query_start,
                      const int32_t* row_slot, int rows, int heads, int kv_heads, int dim, int vdim, int most, hb_stream stream);
// The generalized delta rule's inputs from its first product, rows [r | k | v | g | a] of `dtype` (each heads dim wide,
// `ld` apart) and the low-rank decay projection's output `pre` [tokens, heads dim] in 32-bit: qk = (r, k), v,
// decay = exp(-decay_scale sigmoid(pre + decay_bias)), rate = sigmoid(a + rate_bias) / (sum_head k^2 + unit_eps); with
// `rate` hb_recurrent_scan runs S <- diag(decay) S - (rate o k)(k^T S) + k v^T, both terms on the old S.
int hb_gdelta_prepare(float* qk, float* v, float* decay, float* rate, const void* first, int dtype, long ld,
                      const float* pre, const float* decay_bias, const float* rate_bias, int tokens, int heads, int dim,
                      float decay_scale, float unit_eps, hb_stream stream);
// A delta-rule mixer's first product, rows [q | k | v | b] of `dtype`, `ld` apart, and the outputs of its two low-rank
// projections, low2 [tokens, heads dim + heads vdim] in 32-bit, become the scan's inputs: q, k, v through a causal
// convolution over time (conv [channels, taps], carried inputs conv_state [slots, taps - 1, channels]) and silu; q, k
// unit vectors per head (eps unit_eps), q times q_scale; beta = sigmoid(b); decay = exp(-exp(rate_log[h])
// softplus(low2[:, :heads dim] + dt_bias)) [tokens, heads, dim]; gate = sigmoid(low2[:, heads dim:]) [tokens, heads vdim].
int hb_delta_prepare(float* qk, float* v, float* beta, float* decay, float* gate, const void* first, int dtype, int ld,
                     const void* conv, int taps, const void* conv_state, const float* low2, const float* dt_bias,
                     const float* rate_log, const int32_t* query_start, const int32_t* row_slot, int rows, int tokens,
                     int heads, int kv_heads, int dim, int vdim, float q_scale, float unit_eps, hb_stream stream);
// conv_state <- the last taps - 1 inputs of each row (what was carried, then the step's tokens). After hb_delta_prepare.
int hb_conv_carry(void* conv_state, const void* first, int dtype, int ld, int channels, int taps,
                  const int32_t* query_start, const int32_t* row_slot, int rows, hb_stream stream);
// A retention mixer's first product, rows [q (heads dim) | k (heads dim) | v (heads vdim) | ...]: q and k turned by the
// position (as hb_qk_norm_rope_kv_write turns them), k times k_scale, all to 32-bit.
int hb_retention_prepare(float* qk, float* v, const void* first, int dtype, int ld, const int32_t* positions,
                         const float* table, int rot_dims, int max_positions, int tokens, int heads, int dim, int vdim,
                         float k_scale, hb_stream stream);
// out [tokens, heads, vdim] (`dtype`) = o / sqrt(mean(o^2) + eps) * weight (float [vdim], with `weight_heads` [heads
// vdim], or null) * gate, the gate a 32-bit multiplier gate_mul [tokens, heads vdim], or silu (`gate_sigmoid`: sigmoid)
// of gate_pre (rows `ld` apart, `dtype`), or none.
int hb_head_norm_gate(void* out, const float* o, int dtype, const float* weight, const float* gate_mul,
                      const void* gate_pre, long ld, float eps, int tokens, int heads, int vdim, int weight_heads,
                      int gate_sigmoid, hb_stream stream);

// ---- the matrix memory with exponential gates (csrc/mlstm.cu): the kernels around hb_recurrent_scan with token_decay.
// pre [tokens, ld] 32-bit: the input gate's pre-activations of the heads, then the forget gate's; bias [2 heads] likewise.
// out [3][tokens, heads]: keep = exp(f + m' - m), take = exp(i - m), exp(-m), with i = cap tanh(. / cap),
// f = logsigmoid(cap tanh(. / cap)), m = max(f + m', i); m_state [slots, heads] carries m from step to step.
int hb_mlstm_gates(float* out, const float* pre, int ld, const void* bias, int bias_dtype, float cap, float* m_state,
                   const int32_t* query_start, const int32_t* row_slot, int rows, int tokens, int heads, hb_stream stream);
// first rows [q (heads dim) | k (heads dim) | v (heads vdim) | ...] -> qk [tokens, 2, heads, dim] = (q q_scale, k take[t, h]),
// v1 [tokens, heads, vdim + 1] = [v | 1].
int hb_mlstm_prepare(float* qk, float* v1, const float* take, const void* first, int dtype, int ld, int tokens, int heads,
                     int dim, int vdim, float q_scale, hb_stream stream);
// o1 [tokens, heads, vdim + 1] = the scan's rows: y = o1[:vdim] / (max(|o1[vdim]|, floor[t, h]) + tiny), each head's y
// divided by its root mean square (eps), times weight [heads vdim], times sigmoid(gate_pre) (rows `ld` apart).
int hb_mlstm_read_out(void* out, const float* o1, const float* floor_, int dtype, const void* weight, int weight_dtype,
                      const void* gate_pre, long ld, float eps, float tiny, int tokens, int heads, int vdim, hb_stream stream);

// ---- a norm on a sublayer's output, with the average over the layers' results (csrc/elementwise.cu)
// dst = src + N(y + bias), N(z) = z rsqrt(mean(z^2) + eps) (weight + offset); y null: dst = src. With hist (n_hist tensors
// [rows, dim], hist_stride elements apart, dst the last of them): avg = sum_j coef[j] hist[j]. cast (or null) gets what goes
// on (avg with hist, else dst) as `cast_dtype`.
int hb_out_norm_add(float* dst, const float* src, const void* y, int y_dtype, const void* bias, int bias_dtype,
                    const void* weight, int weight_dtype, float eps, float offset, const float* hist, long hist_stride,
                    int n_hist, const float* coef, float* avg, void* cast, int cast_dtype, int rows, int dim, hb_stream stream);

// ---- attention whose heads share their weights after the softmax, keys and values of unequal sizes (csrc/attention_talking.cu)
// cache [pages, kv_heads, page_size, key_dim + value_dim]. qkv rows [q | k | v] -> bias, RMSNorm of q and k per head with
// q_weight / k_weight [key_dim] (null: none), the first rot_dims channels turned (neighbouring pairs if `interleaved`, else
// half-split; table [table_rows, rot_dims] cosines then sines), values blended with `first` [tokens, kv_heads, value_dim] by
// blend[0]; `keep` receives the unblended values in 32-bit.
int hb_qkv_talking_prepare(void* q_out, void* kv, float* keep, const void* qkv, int dtype, const void* bias, int bias_dtype,
                           const void* q_weight, const void* k_weight, int weight_dtype, float eps, const int32_t* positions,
                           const float* table, int rot_dims, int table_rows, int interleaved, const float* first,
                           const float* blend, const int32_t* write_index, int pages, int page_size, int tokens, int heads,
                           int kv_heads, int key_dim, int value_dim, hb_stream stream);
// out [tokens, heads, value_dim]: softmax of q . k scale head_scale[h] over the keys a query sees (j <= i; chunk C > 0: of its
// own block of C positions; window W > 0: the last W), the heads' weights mixed by talk [heads, heads] (null: not mixed).
int hb_attention_talking(void* out, const void* q, const void* kv, int dtype, const int32_t* block_table, int table_stride,
                         const int32_t* row_slot, const int32_t* query_start, const int32_t* kv_len, int rows, int tokens,
                         int heads, int kv_heads, int key_dim, int value_dim, int pages, int page_size, float scale,
                         const float* head_scale, int chunk, int window, const float* talk, float* partial, int splits,
                         hb_stream stream);
// (splits > 1: every token's keys in that many parts, a block each, merged by a second kernel; partial: float
// [tokens, splits, heads, kv_heads * value_dim + 2] of scratch.)
// The mixing alone: out[t, h, :] = sum_g talk[h, g] wide[t, g, kv(h), :] for tokens token0 .. token0 + count - 1, wide
// [tokens, heads, kv_heads, value_dim] (what hb_attention_prefill_tcgen05_rows leaves with value_heads = kv_heads).
int hb_talking_mix(void* out, const void* wide, int dtype, int token0, int count, int heads, int kv_heads, int value_dim,
                   const float* talk, hb_stream stream);

#ifdef __cplusplus
}
#endif
