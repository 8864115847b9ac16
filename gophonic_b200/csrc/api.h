// The C interface of the kernel library: parameter blocks and entry points.
//
// Every entry point has C linkage, takes raw device pointers and a cudaStream_t, launches on that
// stream and returns 0, or a negative status with the reason in gb_last_error().  Sizes a kernel
// cannot take are refused before anything is launched.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifndef GB_API
#define GB_API extern "C" __attribute__((visibility("default")))
#endif

// Attention over the paged cache: rows of a step, packed sequence by sequence.
struct AttnParams {
    const void* q;
    int64_t q_row_stride;
    void* out;
    int64_t out_row_stride;
    const void* k_plane;
    const void* v_plane;
    const int* block_table;
    int bt_stride;
    const int* seq_slot;
    const int* seq_q_start;
    const int* seq_q_len;
    const int* seq_kv_len;
    int nseq, heads, kv_heads, d;
    int max_q_len;
    float scale;
    int window;
    int num_splits;
    float* scratch;  // [nseq][heads][num_splits][d + 2] when num_splits > 1
    int pages;       // pages of each cache plane, and slots (rows) of the block table: the bounds the
    int max_slots;   // checked build holds every page and slot index against
};

// The same with the options that came later.  AttnParams keeps its layout for callers that fill it
// themselves; the entry points ending in _x take this one (the others behave as if the options were 0).
struct AttnParamsX : AttnParams {
    int dv;          // size of a value head; 0: the same as d.  Only the CUDA-core kernel takes another size.
    int keep_first;  // with a window: keys at positions below this stay visible however far back they lie
    int sink;        // 1: the softmax denominator carries one more term (a key without a value): exp(sinks[head]), or one unit
    const float* sinks;  // [heads] the sink's score per head, in the units of the scaled scores but not scaled itself; null: 0
    int chunk;       // > 0: position i sees j <= i only inside its own block of `chunk` positions, counted from position 0 of the sequence
    int v_share;     // > 1: this many consecutive key heads read one value head (the value plane holds kv_heads / v_share heads)
    int64_t v_row_stride;  // elements between the values of two tokens of a page; 0: dv.  A value plane that is a view of the key
                           // plane (the values are the first dv channels of the keys) has the keys' stride d.
};

// Per-head q/k RMSNorm, rotary embedding and cache write on the rows of a fused q|k|v buffer.
struct QkRopeParams {
    void* qkv;
    int64_t row_stride;
    const float* q_w;
    const float* k_w;
    float eps;
    const float* cos_t;  // [capacity, rot/2] or null when rot == 0
    const float* sin_t;
    int rot;             // rotary width (even, <= d); 0: no rotation
    int table_positions;
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* block_table;
    int bt_stride;
    void* k_plane;
    void* v_plane;
    int write_kv;
    int rows, heads, kv_heads, d;
    int pages;      // pages of each cache plane, and slots (rows) of the block table: the bounds the
    int max_slots;  // checked build holds every page and slot index against
};

// The same with what only the general kernel takes (null / 0: absent); QkRopeParams keeps its layout.
struct QkRopeParamsX : QkRopeParams {
    const float* q_b;  // biases added to the heads before norm and rotation: [heads * d], [kv_heads * d], [kv_heads * dv]
    const float* k_b;
    const float* v_b;
    int pairs;         // 1: channels 2j and 2j + 1 turn together by angle j; 0: channels j and j + rot / 2
    int dv;            // size of a value head; 0: the same as d
    int span;          // 1: q is normed over all its heads together (q_w: [heads * d]) and k likewise (k_w: [kv_heads * d]); 0: per head
    int v_share;       // > 1: the row holds kv_heads / v_share value heads (that many key heads read one value head); 0, 1: kv_heads
};

// A matrix state per (sequence, head), updated token by token: S <- diag(a) S + b k v^T, o = S^T q.
struct LinearStateParams {
    const void* qkv;        // rows of the fused projection (activation dtype): q, k and v heads at the offsets below
    int64_t row_stride;
    int q_off, k_off, v_off;
    float q_scale;          // q is multiplied by this as it is read
    const float* decay;     // per key channel: [rows, decay_stride] holding heads x d factors (scalar_decay 0)
    int64_t decay_stride;
    const float* gates;     // scalar_decay 1: pre-activations of the input gates [heads] then the forget gates [heads] of every row
    int64_t gates_stride;
    const float* gate_bias; // [2 heads] or null
    float gate_cap;         // gates are capped as cap * tanh(x / cap)
    float* coef;            // scalar_decay 1: [rows, heads, 4] scratch (keep, take, running maximum, divisor)
    float* state;           // [slots, ...]: per head d x dv of S, then (scalar_decay 1) d of the normaliser and the maximum
    int64_t slot_stride, head_stride;
    float* out;             // [rows, out_stride]: heads x dv sums S^T q (not yet divided)
    int64_t out_stride;
    const int* seq_slot;
    const int* seq_q_start;
    const int* seq_q_len;
    int nseq, heads, d, dv;
    int scalar_decay;
    int max_slots;
    int max_q_len;          // most rows a sequence brings; 1 selects the kernel for single tokens
};

// y = norm(x / divisor) * weight * gate(g) per (row, head); one warp a head.
struct HeadGateParams {
    const void* x;          // [rows, x_stride]: heads x size
    int64_t x_stride;
    const void* gate;       // [rows, gate_stride]: heads x size pre-activations of the gate (activation dtype)
    int64_t gate_stride;
    void* y;                // [rows, y_stride] (activation dtype)
    int64_t y_stride;
    const float* divisor;   // [rows, heads, divisor_stride] (its first element is used) or null
    int divisor_stride;
    const float* weight;    // [size] or [heads x size] or null
    int weight_per_head;
    int normed;             // 1: x over its root mean square (eps under the root) first
    float eps;
    int gate_kind;          // 0: sigmoid(g); 1: g * sigmoid(g)
    int rows, heads, size;
};

GB_API const char* gb_last_error();

// row-wise kernels
GB_API int gb_add_rmsnorm(float* h, const float* delta, const float* w, float eps, int n, void* out, int out_dtype, const int* row_index,
                          int out_rows, cudaStream_t stream);
GB_API int gb_swiglu(const void* gu, void* out, int dtype, int rows, int inter, int interleave8, cudaStream_t stream);
GB_API int gb_qk_norm_rope_kv_write(const QkRopeParams* p, int dtype, cudaStream_t stream);
GB_API int gb_qk_norm_rope_kv_write_x(const QkRopeParamsX* p, int dtype, cudaStream_t stream);
GB_API int gb_add_bias(float* out, const float* bias, int rows, int n, cudaStream_t stream);
GB_API int gb_concat_cast(const float* h, const float* delta, const float* side, void* out, int out_dtype, int rows, int n, cudaStream_t stream);

// matrix products: C[M, N] = A[M, K] W[N, K]^T
GB_API int gb_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M, int N, int K, int64_t lda,
                        int64_t ldw, int64_t ldc, cudaStream_t stream);
GB_API int gb_gemm_skinny(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy, cudaStream_t stream);
GB_API int gb_gemm_skinny_bias(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy,
                               const float* bias, cudaStream_t stream);
GB_API int gb_gemm_skinny_swiglu(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy,
                                 cudaStream_t stream);
GB_API int gb_gemm_tc5(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc, cudaStream_t stream);
GB_API int gb_gemm_tc5_swiglu(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                              cudaStream_t stream);
GB_API int gb_gemm_tc5_pair(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                            cudaStream_t stream);
GB_API int gb_gemm_tc5_pair_swiglu(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc,
                                   cudaStream_t stream);
GB_API int gb_gemm_tc5_ldw(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc,
                           int pair, cudaStream_t stream);
// Products of groups of rows (sorted by group, bounds in `offsets` on the device) with their own weight blocks, in
// one launch: block e of W is rows e * w_rows .. (by_cols 0; gated: N gate rows then N up rows, and the output is
// silu(f g) * (f u) with f = row_weight[row]) or columns e * K .. (by_cols 1).  With row_map, row r lands in row row_map[r] of C.
GB_API int gb_gemm_tc5_grouped(const void* A, const void* W, void* C, int c_dtype, const int* offsets, int groups, int P, int N, int K,
                               int64_t lda, int64_t ldw, int64_t ldc, int w_rows, int by_cols, int gated, const float* row_weight,
                               const int* row_map, cudaStream_t stream);
GB_API int gb_gemm_tc5_grouped_act(const void* A, const void* W, void* C, int c_dtype, const int* offsets, int groups, int P, int N, int K,
                                   int64_t lda, int64_t ldw, int64_t ldc, int w_rows, int by_cols, int gated, const float* row_weight,
                                   const int* row_map, float act_limit, float act_slope, cudaStream_t stream);
GB_API int gb_gemm_tc5_pair_bias(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, int64_t lda, int64_t ldc, int add,
                                 const float* bias, cudaStream_t stream);
GB_API int gb_gemm_tc5_pair_add(const void* A, const void* W, void* C, int M, int N, int K, int64_t lda, int64_t ldc, cudaStream_t stream);
// most rows the products with the residual's row-wise work folded in take
constexpr int GB_FOLD_MAX_ROWS = 64;
GB_API int gb_gemm_tc5_decode_splits(int M, int N, int K, int sms);
GB_API int gb_gemm_tc5_decode(const void* X, const void* W, void* Y, int c_dtype, int M, int N, int K, int64_t ldx, int64_t ldy, int epi,
                              int splits, cudaStream_t stream);

// attention
GB_API int gb_attention_simt(const AttnParams* p, int dtype, cudaStream_t stream);
GB_API int gb_attention_decode_mma(const AttnParams* p, cudaStream_t stream);
GB_API int gb_attention_prefill_mma(const AttnParams* p, cudaStream_t stream);
GB_API int gb_attention_decode_rope_accepts(int dtype, int d, int rot, int max_q_len);
GB_API int gb_attention_decode_mma_rope(const AttnParams* p, const QkRopeParams* r, cudaStream_t stream);
GB_API int gb_attention_prefill_tc5(const AttnParams* p, int rows, int pages, cudaStream_t stream);
GB_API int gb_attention_simt_x(const AttnParamsX* p, int dtype, cudaStream_t stream);
GB_API int gb_attention_decode_mma_x(const AttnParamsX* p, cudaStream_t stream);
GB_API int gb_attention_prefill_mma_x(const AttnParamsX* p, cudaStream_t stream);
GB_API int gb_attention_prefill_tc5_x(const AttnParamsX* p, int rows, int pages, cudaStream_t stream);
GB_API int gb_attention_algo_x(const AttnParamsX* p, int dtype);
GB_API int gb_attention_latent_accepts(const AttnParamsX* p, int dtype);
GB_API int gb_attention_latent_mma(const AttnParamsX* p, cudaStream_t stream);

// an AttnParams as the kernels take it: the later options off
static inline AttnParamsX gb_attn_widen(const AttnParams& a) {
    AttnParamsX x;
    static_cast<AttnParams&>(x) = a;
    x.dv = x.keep_first = x.sink = 0;
    x.sinks = nullptr;
    x.chunk = x.v_share = 0;
    x.v_row_stride = 0;
    return x;
}

// matrix-state mixers
GB_API int gb_gla_decay(float* z, const float* bias, int rows, int width, float tau, cudaStream_t stream);
GB_API int gb_state_scan(const LinearStateParams* p, int dtype, cudaStream_t stream);
GB_API int gb_head_norm_gate(const HeadGateParams* p, int x_dtype, int dtype, cudaStream_t stream);

// Hyper-connections: S streams of the residual, mixed by a sublayer's output and read for the next norm.
struct HyperParams {
    float* streams;          // stream s, row r: streams + s * stream_stride + r * width
    int64_t stream_stride;
    int n_streams, rows, width;
    const float* y;          // [rows, width] the sublayer's output, or null: the streams are only read
    const float* mix;        // [S, S] indexed [from, to], or null: the identity
    const float* out_coef;   // [S] or null: ones
    float mult;              // on the sublayer's output
    const float* in_coef;    // [S] or null: ones (the plain sum of the streams)
    const float* norm_w;     // [width]: the weight the normed sum is multiplied by
    float eps;
    void* x_out;             // [rows, width] in the activation dtype, or null: nothing is normed
    const int* row_index;    // rows to read (x_out row i from streams row row_index[i]), or null
};
GB_API int gb_hyper_mix_norm(const HyperParams* p, int out_dtype, cudaStream_t stream);
GB_API int gb_embed_streams(const void* table, int table_dtype, const int* ids, int rows, int hidden, int vocab, float* streams,
                            int64_t stream_stride, int n_streams, float scale, cudaStream_t stream);

// The generalized delta rule: S <- diag(w) S - (a u)(u^T S) + k v^T, o = S^T r per (sequence, head).
struct DeltaStateParams {
    const void* rkv;        // rows of the fused projection (activation dtype): r, k and v heads at the offsets below
    int64_t row_stride;
    int r_off, k_off, v_off;
    float* decay;           // [rows, decay_stride]: heads x d pre-activations of the decay; the decays afterwards
    int64_t decay_stride;
    const float* decay_bias;   // [heads * d] or null
    float decay_scale;         // w = exp(-decay_scale * sigmoid(z))
    float* remove;          // [rows, remove_stride]: heads x d pre-activations of the removal rate; a * u afterwards
    int64_t remove_stride;
    const float* remove_bias;
    const float* low;       // single tokens only, or null: [rows, low_stride] holding `rank` numbers whose tanh, times w2, is the
    int64_t low_stride;     // decay's pre-activation (decay is then not read)
    const void* w2;         // [heads * d, rank]
    int rank;
    float key_eps;          // under the root of the key's length
    float* dots;            // [rows, heads, 4] scratch for rows of more than one token: (a u) . r, k . r, 1 / |k|
    float* state;           // [slots, ...]: per head d x dv
    int64_t slot_stride, head_stride;
    float* out;             // [rows, out_stride]: heads x dv sums S^T r
    int64_t out_stride;
    const int* seq_slot;
    const int* seq_q_start;
    const int* seq_q_len;
    int rows, nseq, heads, d, dv;
    int max_slots;
    int max_q_len;          // most rows a sequence brings; 1 selects the kernel for single tokens
};
GB_API int gb_delta_scan(const DeltaStateParams* p, int dtype, int w2_dtype, cudaStream_t stream);
GB_API int gb_delta_fused_max_rank();
GB_API int gb_tanh(float* z, int rows, int cols, int64_t stride, cudaStream_t stream);

// Short causal convolution over time on the projected q | k | v, head norms, q out and k, v into the cache.
struct ConvQkvParams {
    const void* qkv;        // [rows, row_stride]: q heads, k heads, v heads (then anything else)
    int64_t row_stride;
    const float* conv_w;    // [channels, taps] or null with taps 0
    int taps, channels;
    float* state;           // [slots, state_slot_stride]: the last taps - 1 projected rows, [taps - 1][channels]
    int64_t state_slot_stride;
    int qk_norm, v_norm;
    float eps;
    void* q_out;            // [rows, q_out_stride]
    int64_t q_out_stride;
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* seq_q_start;
    const int* seq_q_len;
    const int* block_table;
    int bt_stride;
    void* k_plane;
    void* v_plane;
    int rows, nseq, heads, kv_heads, d, dv;
    int pages, max_slots;
    int max_q_len;          // most rows a sequence brings; 1: the row-wise kernel moves the state on itself
};
GB_API int gb_conv_qkv(const ConvQkvParams* p, int dtype, cudaStream_t stream);

// Attention with sigmoid weights: the softmax kernel's parameters, a bias per head on the score and a gate per head.
struct SigmoidAttnParams : AttnParamsX {
    const float* score_bias;   // [heads] or null
    const void* gate;          // [rows, gate_stride] (activation dtype): heads pre-activations, or null
    int64_t gate_stride;
};
GB_API int gb_attention_sigmoid(const SigmoidAttnParams* p, int dtype, int rows, cudaStream_t stream);

// Mixture of experts.
struct MoeRouteParams {
    const float* logits;    // [rows, logits_stride]
    int64_t logits_stride;
    int rows, experts, top;
    float renorm_eps;
    float* dense;           // [rows, experts]: the weight of every expert, 0 where not chosen
    int* index;             // [rows, top]
    float* weight;          // [rows, top]
    int score_kind;         // 0: softmax over all experts; 1: sigmoid of each logit by itself
    int renorm;             // 1: the chosen scores are divided by their sum + renorm_eps; 0: they are the weights
};
GB_API int gb_moe_route(const MoeRouteParams* p, cudaStream_t stream);
GB_API int gb_moe_act(const void* up, int64_t up_stride, const float* dense, void* act, int64_t act_stride, int rows, int experts, int ff,
                      int dtype, cudaStream_t stream);
struct MoeRowsParams {
    const void* x;          // [rows, x_stride] activation dtype
    int64_t x_stride;
    const void* up;         // [experts * ff, hidden]: the up matrices one above the other
    const void* down;       // [hidden, experts * ff]: the down matrices side by side
    void* act;              // [rows, top, ff] scratch, activation dtype
    float* out;             // [rows, out_stride]
    int64_t out_stride;
    const int* index;
    const float* weight;
    int rows, experts, top, ff, hidden;
    int act_kind;           // 0: relu(up x)^2; 1: gated, silu(gate x) * (up x), `up` holding each expert's gate rows, then its up rows
    int weight_input;       // 1: a pair's weight multiplies its expert's input; 0: its output
    float limit, slope;     // act_kind 2: g sigmoid(slope g) (v + 1) with g = min(gate x, limit), v = clamp(up x, -limit, limit)
};
GB_API int gb_moe_act_kind(const void* up, int64_t up_stride, const float* dense, void* act, int64_t act_stride, int rows, int experts, int ff,
                           int kind, int weight_input, int dtype, cudaStream_t stream);
GB_API int gb_moe_act_clamped(const void* up, int64_t up_stride, const float* dense, void* act, int64_t act_stride, int rows, int experts, int ff,
                              int kind, int weight_input, float limit, float slope, int dtype, cudaStream_t stream);
GB_API int gb_moe_rows(const MoeRowsParams* p, int dtype, int w_dtype, cudaStream_t stream);
GB_API int gb_moe_group_weights(const int* index, int rows, int top, int experts, int* offsets, int* place, int* src_row, const float* weight,
                                float* sorted_weight, cudaStream_t stream);
GB_API int gb_moe_group(const int* index, int rows, int top, int experts, int* offsets, int* place, int* src_row, cudaStream_t stream);
GB_API int gb_moe_gather(const void* x, int64_t x_stride, const int* src_row, void* xs, int pairs, int hidden, int dtype, cudaStream_t stream);
GB_API int gb_relu2(void* z, int64_t n, int dtype, cudaStream_t stream);
GB_API int gb_moe_combine(const float* ys, const int* place, const float* weight, float* out, int64_t out_stride, int rows, int top, int hidden,
                          cudaStream_t stream);
GB_API int gb_moe_rows_grouped(const MoeRowsParams* p, const int* offsets, const int* src_row, float* ys, int dtype, int w_dtype,
                               cudaStream_t stream);

// Layers whose norm stands behind the sublayer, differential attention, latent attention (postnorm.cu).
GB_API int gb_norm_scale_add(float* h, const float* y, const float* w, float eps, int rows, int n, void* x_out, int x_dtype, cudaStream_t stream);
GB_API int gb_diff_combine(const void* ctx, int64_t ctx_stride, void* out, int64_t out_stride, int rows, int heads, int per_group, int dv,
                           float lambda, float eps, float factor, int dtype, cudaStream_t stream);
GB_API int gb_add_rows_gated(float* out, const float* y, const float* z, int64_t z_stride, int rows, int n, cudaStream_t stream);
GB_API int gb_latent_prep(const void* lat, int64_t lat_stride, void* cq, const float* q_w, const float* kv_w, float eps, const float* cos_t,
                          const float* sin_t, int table_positions, const int* row_pos, const int* row_seq, const int* seq_slot,
                          const int* block_table, int bt_stride, void* k_plane, int write_kv, int rows, int q_rank, int kv_rank, int rot, int pages,
                          int max_slots, int dtype, cudaStream_t stream);
GB_API int gb_latent_q_rot(const void* q, int64_t q_stride, void* out, int64_t out_stride, int rows, int heads, int d, int rot, int out_head,
                           const float* cos_t, const float* sin_t, int table_positions, const int* row_pos, int dtype, cudaStream_t stream);
GB_API int gb_head_gemm_mma_accepts(const void* a, int64_t a_row_stride, int64_t a_head_stride, const void* w, const void* out, int64_t o_row_stride,
                                    int64_t o_head_stride, int K, int N);
GB_API int gb_head_gemm_mma(const void* a, int64_t a_row_stride, int64_t a_head_stride, const void* w, void* out, int64_t o_row_stride,
                            int64_t o_head_stride, int rows, int heads, int K, int N, cudaStream_t stream);
GB_API int gb_head_gemm(const void* a, int64_t a_row_stride, int64_t a_head_stride, const void* w, void* out, int64_t o_row_stride,
                        int64_t o_head_stride, int rows, int heads, int K, int N, int dtype, int w_dtype, cudaStream_t stream);
