// Mixture of experts: the router's choice and the experts' activation.
//
// moe_route: per row, scores s = softmax(z) over all experts in fp32, the `top` largest chosen (of equal
// scores the lower index first), weights s / (sum of the chosen s + renorm_eps).  The weights are left
// twice: as a dense row [experts] with zeros for the experts not chosen, which is what the stacked
// products of a step of many rows multiply by, and as `top` (index, weight) pairs for a step of few rows
// that reads only the chosen experts' matrices.
//
// moe_act: act[r, e * ff + i] = weight[r, e] * relu(up[r, e * ff + i])^2: the activation of every expert's
// hidden layer with the row's weight for that expert folded in, so that one product with the experts' down
// matrices side by side gives the weighted sum of the chosen experts' outputs (an expert that was not
// chosen contributes exact zeros).
//
// moe_up_rows / moe_down_rows: the same feed-forward for a step of few rows, reading only the chosen
// experts' matrices (a warp a hidden unit, or an output column, of one (row, choice) pair).
//
// moe_group / moe_gather / relu2 / moe_combine: a step of many rows sorts its (row, choice) pairs by expert
// (counts, offsets, and each pair's place in the sorted order), gathers the rows in that order so that every
// expert's rows lie together for one product an expert, squares the positive part between the two products, and
// adds each row's `top` results up with their weights in the order of the choices.  Where a pair lands inside its
// expert's group may differ from run to run; a row's result does not depend on it.
#include "api.h"
#include "common.cuh"

#include <math.h>

namespace {

constexpr int MAX_EXPERTS_PER_LANE = 16;   // experts up to 512

__global__ void __launch_bounds__(128) moe_route_kernel(MoeRouteParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + warp;
    if (row >= p.rows) return;
    const int E = p.experts;
    const float* z = p.logits + row * p.logits_stride;
    float s[MAX_EXPERTS_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS_PER_LANE; e++) {
        const int i = lane + 32 * e;
        s[e] = i < E ? z[i] : -INFINITY;
        mx = fmaxf(mx, s[e]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < MAX_EXPERTS_PER_LANE; e++) {
        const int i = lane + 32 * e;
        // the key an expert is chosen by: its softmax numerator, or, for sigmoid scores, the logit itself (the
        // sigmoid grows with it, and two large logits stay apart where their sigmoids both round to 1);
        // -inf marks what is absent or taken
        s[e] = i < E ? (p.score_kind == 1 ? s[e] : expf(s[e] - mx)) : -INFINITY;
        if (i < E && p.score_kind != 1) sum += s[e];
    }
    sum = warp_sum(sum);
    const float inv = p.score_kind == 1 ? 1.f : 1.f / sum;     // a sigmoid score stands by itself
    float* dense = p.dense + row * E;
    for (int i = lane; i < E; i += 32) dense[i] = 0.f;
    float chosen_sum = 0.f;
    float my_w = 0.f;      // lane k keeps the k-th choice
    int my_i = 0;
    for (int k = 0; k < p.top; k++) {
        float best = -INFINITY;
        int best_i = 0x7fffffff;
#pragma unroll
        for (int e = 0; e < MAX_EXPERTS_PER_LANE; e++) {
            const int i = lane + 32 * e;
            if (s[e] > best) best = s[e], best_i = i;     // within a lane indices grow with e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ob > best || (ob == best && oi < best_i)) best = ob, best_i = oi;
        }
#pragma unroll
        for (int e = 0; e < MAX_EXPERTS_PER_LANE; e++)
            if (lane + 32 * e == best_i) s[e] = -INFINITY;
        const float sc = p.score_kind == 1 ? 1.f / (1.f + expf(-best)) : best * inv;
        chosen_sum += sc;
        if (lane == (k & 31)) my_w = sc, my_i = best_i;
        if (k >= 32 && lane == 0) {}   // more than 32 choices are refused on the host
    }
    const float norm = p.renorm ? 1.f / (chosen_sum + p.renorm_eps) : 1.f;
    __syncwarp();
    if (lane < p.top) {
        const float w = my_w * norm;
        dense[my_i] = w;
        p.index[row * p.top + lane] = my_i;
        p.weight[row * p.top + lane] = w;
    }
}

// What an expert's hidden unit makes of its product(s) z (and, for a gated expert, u) and the pair's weight w:
// kind 0: relu(z)^2; kind 1: silu(z) * u; kind 2: g sigmoid(slope g) (v + 1) with g = min(z, limit) and
// v = clamp(u, -limit, limit).  The weight multiplies the result, or (weight_input) the expert's
// input, which for products without biases is the same as multiplying z and u.
__device__ __forceinline__ float expert_act(float z, float u, float w, int kind, int weight_input, float limit = 0.f, float slope = 1.f) {
    if (weight_input) z *= w, u *= w;
    float a;
    if (kind == 1) {
        a = z / (1.f + expf(-z)) * u;
    } else if (kind == 2) {
        const float g = fminf(z, limit), v = fminf(fmaxf(u, -limit), limit);
        a = g / (1.f + expf(-slope * g)) * (v + 1.f);
    } else {
        const float r = fmaxf(z, 0.f);
        a = r * r;
    }
    return weight_input ? a : w * a;
}

// up: [rows, experts * (kind 1: 2 ff, gate rows then up rows of each expert; else ff)]; dense null: every weight is 1
template <typename T>
__global__ void moe_act_kernel(const T* __restrict__ up, int64_t up_stride, const float* __restrict__ dense, T* __restrict__ act,
                               int64_t act_stride, int rows, int experts, int ff, int kind, int weight_input, float limit, float slope) {
    const int64_t n = (int64_t)experts * ff;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * n) return;
    const int64_t r = idx / n, c = idx % n;
    const int64_t e = c / ff, i = c - e * ff;
    const float w = dense ? dense[r * experts + e] : 1.f;
    float z, u = 0.f;
    if (kind != 0) {
        z = to_f32<T>(up[r * up_stride + e * 2 * ff + i]);
        u = to_f32<T>(up[r * up_stride + e * 2 * ff + ff + i]);
    } else {
        z = to_f32<T>(up[r * up_stride + c]);
    }
    act[r * act_stride + c] = from_f32<T>(expert_act(z, u, w, kind, weight_input, limit, slope));
}

// a warp's share of the dot product of a weight row and a row of activations, 16 bytes a lane where both allow it
template <typename T, typename TW>
__device__ __forceinline__ float warp_dot(const TW* __restrict__ w, const T* __restrict__ x, int n, int lane) {
    float a = 0.f;
    for (int c = lane; c < n; c += 32) a = fmaf(to_f32<TW>(w[c]), to_f32<T>(x[c]), a);
    return a;
}
template <>
__device__ __forceinline__ float warp_dot<__nv_bfloat16, __nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ x,
                                                                        int n, int lane) {
    float a = 0.f;
    if (!(n & 7) && !((uintptr_t)w & 15) && !((uintptr_t)x & 15)) {
        for (int c = lane * 8; c < n; c += 256) {
            const uint4 wv = *reinterpret_cast<const uint4*>(w + c), xv = *reinterpret_cast<const uint4*>(x + c);
            const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
            const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                a = fmaf(__low2float(wh[e]), __low2float(xh[e]), a);
                a = fmaf(__high2float(wh[e]), __high2float(xh[e]), a);
            }
        }
        return a;
    }
    for (int c = lane; c < n; c += 32) a = fmaf(__bfloat162float(w[c]), __bfloat162float(x[c]), a);
    return a;
}

// few rows: act[r, k, i] = weight[r, k] * relu(W_up[index[r, k]][i, :] . x[r])^2, a warp a hidden unit
template <typename T, typename TW>
__global__ void __launch_bounds__(128) moe_up_rows_kernel(MoeRowsParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * 4 + warp;
    const int pair = blockIdx.y;            // row * top + k
    if (i >= p.ff) return;
    const int r = pair / p.top;
    const int e = p.index[pair];
    const int per = p.act_kind != 0 ? 2 : 1;      // a gated expert holds its gate rows, then its up rows
    const TW* w = (const TW*)p.up + ((int64_t)e * per * p.ff + i) * p.hidden;
    const T* x = (const T*)p.x + (int64_t)r * p.x_stride;
    const float a = warp_sum(warp_dot<T, TW>(w, x, p.hidden, lane));
    const float b = p.act_kind != 0 ? warp_sum(warp_dot<T, TW>(w + (int64_t)p.ff * p.hidden, x, p.hidden, lane)) : 0.f;
    if (lane == 0) {
        // the same roundings as the stacked path: the product in the activation dtype, then the activation
        ((T*)p.act)[(int64_t)pair * p.ff + i] =
            from_f32<T>(expert_act(to_f32<T>(from_f32<T>(a)), to_f32<T>(from_f32<T>(b)), p.weight[pair], p.act_kind, p.weight_input, p.limit, p.slope));
    }
}

// out[r, c] = sum_k W_down[index[r, k]][c, :] . act[r, k, :], a warp an output column of a row
template <typename T, typename TW>
__global__ void __launch_bounds__(128) moe_down_rows_kernel(MoeRowsParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 4 + warp;
    const int r = blockIdx.y;
    if (c >= p.hidden) return;
    float a = 0.f;
    for (int k = 0; k < p.top; k++) {
        const int pair = r * p.top + k;
        const int e = p.index[pair];
        const TW* w = (const TW*)p.down + ((int64_t)c * p.experts + e) * p.ff;      // the down matrices side by side: [hidden, experts * ff]
        a += warp_dot<T, TW>(w, (const T*)p.act + (int64_t)pair * p.ff, p.ff, lane);
    }
    a = warp_sum(a);
    if (lane == 0) p.out[(int64_t)r * p.out_stride + c] = a;
}

// The same two products with the pairs sorted by expert (moe_group): a warp takes a hidden unit (an output column) of
// ONE expert and walks that expert's pairs, so an expert's matrices are read from memory once however many rows chose
// it (the row of the matrix stays in the first-level cache from pair to pair).  act[p, i] = relu(up_e[i] . x[src_row[p]])^2
// at the pair's sorted place p, ys[p, c] = down_e[c] . act[p]; the weights are applied when the rows are added up.
template <typename T, typename TW>
__global__ void __launch_bounds__(128) moe_up_grouped_kernel(MoeRowsParams p, const int* __restrict__ offsets, const int* __restrict__ src_row) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * 4 + warp, e = blockIdx.y;
    const int lo = offsets[e], hi = offsets[e + 1];
    if (i >= p.ff || lo == hi) return;
    const int per = p.act_kind != 0 ? 2 : 1;
    const TW* w = (const TW*)p.up + ((int64_t)e * per * p.ff + i) * p.hidden;
    for (int at = lo; at < hi; at++) {
        const T* x = (const T*)p.x + (int64_t)src_row[at] * p.x_stride;
        const float a = warp_sum(warp_dot<T, TW>(w, x, p.hidden, lane));
        const float b = p.act_kind != 0 ? warp_sum(warp_dot<T, TW>(w + (int64_t)p.ff * p.hidden, x, p.hidden, lane)) : 0.f;
        if (lane == 0) {
            // a weight on the expert's input is applied here (p.weight: the pairs' weights in sorted order), one on its
            // output when the rows are added up
            const float pw = p.weight_input ? p.weight[at] : 1.f;
            ((T*)p.act)[(int64_t)at * p.ff + i] =
                from_f32<T>(expert_act(to_f32<T>(from_f32<T>(a)), to_f32<T>(from_f32<T>(b)), pw, p.act_kind, p.weight_input, p.limit, p.slope));
        }
    }
}

template <typename T, typename TW>
__global__ void __launch_bounds__(128) moe_down_grouped_kernel(MoeRowsParams p, const int* __restrict__ offsets, float* __restrict__ ys) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * 4 + warp, e = blockIdx.y;
    const int lo = offsets[e], hi = offsets[e + 1];
    if (c >= p.hidden || lo == hi) return;
    const TW* w = (const TW*)p.down + ((int64_t)c * p.experts + e) * p.ff;
    for (int at = lo; at < hi; at++) {
        const float a = warp_sum(warp_dot<T, TW>(w, (const T*)p.act + (int64_t)at * p.ff, p.ff, lane));
        if (lane == 0) ys[(int64_t)at * p.hidden + c] = a;
    }
}

constexpr int GROUP_THREADS = 1024;
constexpr int GROUP_MAX_EXPERTS = 512;

// one CTA: counts of the pairs of each expert, offsets of the experts' groups, and a place in its group for every pair
__global__ void __launch_bounds__(GROUP_THREADS) moe_group_kernel(const int* __restrict__ index, int pairs, int top, int experts,
                                                                 int* __restrict__ offsets, int* __restrict__ place, int* __restrict__ src_row,
                                                                 const float* __restrict__ weight, float* __restrict__ sorted_weight) {
    __shared__ int count[GROUP_MAX_EXPERTS], cursor[GROUP_MAX_EXPERTS];
    const int tid = threadIdx.x;
    for (int e = tid; e < experts; e += GROUP_THREADS) count[e] = 0;
    __syncthreads();
    for (int i = tid; i < pairs; i += GROUP_THREADS) atomicAdd(&count[index[i]], 1);
    __syncthreads();
    if (tid == 0) {
        int at = 0;
        for (int e = 0; e < experts; e++) {
            offsets[e] = at;
            cursor[e] = at;
            at += count[e];
        }
        offsets[experts] = at;
    }
    __syncthreads();
    for (int i = tid; i < pairs; i += GROUP_THREADS) {
        const int at = atomicAdd(&cursor[index[i]], 1);
        place[i] = at;
        src_row[at] = i / top;
        if (sorted_weight) sorted_weight[at] = weight[i];
    }
}

// xs[p, :] = x[src_row[p], :], 16 bytes a thread where rows allow it
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, int64_t x_stride, const int* __restrict__ src_row, T* __restrict__ xs, int hidden) {
    const int64_t p = blockIdx.x;
    const T* src = x + (int64_t)src_row[p] * x_stride;
    T* dst = xs + p * hidden;
    constexpr int V = 16 / sizeof(T);
    if (!(hidden % V) && !(x_stride % V) && !((uintptr_t)x & 15) && !((uintptr_t)xs & 15)) {
        for (int c = threadIdx.x; c < hidden / V; c += blockDim.x)
            reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = src[c];
    }
}

template <typename T>
__global__ void relu2_kernel(T* __restrict__ z, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = fmaxf(to_f32<T>(z[i]), 0.f);
    z[i] = from_f32<T>(v * v);
}

// out[r, :] = sum_k weight[r, k] * ys[place[r * top + k], :], in the order of k
__global__ void moe_combine_kernel(const float* __restrict__ ys, const int* __restrict__ place, const float* __restrict__ weight,
                                   float* __restrict__ out, int64_t out_stride, int top, int hidden) {
    const int64_t r = blockIdx.x;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float a = 0.f;
        for (int k = 0; k < top; k++) a = fmaf(weight ? weight[r * top + k] : 1.f, ys[(int64_t)place[r * top + k] * hidden + c], a);
        out[r * out_stride + c] = a;
    }
}

}  // namespace

GB_API int gb_moe_group(const int* index, int rows, int top, int experts, int* offsets, int* place, int* src_row, cudaStream_t stream) {
    return gb_moe_group_weights(index, rows, top, experts, offsets, place, src_row, nullptr, nullptr, stream);
}

// The same, and the pairs' weights in sorted order beside them (sorted_weight[place[i]] = weight[i]) if both are given.
GB_API int gb_moe_group_weights(const int* index, int rows, int top, int experts, int* offsets, int* place, int* src_row, const float* weight,
                                float* sorted_weight, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (experts <= 0 || experts > GROUP_MAX_EXPERTS || top <= 0) GB_REFUSE("moe_group: %d experts, %d a token", experts, top);
    if ((weight != nullptr) != (sorted_weight != nullptr)) GB_REFUSE("moe_group: weights in and out go together");
    moe_group_kernel<<<1, GROUP_THREADS, 0, stream>>>(index, rows * top, top, experts, offsets, place, src_row, weight, sorted_weight);
    GB_CHECK_LAUNCH("moe_group");
    return 0;
}

GB_API int gb_moe_gather(const void* x, int64_t x_stride, const int* src_row, void* xs, int pairs, int hidden, int dtype, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (dtype == GB_F32)
        moe_gather_kernel<float><<<pairs, 128, 0, stream>>>((const float*)x, x_stride, src_row, (float*)xs, hidden);
    else if (dtype == GB_BF16)
        moe_gather_kernel<__nv_bfloat16><<<pairs, 128, 0, stream>>>((const __nv_bfloat16*)x, x_stride, src_row, (__nv_bfloat16*)xs, hidden);
    else
        GB_REFUSE("moe_gather: unknown dtype %d", dtype);
    GB_CHECK_LAUNCH("moe_gather");
    return 0;
}

GB_API int gb_relu2(void* z, int64_t n, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == GB_F32)
        relu2_kernel<float><<<blocks, 256, 0, stream>>>((float*)z, n);
    else if (dtype == GB_BF16)
        relu2_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)z, n);
    else
        GB_REFUSE("relu2: unknown dtype %d", dtype);
    GB_CHECK_LAUNCH("relu2");
    return 0;
}

GB_API int gb_moe_combine(const float* ys, const int* place, const float* weight, float* out, int64_t out_stride, int rows, int top, int hidden,
                          cudaStream_t stream) {
    if (rows <= 0) return 0;
    moe_combine_kernel<<<rows, 256, 0, stream>>>(ys, place, weight, out, out_stride, top, hidden);
    GB_CHECK_LAUNCH("moe_combine");
    return 0;
}

GB_API int gb_moe_route(const MoeRouteParams* pp, cudaStream_t stream) {
    MoeRouteParams p = *pp;
    if (p.rows <= 0) return 0;
    if (p.experts <= 0 || p.experts > 32 * MAX_EXPERTS_PER_LANE) GB_REFUSE("moe_route: %d experts; 1 to %d", p.experts, 32 * MAX_EXPERTS_PER_LANE);
    if (p.top <= 0 || p.top > p.experts || p.top > 32) GB_REFUSE("moe_route: %d of %d experts a token; at most 32", p.top, p.experts);
    if (!p.logits || !p.dense || !p.index || !p.weight) GB_REFUSE("moe_route: a tensor is missing");
    moe_route_kernel<<<(p.rows + 3) / 4, 128, 0, stream>>>(p);
    GB_CHECK_LAUNCH("moe_route");
    return 0;
}

GB_API int gb_moe_act(const void* up, int64_t up_stride, const float* dense, void* act, int64_t act_stride, int rows, int experts, int ff,
                      int dtype, cudaStream_t stream) {
    return gb_moe_act_kind(up, up_stride, dense, act, act_stride, rows, experts, ff, 0, 0, dtype, stream);
}

// kind 0: weight * relu(up)^2; kind 1: gated, silu(gate) * up with each expert's gate columns ahead of its up columns.
// weight_input 1: the weight multiplies the expert's input instead of its output.  dense null: weights of 1.
GB_API int gb_moe_act_kind(const void* up, int64_t up_stride, const float* dense, void* act, int64_t act_stride, int rows, int experts, int ff,
                           int kind, int weight_input, int dtype, cudaStream_t stream) {
    return gb_moe_act_clamped(up, up_stride, dense, act, act_stride, rows, experts, ff, kind, weight_input, 0.f, 1.f, dtype, stream);
}

// kind 2 as well: g sigmoid(slope g) (v + 1), g = min(gate, limit), v = clamp(up, -limit, limit), columns laid out as for kind 1.
GB_API int gb_moe_act_clamped(const void* up, int64_t up_stride, const float* dense, void* act, int64_t act_stride, int rows, int experts, int ff,
                              int kind, int weight_input, float limit, float slope, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (experts <= 0 || ff <= 0) GB_REFUSE("moe_act: %d experts of %d", experts, ff);
    if (kind < 0 || kind > 2) GB_REFUSE("moe_act: unknown activation %d", kind);
    const int64_t total = (int64_t)rows * experts * ff;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == GB_F32)
        moe_act_kernel<float><<<blocks, 256, 0, stream>>>((const float*)up, up_stride, dense, (float*)act, act_stride, rows, experts, ff, kind, weight_input, limit, slope);
    else if (dtype == GB_BF16)
        moe_act_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)up, up_stride, dense, (__nv_bfloat16*)act, act_stride,
                                                                  rows, experts, ff, kind, weight_input, limit, slope);
    else
        GB_REFUSE("moe_act: unknown dtype %d", dtype);
    GB_CHECK_LAUNCH("moe_act");
    return 0;
}

GB_API int gb_moe_rows(const MoeRowsParams* pp, int dtype, int w_dtype, cudaStream_t stream) {
    MoeRowsParams p = *pp;
    if (p.rows <= 0) return 0;
    if (p.experts <= 0 || p.top <= 0 || p.ff <= 0 || p.hidden <= 0) GB_REFUSE("moe_rows: %d experts, %d a token, %d x %d", p.experts, p.top, p.ff, p.hidden);
    if (!p.x || !p.up || !p.down || !p.act || !p.out || !p.index || !p.weight) GB_REFUSE("moe_rows: a tensor is missing");
    dim3 ugrid((p.ff + 3) / 4, p.rows * p.top), dgrid((p.hidden + 3) / 4, p.rows);
    if (ugrid.y > 65535) GB_REFUSE("moe_rows: %d rows exceed one launch", p.rows);
    if (dtype == GB_BF16 && w_dtype == GB_BF16) {
        moe_up_rows_kernel<__nv_bfloat16, __nv_bfloat16><<<ugrid, 128, 0, stream>>>(p);
        moe_down_rows_kernel<__nv_bfloat16, __nv_bfloat16><<<dgrid, 128, 0, stream>>>(p);
    } else if (dtype == GB_F32 && w_dtype == GB_F32) {
        moe_up_rows_kernel<float, float><<<ugrid, 128, 0, stream>>>(p);
        moe_down_rows_kernel<float, float><<<dgrid, 128, 0, stream>>>(p);
    } else {
        GB_REFUSE("moe_rows: activations of dtype %d with weights of dtype %d", dtype, w_dtype);
    }
    GB_CHECK_LAUNCH("moe_rows");
    return 0;
}

// The few-row feed-forward with the pairs sorted by expert: `offsets` and `src_row` as moe_group left them, `ys`
// float32 [rows * top, hidden] receives every pair's output at its sorted place (moe_combine adds them up).
GB_API int gb_moe_rows_grouped(const MoeRowsParams* pp, const int* offsets, const int* src_row, float* ys, int dtype, int w_dtype,
                               cudaStream_t stream) {
    MoeRowsParams p = *pp;
    if (p.rows <= 0) return 0;
    if (p.experts <= 0 || p.experts > 65535 || p.top <= 0 || p.ff <= 0 || p.hidden <= 0) GB_REFUSE("moe_rows: %d experts, %d a token, %d x %d", p.experts, p.top, p.ff, p.hidden);
    if (!p.x || !p.up || !p.down || !p.act || !offsets || !src_row || !ys || (p.weight_input && !p.weight)) GB_REFUSE("moe_rows: a tensor is missing");
    dim3 ugrid((p.ff + 3) / 4, p.experts), dgrid((p.hidden + 3) / 4, p.experts);
    if (dtype == GB_BF16 && w_dtype == GB_BF16) {
        moe_up_grouped_kernel<__nv_bfloat16, __nv_bfloat16><<<ugrid, 128, 0, stream>>>(p, offsets, src_row);
        moe_down_grouped_kernel<__nv_bfloat16, __nv_bfloat16><<<dgrid, 128, 0, stream>>>(p, offsets, ys);
    } else if (dtype == GB_F32 && w_dtype == GB_F32) {
        moe_up_grouped_kernel<float, float><<<ugrid, 128, 0, stream>>>(p, offsets, src_row);
        moe_down_grouped_kernel<float, float><<<dgrid, 128, 0, stream>>>(p, offsets, ys);
    } else {
        GB_REFUSE("moe_rows: activations of dtype %d with weights of dtype %d", dtype, w_dtype);
    }
    GB_CHECK_LAUNCH("moe_rows_grouped");
    return 0;
}
