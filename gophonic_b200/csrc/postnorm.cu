// Row-wise kernels of layers whose norm stands behind the sublayer, of differential attention and of latent attention.
//
// norm_scale_add:   h += y / sqrt(mean(y^2) + eps) * w  on float32 rows (w: the norm's weight with every constant factor of
//                   the sublayer folded in), and, if asked, the new row once more in the activation dtype for the sublayer
//                   that reads it next.  One pass: a thread keeps its share of y in registers between the sum and the store.
// diff_combine:     o = a1 - lambda a2 per head, o / sqrt(mean(o^2) + eps) * factor: the two softmax maps of a head lie
//                   as many heads apart in the attention output as a group has query heads.
// add_rows_gated:   out += sigmoid(z[row]) * y, z one number a row.
// latent_prep:      per row of a fused down-projection [q latent | kv latent | rotated key part]: RMS norm of the q latent
//                   with its weight into a buffer of its own; RMS norm of the kv latent with its weight and the rotation of
//                   the key part (neighbouring channels turn together), both into the key plane at the row's position.
// latent_q_rot:     the rotated channels of every query head, rotated and copied behind the head's absorbed channels.
// head_gemm:        out[r, h, :] = a[r, h, :] W_h for every head h in one launch, W [heads, K, N]; float32 sums.
// head_gemm_mma:    the same for many bfloat16 rows on the tensor cores, W [heads, N, K].
//
// Everything is computed in float32 whatever the activation dtype; a row's result depends on that row alone and the
// order of every sum is fixed by the row's width.
#include "api.h"
#include "common.cuh"
#include "mma.cuh"

#include <math.h>

namespace {

__device__ __forceinline__ float block_sum_256(float v, float* part) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) t += part[i];   // every thread adds the eight warp sums in the same order
    __syncthreads();
    return t;
}

constexpr int NSA_KEEP = 8;     // elements of y a thread keeps in registers (rows up to 2048 wide are read once)

template <typename TO>
__global__ void __launch_bounds__(256) norm_scale_add_kernel(float* __restrict__ h, const float* __restrict__ y, const float* __restrict__ w,
                                                             float eps, int n, TO* __restrict__ x_out) {
    __shared__ float part[8];
    const int64_t row = blockIdx.x;
    const float* yr = y + row * n;
    float* hr = h + row * n;
    float keep[NSA_KEEP];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NSA_KEEP; j++) {
        const int i = threadIdx.x + 256 * j;
        keep[j] = i < n ? yr[i] : 0.f;
        ss += keep[j] * keep[j];
    }
    for (int i = threadIdx.x + 256 * NSA_KEEP; i < n; i += 256) {
        const float v = yr[i];
        ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum_256(ss, part) / (float)n + eps);
#pragma unroll
    for (int j = 0; j < NSA_KEEP; j++) {
        const int i = threadIdx.x + 256 * j;
        if (i < n) {
            const float v = hr[i] + keep[j] * inv * w[i];
            hr[i] = v;
            if (x_out) x_out[row * n + i] = from_f32<TO>(v);
        }
    }
    for (int i = threadIdx.x + 256 * NSA_KEEP; i < n; i += 256) {
        const float v = hr[i] + yr[i] * inv * w[i];
        hr[i] = v;
        if (x_out) x_out[row * n + i] = from_f32<TO>(v);
    }
}

// one warp a (row, head)
template <typename T>
__global__ void __launch_bounds__(128) diff_combine_kernel(const T* __restrict__ ctx, int64_t ctx_stride, T* __restrict__ out, int64_t out_stride,
                                                           int rows, int heads, int per_group, int dv, float lambda, float eps, float factor) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * 4 + warp;
    if (unit >= (int64_t)rows * heads) return;
    const int64_t r = unit / heads;
    const int hd = (int)(unit % heads);
    const int g = hd / per_group, hi = hd % per_group;
    // the attention ran with the query heads of a group ordered [map 1 of every head, map 2 of every head]
    const T* a1 = ctx + r * ctx_stride + ((int64_t)(g * 2) * per_group + hi) * dv;
    const T* a2 = a1 + (int64_t)per_group * dv;
    T* o = out + r * out_stride + (int64_t)hd * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) {
        const float v = to_f32<T>(a1[c]) - lambda * to_f32<T>(a2[c]);
        ss += v * v;
    }
    const float inv = factor / sqrtf(warp_sum(ss) / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) o[c] = from_f32<T>((to_f32<T>(a1[c]) - lambda * to_f32<T>(a2[c])) * inv);
}

__global__ void add_rows_gated_kernel(float* __restrict__ out, const float* __restrict__ y, const float* __restrict__ z, int64_t z_stride, int n) {
    const int64_t r = blockIdx.x;
    const float g = 1.f / (1.f + expf(-z[r * z_stride]));
    for (int c = threadIdx.x; c < n; c += blockDim.x) out[r * n + c] += g * y[r * n + c];
}

struct LatentPrepArgs {
    const void* lat;      // [rows, lat_stride]: q_rank, then kv_rank, then rot channels
    int64_t lat_stride;
    void* cq;             // [rows, q_rank] (activation dtype)
    const float* q_w;     // [q_rank]
    const float* kv_w;    // [kv_rank]
    float eps;
    const float* cos_t;   // [positions, rot / 2]
    const float* sin_t;
    int table_positions;
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* block_table;
    int bt_stride;
    void* k_plane;        // [pages, 1, 64, kv_rank + rot]
    int write_kv;
    int rows, q_rank, kv_rank, rot;
    int pages, max_slots;
};

template <typename T>
__global__ void __launch_bounds__(256) latent_prep_kernel(LatentPrepArgs p) {
    __shared__ float part[8];
    const int64_t r = blockIdx.x;
    const T* src = (const T*)p.lat + r * p.lat_stride;
    // the query latent
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.q_rank; i += 256) {
        const float v = to_f32<T>(src[i]);
        ss += v * v;
    }
    float inv = 1.0f / sqrtf(block_sum_256(ss, part) / (float)p.q_rank + p.eps);
    T* cq = (T*)p.cq + r * p.q_rank;
    for (int i = threadIdx.x; i < p.q_rank; i += 256) cq[i] = from_f32<T>(to_f32<T>(src[i]) * inv * p.q_w[i]);
    if (!p.write_kv) return;
    // the key/value latent and the rotated key part, into the cache
    const T* kv = src + p.q_rank;
    ss = 0.f;
    for (int i = threadIdx.x; i < p.kv_rank; i += 256) {
        const float v = to_f32<T>(kv[i]);
        ss += v * v;
    }
    inv = 1.0f / sqrtf(block_sum_256(ss, part) / (float)p.kv_rank + p.eps);
    const int pos = p.row_pos[r];
    const int slot = p.seq_slot[p.row_seq[r]];
    const int64_t page = page_of(block_table_row(p.block_table, p.bt_stride, slot, p.max_slots), pos, p.bt_stride, p.pages);
    T* dst = (T*)p.k_plane + (page * GB_PAGE + (pos % GB_PAGE)) * (int64_t)(p.kv_rank + p.rot);
    for (int i = threadIdx.x; i < p.kv_rank; i += 256) dst[i] = from_f32<T>(to_f32<T>(kv[i]) * inv * p.kv_w[i]);
    const int half = p.rot / 2;
    const int tpos = (half == 0 || gb_check(pos, p.table_positions, GB_CHECK_ROPE_POSITION)) ? pos : 0;
    const float* c = p.cos_t + (int64_t)tpos * half;
    const float* s = p.sin_t + (int64_t)tpos * half;
    for (int j = threadIdx.x; j < half; j += 256) {
        const float u = to_f32<T>(kv[p.kv_rank + 2 * j]), v = to_f32<T>(kv[p.kv_rank + 2 * j + 1]);
        dst[p.kv_rank + 2 * j] = from_f32<T>(u * c[j] - v * s[j]);
        dst[p.kv_rank + 2 * j + 1] = from_f32<T>(v * c[j] + u * s[j]);
    }
}

// q: [rows, heads, d + rot]; out: [rows, heads, out_head] whose last rot channels receive the rotated ones
template <typename T>
__global__ void latent_q_rot_kernel(const T* __restrict__ q, int64_t q_stride, T* __restrict__ out, int64_t out_stride, int heads, int d, int rot,
                                    int out_head, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_positions,
                                    const int* __restrict__ row_pos) {
    const int64_t r = blockIdx.x;
    const int half = rot / 2;
    const int pos = row_pos[r];
    const int tpos = gb_check(pos, table_positions, GB_CHECK_ROPE_POSITION) ? pos : 0;
    const float* c = cos_t + (int64_t)tpos * half;
    const float* s = sin_t + (int64_t)tpos * half;
    for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
        const int hd = idx / half, j = idx - hd * half;
        const T* src = q + r * q_stride + (int64_t)hd * (d + rot) + d;
        T* dst = out + r * out_stride + (int64_t)hd * out_head + (out_head - rot);
        const float u = to_f32<T>(src[2 * j]), v = to_f32<T>(src[2 * j + 1]);
        dst[2 * j] = from_f32<T>(u * c[j] - v * s[j]);
        dst[2 * j + 1] = from_f32<T>(v * c[j] + u * s[j]);
    }
}

// out[r, h, n] = sum_k a[r, h, k] W[h, k, n] for few rows: a CTA of eight warps takes 8 rows of one head and 32 columns; the
// rows are staged as float32, a lane owns one column, the warps split K (eight loads of W in flight a lane, along n whole
// segments a warp) and their sums meet in shared memory, added in warp order.
constexpr int HG_ROWS = 8, HG_WARPS = 8, HG_COLS = 32;

template <typename T, typename TW>
__global__ void __launch_bounds__(32 * HG_WARPS) head_gemm_kernel(const T* __restrict__ a, int64_t a_row_stride, int64_t a_head_stride,
                                                                 const TW* __restrict__ w, T* __restrict__ out, int64_t o_row_stride,
                                                                 int64_t o_head_stride, int rows, int K, int N) {
    extern __shared__ float as[];   // [HG_ROWS][K], then [HG_WARPS][HG_ROWS][HG_COLS]
    float* red = as + HG_ROWS * K;
    const int hd = blockIdx.y;
    const int r0 = blockIdx.z * HG_ROWS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * HG_COLS + lane;
    for (int idx = threadIdx.x; idx < HG_ROWS * K; idx += 32 * HG_WARPS) {
        const int rr = idx / K, k = idx - rr * K;
        as[idx] = r0 + rr < rows ? to_f32<T>(a[(int64_t)(r0 + rr) * a_row_stride + (int64_t)hd * a_head_stride + k]) : 0.f;
    }
    __syncthreads();
    const int per = (K + HG_WARPS - 1) / HG_WARPS;
    const int k_lo = warp * per, k_hi = k_lo + per < K ? k_lo + per : K;
    float acc[HG_ROWS];
#pragma unroll
    for (int rr = 0; rr < HG_ROWS; rr++) acc[rr] = 0.f;
    if (n < N) {
        const TW* wp = w + (int64_t)hd * K * N + n;
        int k = k_lo;
        for (; k + 7 < k_hi; k += 8) {
            float wv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) wv[u] = to_f32<TW>(wp[(int64_t)(k + u) * N]);
#pragma unroll
            for (int u = 0; u < 8; u++)
#pragma unroll
                for (int rr = 0; rr < HG_ROWS; rr++) acc[rr] = fmaf(as[rr * K + k + u], wv[u], acc[rr]);
        }
        for (; k < k_hi; k++) {
            const float wv = to_f32<TW>(wp[(int64_t)k * N]);
#pragma unroll
            for (int rr = 0; rr < HG_ROWS; rr++) acc[rr] = fmaf(as[rr * K + k], wv, acc[rr]);
        }
    }
#pragma unroll
    for (int rr = 0; rr < HG_ROWS; rr++) red[(warp * HG_ROWS + rr) * HG_COLS + lane] = acc[rr];
    __syncthreads();
    for (int idx = threadIdx.x; idx < HG_ROWS * HG_COLS; idx += 32 * HG_WARPS) {
        const int rr = idx / HG_COLS, c = idx - rr * HG_COLS;
        const int col = blockIdx.x * HG_COLS + c;
        if (r0 + rr >= rows || col >= N) continue;
        float t = 0.f;
#pragma unroll
        for (int ww = 0; ww < HG_WARPS; ww++) t += red[(ww * HG_ROWS + rr) * HG_COLS + c];
        out[(int64_t)(r0 + rr) * o_row_stride + (int64_t)hd * o_head_stride + col] = from_f32<T>(t);
    }
}

// The same product for many rows on the tensor cores (bf16 mma.sync), W as [heads][N][K]: a CTA takes 64 rows and 64
// columns of one head, a warp 16 of the rows; K in pieces of 64, double-buffered with cp.async.
constexpr int HM_T = 64, HM_S = HM_T + 8;

__global__ void __launch_bounds__(128) head_gemm_mma_kernel(const __nv_bfloat16* __restrict__ a, int64_t a_row_stride, int64_t a_head_stride,
                                                            const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                            int64_t o_row_stride, int64_t o_head_stride, int rows, int K, int N) {
    __shared__ __align__(16) __nv_bfloat16 As[2][HM_T][HM_S];
    __shared__ __align__(16) __nv_bfloat16 Ws[2][HM_T][HM_S];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int n0 = blockIdx.x * HM_T, hd = blockIdx.y, r0 = blockIdx.z * HM_T;
    const __nv_bfloat16* ap = a + (int64_t)hd * a_head_stride;
    const __nv_bfloat16* wp = w + (int64_t)hd * N * K;
    const int chunks = (K + HM_T - 1) / HM_T;
    auto load = [&](int c) {
        const int buf = c & 1, k0 = c * HM_T;
        for (int idx = tid; idx < HM_T * 8; idx += 128) {
            const int r = idx >> 3, piece = idx & 7;
            const int k = k0 + piece * 8;
            const bool ka = k < K;
            const bool oka = ka && r0 + r < rows, okw = ka && n0 + r < N;
            cp_async16(&As[buf][r][piece * 8], oka ? ap + (int64_t)(r0 + r) * a_row_stride + k : ap, oka ? 16 : 0);
            cp_async16(&Ws[buf][r][piece * 8], okw ? wp + (int64_t)(n0 + r) * K + k : wp, okw ? 16 : 0);
        }
    };
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[j][e] = 0.f;
    load(0);
    cp_async_commit();
    for (int c = 0; c < chunks; c++) {
        cp_async_wait<0>();
        __syncthreads();
        if (c + 1 < chunks) load(c + 1);
        cp_async_commit();
        const int buf = c & 1;
#pragma unroll
        for (int ks = 0; ks < HM_T / 16; ks++) {
            uint32_t af[4];
            ldmatrix_x4(af, &As[buf][warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
            for (int jp = 0; jp < 4; jp++) {
                uint32_t b[4];
                ldmatrix_x4(b, &Ws[buf][jp * 16 + (lane & 7) + (lane >> 4) * 8][ks * 16 + ((lane >> 3) & 1) * 8]);
                mma_bf16_16816(acc[jp * 2], af[0], af[1], af[2], af[3], b[0], b[1]);
                mma_bf16_16816(acc[jp * 2 + 1], af[0], af[1], af[2], af[3], b[2], b[3]);
            }
        }
    }
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int r = r0 + warp * 16 + g + 8 * e;
        if (r >= rows) continue;
        __nv_bfloat16* op = out + (int64_t)r * o_row_stride + (int64_t)hd * o_head_stride;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int col = n0 + j * 8 + t4 * 2;
            if (col + 1 < N)
                *reinterpret_cast<uint32_t*>(op + col) = pack_bf16(acc[j][2 * e], acc[j][2 * e + 1]);
            else if (col < N)
                op[col] = __float2bfloat16_rn(acc[j][2 * e]);
        }
    }
}

}  // namespace

GB_API int gb_norm_scale_add(float* h, const float* y, const float* w, float eps, int rows, int n, void* x_out, int x_dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n <= 0) GB_REFUSE("norm_scale_add: rows of %d", n);
    if (!h || !y || !w) GB_REFUSE("norm_scale_add: a tensor is missing");
    if (!x_out || x_dtype == GB_F32)
        norm_scale_add_kernel<float><<<rows, 256, 0, stream>>>(h, y, w, eps, n, (float*)x_out);
    else if (x_dtype == GB_BF16)
        norm_scale_add_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>(h, y, w, eps, n, (__nv_bfloat16*)x_out);
    else
        GB_REFUSE("norm_scale_add: unknown dtype %d", x_dtype);
    GB_CHECK_LAUNCH("norm_scale_add");
    return 0;
}

GB_API int gb_diff_combine(const void* ctx, int64_t ctx_stride, void* out, int64_t out_stride, int rows, int heads, int per_group, int dv,
                           float lambda, float eps, float factor, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || per_group <= 0 || heads % per_group || dv <= 0) GB_REFUSE("diff_combine: %d heads in groups of %d, values of %d", heads, per_group, dv);
    const int64_t units = (int64_t)rows * heads;
    const unsigned blocks = (unsigned)((units + 3) / 4);
    if (dtype == GB_F32)
        diff_combine_kernel<float><<<blocks, 128, 0, stream>>>((const float*)ctx, ctx_stride, (float*)out, out_stride, rows, heads, per_group, dv, lambda, eps, factor);
    else if (dtype == GB_BF16)
        diff_combine_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>((const __nv_bfloat16*)ctx, ctx_stride, (__nv_bfloat16*)out, out_stride, rows, heads,
                                                                      per_group, dv, lambda, eps, factor);
    else
        GB_REFUSE("diff_combine: unknown dtype %d", dtype);
    GB_CHECK_LAUNCH("diff_combine");
    return 0;
}

GB_API int gb_add_rows_gated(float* out, const float* y, const float* z, int64_t z_stride, int rows, int n, cudaStream_t stream) {
    if (rows <= 0) return 0;
    add_rows_gated_kernel<<<rows, 256, 0, stream>>>(out, y, z, z_stride, n);
    GB_CHECK_LAUNCH("add_rows_gated");
    return 0;
}

GB_API int gb_latent_prep(const void* lat, int64_t lat_stride, void* cq, const float* q_w, const float* kv_w, float eps, const float* cos_t,
                          const float* sin_t, int table_positions, const int* row_pos, const int* row_seq, const int* seq_slot,
                          const int* block_table, int bt_stride, void* k_plane, int write_kv, int rows, int q_rank, int kv_rank, int rot, int pages,
                          int max_slots, int dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (q_rank <= 0 || kv_rank <= 0 || rot < 0 || (rot & 1)) GB_REFUSE("latent_prep: latents of %d and %d, %d rotated channels", q_rank, kv_rank, rot);
    if (rot > 0 && (!cos_t || !sin_t)) GB_REFUSE("latent_prep: %d rotated channels without an angle table", rot);
    LatentPrepArgs p{lat, lat_stride, cq, q_w, kv_w, eps, cos_t, sin_t, table_positions, row_pos, row_seq, seq_slot, block_table, bt_stride,
                     k_plane, write_kv, rows, q_rank, kv_rank, rot, pages, max_slots};
    if (dtype == GB_F32)
        latent_prep_kernel<float><<<rows, 256, 0, stream>>>(p);
    else if (dtype == GB_BF16)
        latent_prep_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>(p);
    else
        GB_REFUSE("latent_prep: unknown dtype %d", dtype);
    GB_CHECK_LAUNCH("latent_prep");
    return 0;
}

GB_API int gb_latent_q_rot(const void* q, int64_t q_stride, void* out, int64_t out_stride, int rows, int heads, int d, int rot, int out_head,
                           const float* cos_t, const float* sin_t, int table_positions, const int* row_pos, int dtype, cudaStream_t stream) {
    if (rows <= 0 || rot <= 0) return 0;
    if ((rot & 1) || out_head < rot) GB_REFUSE("latent_q_rot: %d rotated channels into heads of %d", rot, out_head);
    if (dtype == GB_F32)
        latent_q_rot_kernel<float><<<rows, 128, 0, stream>>>((const float*)q, q_stride, (float*)out, out_stride, heads, d, rot, out_head, cos_t, sin_t,
                                                             table_positions, row_pos);
    else if (dtype == GB_BF16)
        latent_q_rot_kernel<__nv_bfloat16><<<rows, 128, 0, stream>>>((const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, heads, d, rot,
                                                                     out_head, cos_t, sin_t, table_positions, row_pos);
    else
        GB_REFUSE("latent_q_rot: unknown dtype %d", dtype);
    GB_CHECK_LAUNCH("latent_q_rot");
    return 0;
}

GB_API int gb_head_gemm(const void* a, int64_t a_row_stride, int64_t a_head_stride, const void* w, void* out, int64_t o_row_stride,
                        int64_t o_head_stride, int rows, int heads, int K, int N, int dtype, int w_dtype, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || K <= 0 || N <= 0) GB_REFUSE("head_gemm: %d heads of %d x %d", heads, K, N);
    const size_t smem = ((size_t)HG_ROWS * K + (size_t)HG_WARPS * HG_ROWS * HG_COLS) * sizeof(float);
    if (smem > 96 * 1024) GB_REFUSE("head_gemm: rows of %d exceed what one CTA stages", K);
    dim3 grid((N + HG_COLS - 1) / HG_COLS, heads, (rows + HG_ROWS - 1) / HG_ROWS);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("head_gemm: %d heads, %d rows exceed one launch", heads, rows);
    if (dtype == GB_F32 && w_dtype == GB_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(head_gemm_kernel<float, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        head_gemm_kernel<float, float><<<grid, 32 * HG_WARPS, smem, stream>>>((const float*)a, a_row_stride, a_head_stride, (const float*)w, (float*)out,
                                                                             o_row_stride, o_head_stride, rows, K, N);
    } else if (dtype == GB_BF16 && w_dtype == GB_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(head_gemm_kernel<__nv_bfloat16, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        head_gemm_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 32 * HG_WARPS, smem, stream>>>((const __nv_bfloat16*)a, a_row_stride, a_head_stride,
                                                                                             (const __nv_bfloat16*)w, (__nv_bfloat16*)out, o_row_stride,
                                                                                             o_head_stride, rows, K, N);
    } else {
        GB_REFUSE("head_gemm: activations of dtype %d with weights of dtype %d", dtype, w_dtype);
    }
    GB_CHECK_LAUNCH("head_gemm");
    return 0;
}

// Whether the tensor-core form takes these operands: 16-byte aligned rows of a and W, even strides of the output.
GB_API int gb_head_gemm_mma_accepts(const void* a, int64_t a_row_stride, int64_t a_head_stride, const void* w, const void* out, int64_t o_row_stride,
                                    int64_t o_head_stride, int K, int N) {
    return !(K & 7) && !(a_row_stride & 7) && !(a_head_stride & 7) && !((uintptr_t)a & 15) && !((uintptr_t)w & 15) && !(o_row_stride & 1) &&
           !(o_head_stride & 1) && !((uintptr_t)out & 3) && K > 0 && N > 0;
}

// out[r, h, :] = a[r, h, :] W_h^T with W as [heads][N][K], bfloat16, on the tensor cores.
GB_API int gb_head_gemm_mma(const void* a, int64_t a_row_stride, int64_t a_head_stride, const void* w, void* out, int64_t o_row_stride,
                            int64_t o_head_stride, int rows, int heads, int K, int N, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || !gb_head_gemm_mma_accepts(a, a_row_stride, a_head_stride, w, out, o_row_stride, o_head_stride, K, N))
        GB_REFUSE("head_gemm_mma: %d heads of %d x %d with these strides are not what this kernel takes", heads, K, N);
    dim3 grid((N + HM_T - 1) / HM_T, heads, (rows + HM_T - 1) / HM_T);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("head_gemm_mma: %d heads, %d rows exceed one launch", heads, rows);
    head_gemm_mma_kernel<<<grid, 128, 0, stream>>>((const __nv_bfloat16*)a, a_row_stride, a_head_stride, (const __nv_bfloat16*)w, (__nv_bfloat16*)out,
                                                   o_row_stride, o_head_stride, rows, K, N);
    GB_CHECK_LAUNCH("head_gemm_mma");
    return 0;
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_postnorm)
