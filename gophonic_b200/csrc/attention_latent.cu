// Attention over a cache of latents on the tensor cores (bf16 mma.sync): ONE key head that every query head reads, whose
// first dv channels are also the values (AttnParamsX.v_row_stride == d: the value plane is a view of the key plane), with
// key heads much wider than a usual head (a latent of 512 and 64 rotated channels).  Prompts, portions and single tokens.
//
// A CTA owns 16 or 32 rows (one or two groups of 16, four warps a group), which are (query position, head) pairs of one
// sequence, and walks the cache pages its rows can see, one page of 64 keys a step, double-buffered with cp.async; a page
// is staged ONCE, serves as keys and as values, and is shared by the row groups.  The work of a step is dealt twice inside
// a group: for the scores each warp takes 16 of the 64 keys (Q K^T over all d channels, in four independent chains of
// products so that no product waits for the one before it); after the row maxima have met in shared memory every warp
// writes its probabilities (bf16) into the group's 16 x 64 tile; for the second product each warp takes a quarter of the
// dv value columns (P V over all 64 keys), so a warp's float32 accumulators are 16 x dv / 4.  Scores, maxima, sums and accumulators are float32; masks (causal, window, blocks of
// positions) come from absolute positions and tiles start at multiples of 64, so a row's result does not depend on how its
// sequence was cut into steps or on what else the batch holds.  Single-token steps may cut the keys into splits that a
// merge kernel joins (the same scratch layout as the other attention kernels).
#include "api.h"
#include "common.cuh"
#include "mma.cuh"

#include <math.h>

int gb_attention_merge_launch(const float* scratch, void* out, int dtype, int64_t out_row_stride, const int* seq_q_start, int nseq, int heads,
                              int d, int num_splits, int sink, const float* sinks, cudaStream_t stream);

namespace {

using bf16 = __nv_bfloat16;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
constexpr int GB_KEYS = 64;      // keys a cache page holds
constexpr int PAGE_LIST = 512;     // tiles whose pages a CTA looks up ahead (32768 keys); beyond them, tile by tile

// NT: value columns a warp owns, in tiles of 8; RG: groups of 16 rows a CTA holds; WG: warps a group has (4 or 8), which
// split a page's 64 keys for the scores and the dv = 8 * NT * WG value columns for the second product
// LKT: keys a step stages (a page, or half a page); STAGES: steps staged at a time.
template <int NT, int RG, int WG, int LKT, int STAGES>
__global__ void __launch_bounds__(32 * WG * RG) attn_latent_mma_kernel(AttnParamsX p) {
    constexpr int LROWS = 16 * RG, THREADS = 32 * WG * RG, LPS = LKT + 8;
    constexpr int KW = LKT / WG, J = KW / 8;      // keys a warp scores, in tiles of 8
    const int d = p.d, SD = d + 8, KS = d / 16;
    constexpr int DV = 8 * NT * WG;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);          // [16][SD]
    bf16* Ks = Qs + LROWS * SD;                            // [STAGES][LKT][SD]
    bf16* Ps_all = Ks + STAGES * LKT * SD;                 // [RG][16][LKT + 8]
    float* red_all = reinterpret_cast<float*>(Ps_all + LROWS * LPS);   // [RG][WG warps][16 rows]
    __shared__ int page_list[PAGE_LIST];

    const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int rg = (tid >> 5) / WG, warp = (tid >> 5) % WG;      // row group, and the warp's place inside it
    bf16* Ps = Ps_all + rg * 16 * LPS;
    float* red = red_all + rg * (16 * WG);
    const bf16* Qg = Qs + rg * 16 * SD;
    const int H = p.heads;
    const int HC = H < LROWS ? H : LROWS;       // heads a CTA holds
    const int QT = LROWS / HC;                  // query positions a CTA holds
    const int seq = blockIdx.z / p.num_splits, split = blockIdx.z % p.num_splits;
    const int h0 = blockIdx.y * HC;
    const int q_len = p.seq_q_len[seq], kv_len = p.seq_kv_len[seq];
    const int q0 = blockIdx.x * QT;
    if (q0 >= q_len) return;
    const int past = kv_len - q_len;
    const int q_start = p.seq_q_start[seq];
    const int* bt = block_table_row(p.block_table, p.bt_stride, p.seq_slot[seq], p.max_slots);

    // this thread's two rows of the tile: g and g + 8
    int rpos[2], rq[2], rhead[2];
    bool rok[2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int r = rg * 16 + g + 8 * e;
        const int qi = r / HC, hd = h0 + r % HC;
        rok[e] = qi < QT && q0 + qi < q_len && hd < H;
        rq[e] = q0 + qi;
        rhead[e] = hd;
        rpos[e] = past + q0 + qi;
    }
    const int last_q = (q0 + QT < q_len ? q0 + QT : q_len) - 1;
    const int hi_pos = past + last_q;
    int lo_pos = 0;
    if (p.window > 0) {
        lo_pos = past + q0 - p.window + 1;
        if (lo_pos < 0) lo_pos = 0;
    }
    if (p.chunk > 0) {
        const int b = (past + q0) - (past + q0) % p.chunk;
        if (b > lo_pos) lo_pos = b;
    }
    const int t_lo = lo_pos / LKT, t_hi = hi_pos / LKT + 1;
    const int n_tiles = t_hi - t_lo;
    const int per = (n_tiles + p.num_splits - 1) / p.num_splits;
    const int my_lo = t_lo + split * per;
    const int my_hi = my_lo + per < t_hi ? my_lo + per : t_hi;
    const int n = my_hi > my_lo ? my_hi - my_lo : 0;

    const int CH = d / 8;     // 16-byte pieces of a row
    // the physical pages of this CTA's tiles, looked up once: a tile's copies are then issued without waiting for the block table
    for (int i = tid; i < n && i < PAGE_LIST; i += THREADS) page_list[i] = (int)page_of(bt, (my_lo + i) * LKT, p.bt_stride, p.pages);
    __syncthreads();
    auto load_tile = [&](int i) {
        const int64_t page = i < PAGE_LIST ? page_list[i] : page_of(bt, (my_lo + i) * LKT, p.bt_stride, p.pages);
        const bf16* src = (const bf16*)p.k_plane + (page * GB_KEYS + ((my_lo + i) * LKT) % GB_KEYS) * (int64_t)d;
        bf16* st = Ks + (i % STAGES) * LKT * SD;
        // a warp copies whole rows, its lanes the row's 16-byte pieces
        for (int key = tid >> 5; key < LKT; key += THREADS / 32)
            for (int c = lane; c < CH; c += 32) cp_async16(st + key * SD + c * 8, src + (int64_t)key * d + c * 8, 16);
    };
    {
        for (int idx = tid; idx < LROWS * CH; idx += THREADS) {
            const int r = idx / CH, c = idx - r * CH;
            const int qi = r / HC, hd = h0 + r % HC;
            const bool ok = qi < QT && q0 + qi < q_len && hd < H;
            const bf16* src = (const bf16*)p.q + (ok ? (int64_t)(q_start + q0 + qi) * p.q_row_stride + (int64_t)hd * d + c * 8 : 0);
            cp_async16(Qs + r * SD + c * 8, src, ok ? 16 : 0);
        }
        if (n > 0) load_tile(0);
        cp_async_commit();
#pragma unroll
        for (int u = 1; u < STAGES - 1; u++) {
            if (u < n) load_tile(u);
            cp_async_commit();
        }
    }

    const float sc = p.scale * LOG2E;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[j][e] = 0.f;

    for (int i = 0; i < n; i++) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                       // tile i has landed; everyone is done with tile i - 1, the probabilities and the maxima
        if (i + STAGES - 1 < n) load_tile(i + STAGES - 1);
        cp_async_commit();
        const bf16* kt = Ks + (i % STAGES) * LKT * SD;
        const int t = my_lo + i;
        // scores of this warp's keys: four chains of products over the channels (steps ks, ks + 1, ks + 2, ks + 3), added up
        // in a fixed order
        float s[J][4], part[3][J][4];
#pragma unroll
        for (int j = 0; j < J; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[j][e] = part[0][j][e] = part[1][j][e] = part[2][j][e] = 0.f;
        const bf16* qa = Qg + ((lane & 7) + ((lane >> 3) & 1) * 8) * SD + (lane >> 4) * 8;
        // 16 keys: four 8 x 8 pieces (keys 0-7 and 8-15, channels 0-7 and 8-15); 8 keys: two pieces, addressed by lanes 0-15
        const bf16* kb = J == 2 ? kt + (warp * KW + (lane & 7) + (lane >> 4) * 8) * SD + ((lane >> 3) & 1) * 8
                                : kt + (warp * KW + (lane & 7)) * SD + ((lane >> 3) & 1) * 8;
        // the operands of a step: a query fragment and the fragment(s) of this warp's keys
        auto fetch = [&](uint32_t (&a)[4], uint32_t (&b)[4], int step) {
            ldmatrix_x4(a, qa + step * 16);
            if (J == 2) {
                ldmatrix_x4(b, kb + step * 16);
            } else {
                uint32_t b2[2];
                ldmatrix_x2(b2, kb + step * 16);
                b[0] = b2[0];
                b[1] = b2[1];
            }
        };
        auto products = [&](float (&acc)[J][4], const uint32_t (&a)[4], const uint32_t (&b)[4]) {
            mma_bf16_16816(acc[0], a[0], a[1], a[2], a[3], b[0], b[1]);
            if (J == 2) mma_bf16_16816(acc[J - 1], a[0], a[1], a[2], a[3], b[2], b[3]);
        };
        int ks = 0;
        for (; ks + 3 < KS; ks += 4) {
            // all eight fragments are asked for before the first product needs one
            uint32_t a[4][4], b[4][4];
#pragma unroll
            for (int u = 0; u < 4; u++) fetch(a[u], b[u], ks + u);
            products(s, a[0], b[0]);
            products(part[0], a[1], b[1]);
            products(part[1], a[2], b[2]);
            products(part[2], a[3], b[3]);
        }
        for (; ks < KS; ks++) {
            uint32_t a[4], b[4];
            fetch(a, b, ks);
            products(s, a, b);
        }
#pragma unroll
        for (int j = 0; j < J; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[j][e] = (s[j][e] + part[0][j][e]) + (part[1][j][e] + part[2][j][e]);
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < J; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = t * LKT + warp * KW + j * 8 + t4 * 2 + (e & 1);
                const int w = e >> 1;
                const int pos = rpos[w];
                const bool ok = rok[w] && key <= pos && (p.window <= 0 || key > pos - p.window) && (p.chunk <= 0 || key >= pos - pos % p.chunk);
                const float v = ok ? s[j][e] * sc : -INFINITY;
                s[j][e] = v;
                if (w) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if (t4 == 0) {
            red[warp * 16 + g] = mx0;
            red[warp * 16 + g + 8] = mx1;
        }
        __syncthreads();
        mx0 = m0;
        mx1 = m1;
#pragma unroll
        for (int ww = 0; ww < WG; ww++) {
            mx0 = fmaxf(mx0, red[ww * 16 + g]);
            mx1 = fmaxf(mx1, red[ww * 16 + g + 8]);
        }
        const float base0 = mx0 == -INFINITY ? 0.f : mx0, base1 = mx1 == -INFINITY ? 0.f : mx1;
        const float c0 = exp2f(m0 - base0), c1 = exp2f(m1 - base1);
        m0 = mx0;
        m1 = mx1;
        l0 *= c0;
        l1 *= c1;
#pragma unroll
        for (int j = 0; j < NT; j++) {
            o[j][0] *= c0;
            o[j][1] *= c0;
            o[j][2] *= c1;
            o[j][3] *= c1;
        }
#pragma unroll
        for (int j = 0; j < J; j++) {
            const float p0 = exp2f(s[j][0] - base0), p1 = exp2f(s[j][1] - base0), p2 = exp2f(s[j][2] - base1), p3 = exp2f(s[j][3] - base1);
            l0 += p0 + p1;
            l1 += p2 + p3;
            const int col = warp * KW + j * 8 + t4 * 2;
            *reinterpret_cast<uint32_t*>(Ps + g * LPS + col) = pack_bf16(p0, p1);
            *reinterpret_cast<uint32_t*>(Ps + (g + 8) * LPS + col) = pack_bf16(p2, p3);
        }
        __syncthreads();
        // this warp's value columns over all 64 keys: the values are the first channels of the keys
        {
            // the value fragments are asked for one pair of column tiles ahead of the products that take them
            const bf16* vb = kt + ((lane & 7) + ((lane >> 3) & 1) * 8) * SD + warp * (NT * 8) + (lane >> 4) * 8;
            constexpr int PAIRS = NT / 2, STEPS = (LKT / 16) * PAIRS;
            uint32_t pa[4], b[2][4];
            ldmatrix_x4(pa, Ps + ((lane & 7) + ((lane >> 3) & 1) * 8) * LPS + (lane >> 4) * 8);
            ldmatrix_x4_trans(b[0], vb);
#pragma unroll
            for (int st = 0; st < STEPS; st++) {
                const int kk = st / PAIRS, c = st % PAIRS;
                uint32_t pn[4];
                if (st + 1 < STEPS) {
                    const int kn = (st + 1) / PAIRS, cn = (st + 1) % PAIRS;
                    ldmatrix_x4_trans(b[(st + 1) & 1], vb + kn * 16 * SD + cn * 16);
                    if (cn == 0) ldmatrix_x4(pn, Ps + ((lane & 7) + ((lane >> 3) & 1) * 8) * LPS + kn * 16 + (lane >> 4) * 8);
                }
                mma_bf16_16816(o[c * 2], pa[0], pa[1], pa[2], pa[3], b[st & 1][0], b[st & 1][1]);
                mma_bf16_16816(o[c * 2 + 1], pa[0], pa[1], pa[2], pa[3], b[st & 1][2], b[st & 1][3]);
                if (st + 1 < STEPS && (st + 1) % PAIRS == 0) {
#pragma unroll
                    for (int e = 0; e < 4; e++) pa[e] = pn[e];
                }
                (void)kk;
            }
        }
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();
    if (t4 == 0) {
        red[warp * 16 + g] = l0;
        red[warp * 16 + g + 8] = l1;
    }
    __syncthreads();
    float L0 = 0.f, L1 = 0.f;
#pragma unroll
    for (int ww = 0; ww < WG; ww++) {      // in warp order
        L0 += red[ww * 16 + g];
        L1 += red[ww * 16 + g + 8];
    }
#pragma unroll
    for (int e = 0; e < 2; e++) {
        if (!rok[e]) continue;
        const float L = e ? L1 : L0, M = e ? m1 : m0;
        if (p.num_splits == 1) {
            bf16* op = (bf16*)p.out + (int64_t)(q_start + rq[e]) * p.out_row_stride + (int64_t)rhead[e] * DV + warp * (NT * 8) + t4 * 2;
            const float inv = 1.f / L;
#pragma unroll
            for (int j = 0; j < NT; j++) *reinterpret_cast<uint32_t*>(op + j * 8) = pack_bf16(o[j][2 * e] * inv, o[j][2 * e + 1] * inv);
        } else {
            float* sp = p.scratch + (((int64_t)seq * p.heads + rhead[e]) * p.num_splits + split) * (DV + 2);
            if (warp == 0 && t4 == 0) {
                sp[0] = M == -INFINITY ? -INFINITY : M * LN2;     // natural-log units, as the merge kernel expects
                sp[1] = L;
            }
#pragma unroll
            for (int j = 0; j < NT; j++) {
                sp[2 + warp * (NT * 8) + j * 8 + t4 * 2] = o[j][2 * e];
                sp[2 + warp * (NT * 8) + j * 8 + t4 * 2 + 1] = o[j][2 * e + 1];
            }
        }
    }
}

template <int NT, int RG, int WG, int LKT, int STAGES>
int launch_latent(const AttnParamsX& p, cudaStream_t stream) {
    constexpr int LPS = LKT + 8;
    constexpr int LROWS = 16 * RG;
    const int HC = p.heads < LROWS ? p.heads : LROWS, QT = LROWS / HC;
    dim3 grid(ceil_div(p.max_q_len, QT), ceil_div(p.heads, HC), p.nseq * p.num_splits);
    if (grid.y > 65535 || grid.z > 65535) GB_REFUSE("attention_latent: grid (%u, %u, %u) exceeds one launch", grid.x, grid.y, grid.z);
    const size_t smem = ((size_t)(LROWS + STAGES * LKT) * (p.d + 8) + (size_t)LROWS * LPS) * sizeof(bf16) + WG * LROWS * sizeof(float);
    if (smem > 220 * 1024 - PAGE_LIST * sizeof(int)) GB_REFUSE("attention_latent: keys of %d channels exceed what one CTA stages", p.d);
    static size_t configured = 0;      // always opted in: the static page list counts towards the 48 KB a kernel has without
    if (configured == 0) {
        cudaError_t e = cudaFuncSetAttribute(attn_latent_mma_kernel<NT, RG, WG, LKT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) GB_REFUSE("attention_latent: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = 220 * 1024;
    }
    attn_latent_mma_kernel<NT, RG, WG, LKT, STAGES><<<grid, 32 * WG * RG, smem, stream>>>(p);
    GB_CHECK_LAUNCH("attention_latent");
    if (p.num_splits > 1) return gb_attention_merge_launch(p.scratch, p.out, GB_BF16, p.out_row_stride, p.seq_q_start, p.nseq, p.heads, 8 * NT * WG, p.num_splits, 0, nullptr, stream);
    return 0;
}

}  // namespace

// Whether the kernel takes this geometry: bf16, one key head whose first dv channels are the values, dv 64 / 128 / 256 / 512,
// key size a multiple of 16 up to 640, 16-byte aligned rows.
GB_API int gb_attention_latent_accepts(const AttnParamsX* p, int dtype) {
    const int dv = p->dv ? p->dv : p->d;
    return dtype == GB_BF16 && p->kv_heads == 1 && p->v_share <= 1 && p->v_row_stride == p->d && p->v_plane == p->k_plane && !(p->d & 15) &&
           p->d <= 640 && (dv == 64 || dv == 128 || dv == 256 || dv == 512) && dv <= p->d && !p->sink && !p->keep_first &&
           !((uintptr_t)p->q & 15) && !(p->q_row_stride & 7) && !((uintptr_t)p->k_plane & 15) && !((uintptr_t)p->out & 3) && !(p->out_row_stride & 1);
}

GB_API int gb_attention_latent_mma(const AttnParamsX* pp, cudaStream_t stream) {
    AttnParamsX p = *pp;
    if (p.nseq <= 0 || p.max_q_len <= 0) return 0;
    if (!gb_attention_latent_accepts(&p, GB_BF16)) GB_REFUSE("attention_latent: %d heads over %d key heads of %d with values of %d are not what this kernel takes", p.heads, p.kv_heads, p.d, p.dv);
    if (p.num_splits < 1 || (p.num_splits > 1 && (p.max_q_len != 1 || !p.scratch))) GB_REFUSE("attention_latent: %d key splits", p.num_splits);
    if (p.window < 0 || p.chunk < 0) GB_REFUSE("attention_latent: window %d, blocks of %d", p.window, p.chunk);
    // two groups of rows share a staged page where a sequence brings that many (query position, head) pairs; a single group
    // (single tokens of up to 16 heads) gets eight warps, two a scheduler, where its value heads are wide enough to deal out.
    // (Half pages staged four deep, <.., 1, 4, 32, 4>, measured slower for single tokens: 65 against 54 us for 64 sequences of
    // 16 heads over 1024 keys of 576: the step is bound by its products, not by the copies.)
    const bool two = (int64_t)p.max_q_len * p.heads > 16;
    switch ((p.dv ? p.dv : p.d) / 64) {
        case 1: return two ? launch_latent<2, 2, 4, 64, 2>(p, stream) : launch_latent<2, 1, 4, 64, 2>(p, stream);
        case 2: return two ? launch_latent<4, 2, 4, 64, 2>(p, stream) : launch_latent<2, 1, 8, 64, 2>(p, stream);
        case 4: return two ? launch_latent<8, 2, 4, 64, 2>(p, stream) : launch_latent<4, 1, 8, 64, 2>(p, stream);
        default: return two ? launch_latent<16, 2, 4, 64, 2>(p, stream) : launch_latent<8, 1, 8, 64, 2>(p, stream);
    }
}

// the checked build's record of the first index this file's kernels found out of bounds
GB_CHECK_READER(gb_checked_status_attention_latent)
