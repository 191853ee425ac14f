// Attention over a cache of latents: every token keeps one vector [c ; r] -- a normed latent c of C values from
// which every head's unrotated key and value are linear maps (k_h = Wuk_h c, v_h = Wuv_h c), and one rotated
// key part r of R values that all heads share.  A query head brings D unrotated and R rotated values.  The score
//     s = (q_plain . Wuk_h c + q_rot . r) * scale
// is computed without ever making the keys: q_plain is carried through the key map once per query,
//     qc = Wuk_h^T q_plain   (C values),   s = (qc . c + q_rot . r) * scale,
// and the values are made after the weighted sum: o_h = Wuv_h (sum_t p_t c_t).  Both maps cost D x C and V x C
// multiply-adds per (row, head), whatever the number of keys, and the cache row is read as it lies.
//
// `llmx_latent_write`: per row of the stacked down projections, the query latent's RMS norm (for the product that
// makes the queries), and the key/value latent's RMS norm and the rotated key part, stored to the row's cache slot.
// `llmx_latent_attention`: one block per (row, head): rotation of the query's rotated part, the key map, an online
// softmax over the row's keys lo..p (lo = max(0, p - window + 1), window <= 0: all), warps taking every fourth key
// in increasing order and merged in warp order, then the value map.  Scores, weights and sums are 32-bit.
//
// Rotation: pair i < dims / 2 of the rotated part turns by angle p * f_i, the frequencies f_i given as a float table
// (base^(-2i / dims), or whatever blend of scaled frequencies the design asks for); the angle is the float product, its
// cosine and sine the precise functions, both times `rot_mag` (a design's factor on rotated parts; 1 for none).  The
// pair's members are neighbours (2i, 2i + 1), or with `rot_halves` the two halves' values (i, i + dims / 2).
#include "common.cuh"
#include "attn_common.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;

// Where the two members of rotation pair i lie in a part whose first 2 * pairs values are rotated.
__device__ __forceinline__ int pair_first(int i, int pairs, int halves) { return halves ? i : 2 * i; }
__device__ __forceinline__ int pair_second(int i, int pairs, int halves) { return halves ? i + pairs : 2 * i + 1; }

// A row of the stacked down projections is [query latent (Q) | key/value latent (C) | rotated key part (R)].  One block
// per row: the query latent's RMS norm (weight wq) goes to `cq` in the type the next product reads; the key/value
// latent's RMS norm (weight w) and the rotated part go to the row's cache slot (skipped when the slot is negative).
template <typename KVT, typename QT>
__global__ void __launch_bounds__(128)
latent_write_kernel(const float* __restrict__ down, int stride, int Q, const float* __restrict__ wq, QT* __restrict__ cq,
                    const float* __restrict__ w, float eps, const float* __restrict__ freq, int rot_pairs, int rot_halves,
                    float rot_mag, const int* __restrict__ positions, const int* __restrict__ slots, KVT* __restrict__ cache,
                    int C, int R) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int row = blockIdx.x;
    const float* qsrc = down + (size_t)row * stride;
    if (Q > 0) {
        float s = 0.0f;
        for (int i = threadIdx.x; i < Q; i += blockDim.x) s = fmaf(qsrc[i], qsrc[i], s);
        const float rr = 1.0f / sqrtf(block_sum(s, scratch) / (float)Q + eps);
        for (int i = threadIdx.x; i < Q; i += blockDim.x) cq[(size_t)row * Q + i] = from_float<QT>(qsrc[i] * (rr * wq[i]));
    }
    const int slot = slots[row];
    if (slot < 0) return;
    const float* src = qsrc + Q;
    KVT* dst = cache + (size_t)slot * (C + R);
    float s = 0.0f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) s = fmaf(src[i], src[i], s);
    const float rr = 1.0f / sqrtf(block_sum(s, scratch) / (float)C + eps);
    for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = from_float<KVT>(src[i] * rr * w[i]);
    const float p = (float)positions[row];
    for (int i = threadIdx.x; i < rot_pairs; i += blockDim.x) {
        const int ia = C + pair_first(i, rot_pairs, rot_halves), ib = C + pair_second(i, rot_pairs, rot_halves);
        const float a = src[ia], b = src[ib];
        float sn, cs;
        sincosf(p * freq[i], &sn, &cs);
        sn *= rot_mag;
        cs *= rot_mag;
        dst[ia] = from_float<KVT>(a * cs - b * sn);
        dst[ib] = from_float<KVT>(b * cs + a * sn);
    }
    for (int i = 2 * rot_pairs + threadIdx.x; i < R; i += blockDim.x) dst[C + i] = from_float<KVT>(src[C + i]);
}

// PL: values of a cache row a lane holds (C + R <= 32 * PL).
template <typename WT, typename KVT, int PL>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_kernel(const float* __restrict__ q, int q_stride, const KVT* __restrict__ cache,
                        const WT* __restrict__ w_uk, const WT* __restrict__ w_uv, WT* __restrict__ out,
                        const float* __restrict__ freq, int rot_pairs, int rot_halves, float rot_mag,
                        const int* __restrict__ row_request,
                        const int* __restrict__ positions, const int* __restrict__ block_tables, int table_stride,
                        int heads, int D, int R, int V, int C, int page_size, int window, float scale) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int W = C + R;
    float* qraw = smem;                       // D + R: the query head, its rotated part turned
    float* qk = qraw + D + R;                 // W: [Wuk^T q_plain ; q_rot] * scale
    float* part = qk + W;                     // WARPS * (C + 2)
    const int row = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[row];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_tables + (size_t)row_request[row] * table_stride;

    const float* qrow = q + (size_t)row * q_stride + (size_t)h * (D + R);
    for (int i = threadIdx.x; i < D + R; i += blockDim.x) qraw[i] = qrow[i];
    __syncthreads();
    for (int i = threadIdx.x; i < rot_pairs; i += blockDim.x) {
        const int ia = pair_first(i, rot_pairs, rot_halves), ib = pair_second(i, rot_pairs, rot_halves);
        const float a = qraw[D + ia], b = qraw[D + ib];
        float sn, cs;
        sincosf((float)pos * freq[i], &sn, &cs);
        sn *= rot_mag;
        cs *= rot_mag;
        qk[C + ia] = (a * cs - b * sn) * scale;
        qk[C + ib] = (b * cs + a * sn) * scale;
    }
    for (int i = 2 * rot_pairs + threadIdx.x; i < R; i += blockDim.x) qk[C + i] = qraw[D + i] * scale;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const WT* col = w_uk + (size_t)h * D * C + c;
        float s = 0.0f;
        for (int d = 0; d < D; ++d) s = fmaf(qraw[d], to_float(col[(size_t)d * C]), s);
        qk[c] = s * scale;
    }
    __syncthreads();

    float qv[PL], acc[PL];
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int e = lane + 32 * i;
        qv[i] = e < W ? qk[e] : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int t = lo + warp; t <= pos; t += WARPS) {
        const KVT* kp = cache + ((size_t)table[t / page_size] * page_size + t % page_size) * W;
        float kv[PL];
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < PL; ++i) {
            const int e = lane + 32 * i;
            kv[i] = e < W ? to_float(kp[e]) : 0.0f;
            s = fmaf(qv[i], kv[i], s);
        }
        s = warp_sum(s);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        const float e = expf(s - m_new);
        l = l * corr + e;
#pragma unroll
        for (int i = 0; i < PL; ++i) acc[i] = fmaf(e, kv[i], acc[i] * corr);
        m = m_new;
    }
    float* mine = part + warp * (C + 2);
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int e = lane + 32 * i;
        if (e < C) mine[e] = acc[i];
    }
    if (lane == 0) {
        mine[C] = m;
        mine[C + 1] = l;
    }
    __syncthreads();
    // The four partial states merged in warp order; the weighted sum of latents ends in part[0 .. C).
    float mm = -INFINITY;
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, part[w * (C + 2) + C]);
    float f[WARPS], ll = 0.0f;
    for (int w = 0; w < WARPS; ++w) {
        const float mw = part[w * (C + 2) + C];
        f[w] = mw == -INFINITY ? 0.0f : expf(mw - mm);
        ll += part[w * (C + 2) + C + 1] * f[w];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float o = 0.0f;
        for (int w = 0; w < WARPS; ++w) o += part[w * (C + 2) + c] * f[w];
        qk[c] = o / ll;                        // qk is free now: the merged latent
    }
    __syncthreads();
    WT* orow = out + ((size_t)row * heads + h) * V;
    for (int v = warp; v < V; v += WARPS) {
        const WT* wr = w_uv + ((size_t)h * V + v) * C;
        float s = 0.0f;
        for (int c = lane; c < C; c += 32) s = fmaf(to_float(wr[c]), qk[c], s);
        s = warp_sum(s);
        if (lane == 0) orow[v] = from_float<WT>(s);
    }
}

template <typename WT, typename KVT>
int launch_attention(int pl, dim3 grid, size_t smem, cudaStream_t stream, const float* q, int q_stride, const void* cache,
                     const void* w_uk, const void* w_uv, void* out, const float* freq, int rot_pairs, int rot_halves,
                     float rot_mag, const int* row_request,
                     const int* positions, const int* block_tables, int table_stride, int heads, int D, int R, int V, int C,
                     int page_size, int window, float scale) {
#define LLMX_LAT(P)                                                                                                       \
    do {                                                                                                                  \
        if (smem > 48 * 1024)                                                                                             \
            cudaFuncSetAttribute(latent_attention_kernel<WT, KVT, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_kernel(latent_attention_kernel<WT, KVT, P>, grid, dim3(WARPS * 32), smem, stream, q, q_stride,             \
                      (const KVT*)cache, (const WT*)w_uk, (const WT*)w_uv, (WT*)out, freq, rot_pairs, rot_halves, rot_mag, row_request, \
                      positions, block_tables, table_stride, heads, D, R, V, C, page_size, window, scale);               \
    } while (0)
    if (pl <= 2) LLMX_LAT(2);
    else if (pl <= 4) LLMX_LAT(4);
    else if (pl <= 8) LLMX_LAT(8);
    else if (pl <= 12) LLMX_LAT(12);
    else if (pl <= 20) LLMX_LAT(20);
    else if (pl <= 32) LLMX_LAT(32);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_LAT
    return launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
// The tiled form: three kernels.
//   latent_query   one block per (row, head): rotation, the key map, the scale -> qk [rows, heads, C + R] floats
//   latent_scores  one block per (tile of rows, group of heads, range of keys): 16 (row, head) pairs, two to a warp,
//                  share every key: a tile of keys is copied from the pages into shared memory once (the next tile's
//                  copy in flight in registers meanwhile) and each warp walks it for its two pairs, a lane holding
//                  neighbouring pairs of a key's values; partial (sum of weighted latents, maximum, sum) per range
//   latent_merge   one block per (row, head): the ranges merged in order, then the value map
// Prompt portions fill the grid with row tiles; decoding rows, few and with long histories, with key ranges.
// ---------------------------------------------------------------------------------------------------------------
// ROWS_Q: rows a block of the query or the merge kernel holds: a map's weights are read once for them (8 when a step has
// many rows; 1 when it has few, so that the blocks are many).
template <typename WT, int ROWS_Q>
__global__ void __launch_bounds__(128)
latent_query_kernel(const float* __restrict__ q, int q_stride, const WT* __restrict__ w_uk, float* __restrict__ qk,
                    const float* __restrict__ freq, int rot_pairs, int rot_halves, float rot_mag,
                    const int* __restrict__ positions, int rows, int heads, int D, int R, int C, float scale) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float qraw[];            // ROWS_Q * (D + R)
    const int r0 = blockIdx.x * ROWS_Q, h = blockIdx.y;
    const int n = min(ROWS_Q, rows - r0);
    const int DR = D + R;
    for (int i = threadIdx.x; i < ROWS_Q * DR; i += blockDim.x) {
        const int r = i / DR;
        qraw[i] = r < n ? q[(size_t)(r0 + r) * q_stride + (size_t)h * DR + i % DR] : 0.0f;
    }
    __syncthreads();
    if (blockIdx.z == 0) {
        for (int i = threadIdx.x; i < n * rot_pairs; i += blockDim.x) {
            const int r = i / rot_pairs, k = i % rot_pairs;
            const int ia = pair_first(k, rot_pairs, rot_halves), ib = pair_second(k, rot_pairs, rot_halves);
            const float a = qraw[r * DR + D + ia], b = qraw[r * DR + D + ib];
            float sn, cs;
            sincosf((float)positions[r0 + r] * freq[k], &sn, &cs);
            sn *= rot_mag;
            cs *= rot_mag;
            float* dst = qk + ((size_t)(r0 + r) * heads + h) * (C + R) + C;
            dst[ia] = (a * cs - b * sn) * scale;
            dst[ib] = (b * cs + a * sn) * scale;
        }
        const int rest = R - 2 * rot_pairs;                       // values of the rotated part that no pair holds
        for (int i = threadIdx.x; i < n * rest; i += blockDim.x) {
            const int r = i / rest, k = 2 * rot_pairs + i % rest;
            qk[((size_t)(r0 + r) * heads + h) * (C + R) + C + k] = qraw[r * DR + D + k] * scale;
        }
    }
    const int c = blockIdx.z * blockDim.x + threadIdx.x;      // one column of the key map a thread
    if (c < C) {
        const WT* col = w_uk + (size_t)h * D * C + c;
        float s[ROWS_Q];
#pragma unroll
        for (int r = 0; r < ROWS_Q; ++r) s[r] = 0.0f;
#pragma unroll 8
        for (int d = 0; d < D; ++d) {
            const float w = to_float(col[(size_t)d * C]);
#pragma unroll
            for (int r = 0; r < ROWS_Q; ++r) s[r] = fmaf(qraw[r * DR + d], w, s[r]);
        }
#pragma unroll
        for (int r = 0; r < ROWS_Q; ++r)
            if (r < n) qk[((size_t)(r0 + r) * heads + h) * (C + R) + c] = s[r] * scale;
    }
}

__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

constexpr int TILE_THREADS = 256;

// PLP: neighbouring pairs of a key's values a lane holds (C + R <= 64 * PLP; FULL: equal, so no value is out of range).
// A tile has 64 / sizeof(KVT) keys.
template <typename KVT, int PLP, bool FULL>
__global__ void __launch_bounds__(TILE_THREADS)
latent_scores_kernel(const float* __restrict__ qk, const KVT* __restrict__ cache, float* __restrict__ part,
                     const int* __restrict__ tiles, const int* __restrict__ row_request, const int* __restrict__ positions,
                     const int* __restrict__ block_tables, int table_stride, int heads, int C, int R, int HT, int splits,
                     int page_size, int window) {
    pdl_trigger();
    pdl_wait();
    constexpr int KT = 64 / (int)sizeof(KVT);
    extern __shared__ __align__(16) unsigned char tile_mem[];
    const int W = C + R, Wp = (W + 1) & ~1;
    KVT* bufs[2] = {reinterpret_cast<KVT*>(tile_mem), reinterpret_cast<KVT*>(tile_mem) + (size_t)KT * Wp};
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = tiles[2 * blockIdx.x], tile_rows = tiles[2 * blockIdx.x + 1];
    const int half = HT / 2;
    const int my_row = warp / half;
    const int h0 = blockIdx.y * HT + 2 * (warp % half), h1 = h0 + 1;
    const bool row_ok = my_row < tile_rows;
    const int row = row0 + (row_ok ? my_row : 0);
    const int pos = positions[row];
    const int lo_row = window > 0 ? max(0, pos - window + 1) : 0;
    // The block's keys: from the first row's lowest to the last row's own, cut into `splits` ranges of whole tiles.
    const int pos_first = positions[row0], pos_last = positions[row0 + tile_rows - 1];
    const int lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int total = pos_last + 1 - lo;
    const int chunk = ((total + splits - 1) / splits + KT - 1) / KT * KT;
    const int begin = lo + (int)blockIdx.z * chunk;
    const int end = min(begin + chunk, pos_last + 1);
    const int* table = block_tables + (size_t)row_request[row0] * table_stride;

    float q0[2 * PLP], q1[2 * PLP], acc0[2 * PLP], acc1[2 * PLP];
#pragma unroll
    for (int i = 0; i < PLP; ++i)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int e = 2 * lane + 64 * i + u;
            q0[2 * i + u] = (row_ok && h0 < heads && e < W) ? qk[((size_t)row * heads + h0) * W + e] : 0.0f;
            q1[2 * i + u] = (row_ok && h1 < heads && e < W) ? qk[((size_t)row * heads + h1) * W + e] : 0.0f;
            acc0[2 * i + u] = 0.0f;
            acc1[2 * i + u] = 0.0f;
        }
    float m0 = -INFINITY, l0 = 0.0f, m1 = -INFINITY, l1 = 0.0f;

    const int row_bytes = W * (int)sizeof(KVT);
    const bool vec = (row_bytes % 16) == 0;
    const int per_row = row_bytes / 16;                 // 16-byte pieces a key has (vector path)
    const int pieces = KT * per_row;
    uint4 stage[PLP];
    auto fetch = [&](int t0) {
#pragma unroll
        for (int j = 0; j < PLP; ++j) {
            const int c = threadIdx.x + j * TILE_THREADS;
            stage[j] = make_uint4(0u, 0u, 0u, 0u);
            if (c < pieces) {
                const int key = c / per_row, t = t0 + key;
                if (t < end) {
                    const KVT* src = cache + ((size_t)table[t / page_size] * page_size + t % page_size) * W;
                    stage[j] = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(src) + (size_t)(c % per_row) * 16);
                }
            }
        }
    };
    auto stash = [&](KVT* buf) {
#pragma unroll
        for (int j = 0; j < PLP; ++j) {
            const int c = threadIdx.x + j * TILE_THREADS;
            if (c < pieces)
                *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(buf) + ((size_t)(c / per_row) * Wp * sizeof(KVT)) + (size_t)(c % per_row) * 16) = stage[j];
        }
    };
    auto copy_plain = [&](KVT* buf, int t0) {          // rows that are no multiple of 16 bytes: value by value
        for (int i = threadIdx.x; i < KT * Wp; i += TILE_THREADS) {
            const int key = i / Wp, e = i % Wp, t = t0 + key;
            KVT v = from_float<KVT>(0.0f);
            if (t < end && e < W) v = cache[((size_t)table[t / page_size] * page_size + t % page_size) * W + e];
            buf[i] = v;
        }
    };

    const int n_tiles = end > begin ? (end - begin + KT - 1) / KT : 0;
    if (n_tiles > 0) {
        if (vec) {
            fetch(begin);
            stash(bufs[0]);
        } else {
            copy_plain(bufs[0], begin);
        }
    }
    __syncthreads();
    for (int it = 0; it < n_tiles; ++it) {
        const int t0 = begin + it * KT;
        const bool more = it + 1 < n_tiles;
        if (more && vec) fetch(t0 + KT);
        const KVT* buf = bufs[it & 1];
        if (row_ok) {
            const int j_hi = min(KT, min(end, pos + 1) - t0);
            int j = max(0, lo_row - t0);
            // Two keys a turn: their sums over the lanes and their exponentials overlap; the last odd key goes alone.
            for (; j + 1 < j_hi; j += 2) {
                const KVT* ka_row = buf + (size_t)j * Wp;
                const KVT* kb_row = ka_row + Wp;
                float ka[2 * PLP], kb[2 * PLP];
                float s0a = 0.0f, s1a = 0.0f, s0b = 0.0f, s1b = 0.0f;
#pragma unroll
                for (int i = 0; i < PLP; ++i) {
                    const int e = 2 * lane + 64 * i;
                    const float2 x = (FULL || e < Wp) ? load2(ka_row + e) : make_float2(0.0f, 0.0f);
                    const float2 y = (FULL || e < Wp) ? load2(kb_row + e) : make_float2(0.0f, 0.0f);
                    ka[2 * i] = x.x;
                    ka[2 * i + 1] = x.y;
                    kb[2 * i] = y.x;
                    kb[2 * i + 1] = y.y;
                    s0a = fmaf(q0[2 * i], x.x, s0a);
                    s1a = fmaf(q1[2 * i], x.x, s1a);
                    s0b = fmaf(q0[2 * i], y.x, s0b);
                    s1b = fmaf(q1[2 * i], y.x, s1b);
                    s0a = fmaf(q0[2 * i + 1], x.y, s0a);
                    s1a = fmaf(q1[2 * i + 1], x.y, s1a);
                    s0b = fmaf(q0[2 * i + 1], y.y, s0b);
                    s1b = fmaf(q1[2 * i + 1], y.y, s1b);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    s0a += __shfl_xor_sync(0xffffffffu, s0a, o);
                    s1a += __shfl_xor_sync(0xffffffffu, s1a, o);
                    s0b += __shfl_xor_sync(0xffffffffu, s0b, o);
                    s1b += __shfl_xor_sync(0xffffffffu, s1b, o);
                }
                const float n0 = fmaxf(s0a, s0b), n1 = fmaxf(s1a, s1b);
                if (n0 > m0) {
                    const float corr = expf(m0 - n0);
                    l0 *= corr;
#pragma unroll
                    for (int i = 0; i < 2 * PLP; ++i) acc0[i] *= corr;
                    m0 = n0;
                }
                if (n1 > m1) {
                    const float corr = expf(m1 - n1);
                    l1 *= corr;
#pragma unroll
                    for (int i = 0; i < 2 * PLP; ++i) acc1[i] *= corr;
                    m1 = n1;
                }
                const float p0a = expf(s0a - m0), p0b = expf(s0b - m0), p1a = expf(s1a - m1), p1b = expf(s1b - m1);
                l0 += p0a + p0b;
                l1 += p1a + p1b;
#pragma unroll
                for (int i = 0; i < 2 * PLP; ++i) {
                    acc0[i] = fmaf(p0b, kb[i], fmaf(p0a, ka[i], acc0[i]));
                    acc1[i] = fmaf(p1b, kb[i], fmaf(p1a, ka[i], acc1[i]));
                }
            }
            for (; j < j_hi; ++j) {
                const KVT* krow = buf + (size_t)j * Wp;
                float kv[2 * PLP];
                float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
                for (int i = 0; i < PLP; ++i) {
                    const int e = 2 * lane + 64 * i;
                    const float2 x = (FULL || e < Wp) ? load2(krow + e) : make_float2(0.0f, 0.0f);
                    kv[2 * i] = x.x;
                    kv[2 * i + 1] = x.y;
                    s0 = fmaf(q0[2 * i], x.x, s0);
                    s0 = fmaf(q0[2 * i + 1], x.y, s0);
                    s1 = fmaf(q1[2 * i], x.x, s1);
                    s1 = fmaf(q1[2 * i + 1], x.y, s1);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    s0 += __shfl_xor_sync(0xffffffffu, s0, o);
                    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
                }
                if (s0 > m0) {
                    const float corr = expf(m0 - s0);
                    l0 *= corr;
#pragma unroll
                    for (int i = 0; i < 2 * PLP; ++i) acc0[i] *= corr;
                    m0 = s0;
                }
                if (s1 > m1) {
                    const float corr = expf(m1 - s1);
                    l1 *= corr;
#pragma unroll
                    for (int i = 0; i < 2 * PLP; ++i) acc1[i] *= corr;
                    m1 = s1;
                }
                const float p0 = expf(s0 - m0), p1 = expf(s1 - m1);
                l0 += p0;
                l1 += p1;
#pragma unroll
                for (int i = 0; i < 2 * PLP; ++i) {
                    acc0[i] = fmaf(p0, kv[i], acc0[i]);
                    acc1[i] = fmaf(p1, kv[i], acc1[i]);
                }
            }
        }
        if (more) {
            if (vec) stash(bufs[(it + 1) & 1]);
            else copy_plain(bufs[(it + 1) & 1], t0 + KT);
        }
        __syncthreads();
    }
    if (!row_ok) return;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int h = u == 0 ? h0 : h1;
        if (h >= heads) continue;
        float* dst = part + (((size_t)row * heads + h) * splits + blockIdx.z) * (C + 2);
#pragma unroll
        for (int i = 0; i < 2 * PLP; ++i) {
            const int e = 2 * lane + 64 * (i >> 1) + (i & 1);
            if (e < C) dst[e] = u == 0 ? acc0[i] : acc1[i];
        }
        if (lane == 0) {
            dst[C] = u == 0 ? m0 : m1;
            dst[C + 1] = u == 0 ? l0 : l1;
        }
    }
}

template <typename WT, int ROWS_Q>
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ part, const WT* __restrict__ w_uv, WT* __restrict__ out, int rows, int heads,
                    int V, int C, int splits) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float lat[];             // ROWS_Q * C
    const int r0 = blockIdx.x * ROWS_Q, h = blockIdx.y;
    const int n = min(ROWS_Q, rows - r0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = 0; r < ROWS_Q; ++r) {
        if (r >= n) {
            for (int c = threadIdx.x; c < C; c += blockDim.x) lat[r * C + c] = 0.0f;
            continue;
        }
        const float* src = part + ((size_t)(r0 + r) * heads + h) * splits * (C + 2);
        float mm = -INFINITY;
        for (int s = 0; s < splits; ++s) mm = fmaxf(mm, src[(size_t)s * (C + 2) + C]);
        float ll = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float ms = src[(size_t)s * (C + 2) + C];
            ll += ms == -INFINITY ? 0.0f : src[(size_t)s * (C + 2) + C + 1] * expf(ms - mm);
        }
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            float o = 0.0f;
            for (int s = 0; s < splits; ++s) {
                const float ms = src[(size_t)s * (C + 2) + C];
                if (ms != -INFINITY) o = fmaf(src[(size_t)s * (C + 2) + c], expf(ms - mm), o);
            }
            lat[r * C + c] = o / ll;
        }
    }
    __syncthreads();
    const int v_per = (V + gridDim.z - 1) / gridDim.z;
    const int v_end = min(V, (int)(blockIdx.z + 1) * v_per);
    for (int v = blockIdx.z * v_per + warp; v < v_end; v += 4) {
        const WT* wr = w_uv + ((size_t)h * V + v) * C;
        float s[ROWS_Q];
#pragma unroll
        for (int r = 0; r < ROWS_Q; ++r) s[r] = 0.0f;
        for (int c = lane; c < C; c += 32) {
            const float w = to_float(wr[c]);
#pragma unroll
            for (int r = 0; r < ROWS_Q; ++r) s[r] = fmaf(w, lat[r * C + c], s[r]);
        }
#pragma unroll
        for (int r = 0; r < ROWS_Q; ++r) {
            const float t = warp_sum(s[r]);
            if (lane == 0 && r < n) out[((size_t)(r0 + r) * heads + h) * V + v] = from_float<WT>(t);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The scores step on the tensor cores (bfloat16 cache, C a multiple of 128 up to 512, C + R a multiple of 32).
// The 16 (row, head) pairs of a block are the 16 rows of an m16n8k16 product.  A 32-bit factor enters such a product
// as the sum of three bfloat16 values (x = hi + mid + lo, each the rounding of what the ones before left over): the
// products with the cache's bfloat16 values are exact and are added in 32-bit, so scores and weights keep 32-bit
// precision although the instruction takes 16-bit operands, at three instructions for one.
//   scores: warp w makes S[16 pairs, 16 of the tile's 64 keys] = (Qhi + Qmid + Qlo) K^T over half of C + R; the halves
//           are added when the weights are made
//   weights: warp w takes pairs 2w, 2w + 1: mask, running maximum and sum, p = exp(s - m) split three ways
//   values: warp w owns C / 8 columns of the weighted sum of latents: O = corr O + (Phi + Pmid + Plo) Kc
// Key tiles come by cp.async into two buffers (rows padded so that fragment loads meet no bank twice).
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void split3(float x, __nv_bfloat16& hi, __nv_bfloat16& mid, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(hi);
    mid = __float2bfloat16_rn(r1);
    lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool real) {
    const int n = real ? 16 : 0;               // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

constexpr int TC_KT = 64;                      // keys a tile
constexpr int TC_PS = TC_KT + 8;               // row stride of the weights' three parts (elements)
constexpr int TC_SS = TC_KT + 4;               // row stride of the scores (floats)

static inline size_t tc_smem_bytes(int W) {
    const size_t ws = (size_t)W + 8;
    return 2 * TC_KT * ws * 2 + 3 * 16 * ws * 2 + 3 * 16 * TC_PS * 2 + 2 * 16 * TC_SS * 4 + 16 * 4 * 6;
}

template <int NB>                              // n-blocks of 8 columns a warp owns: C = 64 * NB
__global__ void __launch_bounds__(TILE_THREADS, 1)
latent_scores_tc_kernel(const float* __restrict__ qk, const __nv_bfloat16* __restrict__ cache, float* __restrict__ part,
                        const int* __restrict__ tiles, const int* __restrict__ row_request,
                        const int* __restrict__ positions, const int* __restrict__ block_tables, int table_stride,
                        int heads, int C, int R, int HT, int splits, int page_size, int window) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char tc_mem[];
    const int W = C + R, WS = W + 8;
    __nv_bfloat16* keys = reinterpret_cast<__nv_bfloat16*>(tc_mem);                 // [2][TC_KT][WS]
    __nv_bfloat16* qs = keys + (size_t)2 * TC_KT * WS;                              // [3][16][WS]
    __nv_bfloat16* ps = qs + (size_t)3 * 16 * WS;                                   // [3][16][TC_PS]
    float* ss = reinterpret_cast<float*>(ps + 3 * 16 * TC_PS);                      // [2][16][TC_SS]: the scores' two halves of columns
    float* row_m = ss + 2 * 16 * TC_SS;                                                 // [16] running maximum
    float* row_l = row_m + 16;                                                      // [16] running sum
    float* row_c = row_l + 16;                                                      // [16] this tile's correction
    int* pair_row = reinterpret_cast<int*>(row_c + 16);                             // [16] row of the pair, or -1
    int* pair_lo = pair_row + 16;
    int* pair_pos = pair_lo + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c2 = (lane & 3) * 2;
    const int row0 = tiles[2 * blockIdx.x], tile_rows = tiles[2 * blockIdx.x + 1];
    const int pos_first = positions[row0], pos_last = positions[row0 + tile_rows - 1];
    const int lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int total = pos_last + 1 - lo;
    const int chunk = ((total + splits - 1) / splits + TC_KT - 1) / TC_KT * TC_KT;
    const int begin = lo + (int)blockIdx.z * chunk;
    const int end = min(begin + chunk, pos_last + 1);
    const int* table = block_tables + (size_t)row_request[row0] * table_stride;

    if (threadIdx.x < 16) {
        const int p = threadIdx.x, ri = p / HT, h = blockIdx.y * HT + p % HT;
        const bool ok = ri < tile_rows && h < heads;
        const int pos = ok ? positions[row0 + ri] : 0;
        pair_row[p] = ok ? row0 + ri : -1;
        pair_pos[p] = pos;
        pair_lo[p] = window > 0 ? max(0, pos - window + 1) : 0;
        row_m[p] = -INFINITY;
        row_l[p] = 0.0f;
    }
    for (int i = threadIdx.x; i < 16 * W; i += TILE_THREADS) {
        const int p = i / W, e = i % W, ri = p / HT, h = blockIdx.y * HT + p % HT;
        const float x = (ri < tile_rows && h < heads) ? qk[((size_t)(row0 + ri) * heads + h) * W + e] : 0.0f;
        __nv_bfloat16 a, b, c;
        split3(x, a, b, c);
        qs[(size_t)(0 * 16 + p) * WS + e] = a;
        qs[(size_t)(1 * 16 + p) * WS + e] = b;
        qs[(size_t)(2 * 16 + p) * WS + e] = c;
    }
    const int per_row = W / 8;                      // 16-byte pieces a key has
    auto issue = [&](int t0, int which) {
        const uint32_t base = (uint32_t)__cvta_generic_to_shared(keys + (size_t)which * TC_KT * WS);
        for (int c = threadIdx.x; c < TC_KT * per_row; c += TILE_THREADS) {
            const int key = c / per_row, piece = c % per_row, t = t0 + key;
            const bool real = t < end;
            const __nv_bfloat16* src = cache;
            if (real) src = cache + ((size_t)table[t / page_size] * page_size + t % page_size) * W + piece * 8;
            cp_async_16(base + (uint32_t)(key * WS + piece * 8) * 2, src, real);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float o[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[nb][i] = 0.0f;

    const int n_tiles = end > begin ? (end - begin + TC_KT - 1) / TC_KT : 0;
    if (n_tiles > 0) issue(begin, 0);
    const uint32_t qs_addr = (uint32_t)__cvta_generic_to_shared(qs);
    const uint32_t ps_addr = (uint32_t)__cvta_generic_to_shared(ps);
    for (int it = 0; it < n_tiles; ++it) {
        const int t0 = begin + it * TC_KT;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                             // tile `it` has landed; everyone is done with the other buffer
        if (it + 1 < n_tiles) issue(t0 + TC_KT, (it + 1) & 1);
        const uint32_t kaddr = (uint32_t)__cvta_generic_to_shared(keys + (size_t)(it & 1) * TC_KT * WS);
        // ---- scores: this warp's 16 keys over its half of the columns (a query fragment serves two blocks of 8 keys)
        {
            float sacc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
            const int n0 = (warp & 3) * 16, half = warp >> 2;
            const int k_begin = half * (W / 64) * 32, k_end = half == 0 ? (W / 64) * 32 : W;      // whole pairs of k-steps each
            for (int k0 = k_begin; k0 < k_end; k0 += 32) {
                // The instruction's own additions are cut off, not rounded, at the size of its accumulator: each 32
                // columns start from nothing and join the score by a rounded addition, the small parts first.
                float t[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
#pragma unroll
                for (int kk = 0; kk < 32; kk += 16) {
                    uint32_t b0, b1, b2, b3;     // (b0, b1): keys n0 .. n0 + 7; (b2, b3): the next eight; columns k0 + kk .. + 15
                    attn::ldmatrix_x4(kaddr + (uint32_t)((n0 + (lane & 7) + ((lane >> 4) << 3)) * WS + k0 + kk + ((lane >> 3) & 1) * 8) * 2,
                                      b0, b1, b2, b3);
#pragma unroll
                    for (int sp = 2; sp >= 0; --sp) {
                        uint32_t a[4];
                        attn::ldmatrix_x4(qs_addr + (uint32_t)((sp * 16 + (lane & 15)) * WS + k0 + kk + (lane >> 4) * 8) * 2, a[0], a[1], a[2], a[3]);
                        attn::mma_16816(t[0], a, b0, b1);
                        attn::mma_16816(t[1], a, b2, b3);
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    sacc[0][i] += t[0][i];
                    sacc[1][i] += t[1][i];
                }
            }
            float* mine = ss + half * 16 * TC_SS;
#pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
                mine[g * TC_SS + n0 + nb * 8 + c2] = sacc[nb][0];
                mine[g * TC_SS + n0 + nb * 8 + c2 + 1] = sacc[nb][1];
                mine[(g + 8) * TC_SS + n0 + nb * 8 + c2] = sacc[nb][2];
                mine[(g + 8) * TC_SS + n0 + nb * 8 + c2 + 1] = sacc[nb][3];
            }
        }
        __syncthreads();
        // ---- weights: pairs 2 * warp and 2 * warp + 1, two keys a lane
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int p = 2 * warp + u;
            const bool ok = pair_row[p] >= 0;
            const int plo = pair_lo[p], ppos = pair_pos[p];
            float sv[2];
            bool valid[2];
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const int t = t0 + lane + 32 * x;
                valid[x] = ok && t < end && t >= plo && t <= ppos;
                sv[x] = valid[x] ? ss[p * TC_SS + lane + 32 * x] + ss[(16 + p) * TC_SS + lane + 32 * x] : -INFINITY;
            }
            const float m_old = row_m[p];
            const float m_new = fmaxf(m_old, warp_max(fmaxf(sv[0], sv[1])));
            const float corr = m_new == -INFINITY ? 1.0f : expf(m_old - m_new);
            float psum = 0.0f;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const float pv = valid[x] ? expf(sv[x] - m_new) : 0.0f;
                psum += pv;
                __nv_bfloat16 a, b, c;
                split3(pv, a, b, c);
                ps[(0 * 16 + p) * TC_PS + lane + 32 * x] = a;
                ps[(1 * 16 + p) * TC_PS + lane + 32 * x] = b;
                ps[(2 * 16 + p) * TC_PS + lane + 32 * x] = c;
            }
            psum = warp_sum(psum);
            __syncwarp();
            if (lane == 0) {
                row_m[p] = m_new;
                row_l[p] = row_l[p] * corr + psum;
                row_c[p] = corr;
            }
        }
        __syncthreads();
        // ---- values: this warp's C / 8 columns
        {
            const float ca = row_c[g], cb = row_c[g + 8];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                o[nb][0] *= ca;
                o[nb][1] *= ca;
                o[nb][2] *= cb;
                o[nb][3] *= cb;
            }
            const int col0 = warp * NB * 8;
#pragma unroll
            for (int ks = 0; ks < TC_KT / 16; ++ks) {
                uint32_t a[3][4];
#pragma unroll
                for (int sp = 0; sp < 3; ++sp)
                    attn::ldmatrix_x4(ps_addr + (uint32_t)((sp * 16 + (lane & 15)) * TC_PS + ks * 16 + (lane >> 4) * 8) * 2,
                                      a[sp][0], a[sp][1], a[sp][2], a[sp][3]);
                const int key = ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
                for (int nb = 0; nb < NB; nb += 2) {
                    uint32_t b0, b1, b2, b3;
                    attn::ldmatrix_x4_trans(kaddr + (uint32_t)(key * WS + col0 + nb * 8 + (lane >> 4) * 8) * 2, b0, b1, b2, b3);
#pragma unroll
                    for (int sp = 0; sp < 3; ++sp) {
                        attn::mma_16816(o[nb], a[sp], b0, b1);
                        attn::mma_16816(o[nb + 1], a[sp], b2, b3);
                    }
                }
            }
        }
    }
    __syncthreads();
    // ---- the range's partial result: the weighted sum of latents, the maximum, the sum
    const int col0 = warp * NB * 8;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int p = g + 8 * half;
        const int row = pair_row[p];
        if (row < 0) continue;
        const int h = blockIdx.y * HT + p % HT;
        float* dst = part + (((size_t)row * heads + h) * splits + blockIdx.z) * (C + 2);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            dst[col0 + nb * 8 + c2] = o[nb][2 * half];
            dst[col0 + nb * 8 + c2 + 1] = o[nb][2 * half + 1];
        }
    }
    if (threadIdx.x < 16 && pair_row[threadIdx.x] >= 0) {
        const int p = threadIdx.x, h = blockIdx.y * HT + p % HT;
        float* dst = part + (((size_t)pair_row[p] * heads + h) * splits + blockIdx.z) * (C + 2);
        dst[C] = row_m[p];
        dst[C + 1] = row_l[p];
    }
}

template <typename KVT>
int launch_scores(int plp, dim3 grid, size_t smem, cudaStream_t stream, const float* qk, const void* cache, float* part,
                  const int* tiles, const int* row_request, const int* positions, const int* block_tables, int table_stride,
                  int heads, int C, int R, int HT, int splits, int page_size, int window) {
#define LLMX_SC(P)                                                                                                        \
    do {                                                                                                                  \
        if (C + R == 64 * P) {                                                                                            \
            if (smem > 48 * 1024)                                                                                         \
                cudaFuncSetAttribute(latent_scores_kernel<KVT, P, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            launch_kernel(latent_scores_kernel<KVT, P, true>, grid, dim3(TILE_THREADS), smem, stream, qk, (const KVT*)cache, \
                          part, tiles, row_request, positions, block_tables, table_stride, heads, C, R, HT, splits,     \
                          page_size, window);                                                                             \
        } else {                                                                                                          \
            if (smem > 48 * 1024)                                                                                         \
                cudaFuncSetAttribute(latent_scores_kernel<KVT, P, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            launch_kernel(latent_scores_kernel<KVT, P, false>, grid, dim3(TILE_THREADS), smem, stream, qk, (const KVT*)cache, \
                          part, tiles, row_request, positions, block_tables, table_stride, heads, C, R, HT, splits,     \
                          page_size, window);                                                                             \
        }                                                                                                                 \
    } while (0)
    if (plp <= 1) LLMX_SC(1);
    else if (plp <= 2) LLMX_SC(2);
    else if (plp <= 4) LLMX_SC(4);
    else if (plp <= 6) LLMX_SC(6);
    else if (plp <= 9) LLMX_SC(9);
    else if (plp <= 12) LLMX_SC(12);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_SC
    return launch_status();
}
}  // namespace

// How the tiled form cuts a step: heads a block holds (even, at most 16), rows a tile holds (16 / that).
LLMX_EXPORT void llmx_latent_tile_shape(int heads, int* heads_per_block, int* rows_per_tile) {
    int ht = (heads + 1) & ~1;
    ht = ht > 16 ? 16 : ht;
    while (16 % ht) ht += 2;                   // 2, 4, 8 or 16
    *heads_per_block = ht;
    *rows_per_tile = 16 / ht;
}

// The tiled form's three steps, each an entry point of its own (so that each shows in a profile).  Shapes as in
// llmx_latent_attention.  qk: float [rows, heads, C + R]; part: float [rows, heads, splits, C + 2].
LLMX_EXPORT int llmx_latent_query(const float* q, int q_stride, const void* w_uk, int w_dtype, float* qk, const float* freq,
                                  int rot_pairs, int rot_halves, float rot_mag, const int* positions, int rows, int heads, int D,
                                  int R, int C, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || heads > 65535 || D <= 0 || R < 0 || C <= 0 || 2 * rot_pairs > R) return LLMX_ERR_BAD_ARGUMENT;
    const int rq = rows > 64 ? 8 : 1;
    const size_t smem = (size_t)rq * (D + R) * sizeof(float);
    if (smem > 48 * 1024) return LLMX_ERR_UNSUPPORTED;
    const dim3 grid((rows + rq - 1) / rq, heads, (C + 127) / 128);
#define LLMX_Q(WT, RQ)                                                                                                    \
    launch_kernel(latent_query_kernel<WT, RQ>, grid, dim3(128), smem, stream, q, q_stride, (const WT*)w_uk, qk, freq,      \
                  rot_pairs, rot_halves, rot_mag, positions, rows, heads, D, R, C, scale)
    if (w_dtype == LLMX_BF16) {
        if (rq == 8) LLMX_Q(__nv_bfloat16, 8);
        else LLMX_Q(__nv_bfloat16, 1);
    } else if (w_dtype == LLMX_F32) {
        if (rq == 8) LLMX_Q(float, 8);
        else LLMX_Q(float, 1);
    } else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_Q
    return launch_status();
}

// `tiles` (device, int32 [n_tiles, 2]): first row and number of rows (at most the tile shape's) of every row tile, rows
// of one request each; `splits`: ranges the keys of a tile are cut into; `plain_cores`: never the tensor-core form.
LLMX_EXPORT int llmx_latent_scores(const float* qk, const void* cache, int cache_dtype, float* part, const int* tiles,
                                   int n_tiles, int splits, const int* row_request, const int* positions,
                                   const int* block_tables, int table_stride, int heads, int C, int R, int page_size,
                                   int window, int plain_cores, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (heads <= 0 || R < 0 || C <= 0 || page_size <= 0 || splits <= 0 || splits > 65535) return LLMX_ERR_BAD_ARGUMENT;
    const int W = C + R, Wp = (W + 1) & ~1;
    const int plp = (W + 63) / 64;
    int HT, RT;
    llmx_latent_tile_shape(heads, &HT, &RT);
    const dim3 grid(n_tiles, (heads + HT - 1) / HT, splits);
    const size_t smem = (size_t)2 * 64 * Wp;          // two tiles of 64 / sizeof(element) keys
    if (smem > 200 * 1024) return LLMX_ERR_UNSUPPORTED;
    if (cache_dtype == LLMX_BF16 && !plain_cores && W % 32 == 0 && (C == 128 || C == 256 || C == 512) && tc_smem_bytes(W) <= 220 * 1024) {
        const size_t tsm = tc_smem_bytes(W);
#define LLMX_TC(NB)                                                                                                       \
        do {                                                                                                              \
            cudaFuncSetAttribute(latent_scores_tc_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsm);     \
            launch_kernel(latent_scores_tc_kernel<NB>, grid, dim3(TILE_THREADS), tsm, stream, qk, (const __nv_bfloat16*)cache, \
                          part, tiles, row_request, positions, block_tables, table_stride, heads, C, R, HT, splits,     \
                          page_size, window);                                                                             \
        } while (0)
        if (C == 128) LLMX_TC(2);
        else if (C == 256) LLMX_TC(4);
        else LLMX_TC(8);
#undef LLMX_TC
        return launch_status();
    }
    if (cache_dtype == LLMX_BF16)
        return launch_scores<__nv_bfloat16>(plp, grid, smem, stream, qk, cache, part, tiles, row_request, positions, block_tables, table_stride, heads, C, R, HT, splits, page_size, window);
    if (cache_dtype == LLMX_F32)
        return launch_scores<float>(plp, grid, smem, stream, qk, cache, part, tiles, row_request, positions, block_tables, table_stride, heads, C, R, HT, splits, page_size, window);
    return LLMX_ERR_UNSUPPORTED;
}

LLMX_EXPORT int llmx_latent_merge(const float* part, const void* w_uv, int w_dtype, void* out, int rows, int heads, int V,
                                  int C, int splits, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || heads > 65535 || V <= 0 || C <= 0 || splits <= 0) return LLMX_ERR_BAD_ARGUMENT;
    const int rq = rows > 64 ? 8 : 1;
    const size_t smem = (size_t)rq * C * sizeof(float);
    if (smem > 48 * 1024) return LLMX_ERR_UNSUPPORTED;
    const dim3 grid((rows + rq - 1) / rq, heads, rq == 1 ? (V + 15) / 16 : (V + 63) / 64);      // 16 (few rows) or 64 value rows a block
#define LLMX_M(WT, RQ)                                                                                                    \
    launch_kernel(latent_merge_kernel<WT, RQ>, grid, dim3(128), smem, stream, part, (const WT*)w_uv, (WT*)out, rows,      \
                  heads, V, C, splits)
    if (w_dtype == LLMX_BF16) {
        if (rq == 8) LLMX_M(__nv_bfloat16, 8);
        else LLMX_M(__nv_bfloat16, 1);
    } else if (w_dtype == LLMX_F32) {
        if (rq == 8) LLMX_M(float, 8);
        else LLMX_M(float, 1);
    } else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_M
    return launch_status();
}

// down float [rows, stride]: Q query-latent values, C latent values, R rotated-part values; wq float [Q], w float [C];
// cq [rows, Q] of `cq_dtype` (Q may be 0: no query latent in the rows); freq float [rot_pairs]; slots[row] = page *
// page_size + offset (negative: no cache write for the row); cache [pages * page_size, C + R] of `cache_dtype`.
LLMX_EXPORT int llmx_latent_write(const float* down, int stride, int Q, const float* wq, void* cq, int cq_dtype, const float* w,
                                  float eps, const float* freq, int rot_pairs, int rot_halves, float rot_mag,
                                  const int* positions, const int* slots, void* cache, int cache_dtype, int rows, int C, int R,
                                  cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (C <= 0 || R < 0 || Q < 0 || 2 * rot_pairs > R || stride < Q + C + R) return LLMX_ERR_BAD_ARGUMENT;
#define LLMX_LW(KVT, QT)                                                                                                  \
    launch_kernel(latent_write_kernel<KVT, QT>, dim3(rows), dim3(128), 0, stream, down, stride, Q, wq, (QT*)cq, w, eps,   \
                  freq, rot_pairs, rot_halves, rot_mag, positions, slots, (KVT*)cache, C, R)
    if (cache_dtype == LLMX_BF16 && cq_dtype == LLMX_BF16) LLMX_LW(__nv_bfloat16, __nv_bfloat16);
    else if (cache_dtype == LLMX_BF16 && cq_dtype == LLMX_F32) LLMX_LW(__nv_bfloat16, float);
    else if (cache_dtype == LLMX_F32 && cq_dtype == LLMX_BF16) LLMX_LW(float, __nv_bfloat16);
    else if (cache_dtype == LLMX_F32 && cq_dtype == LLMX_F32) LLMX_LW(float, float);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_LW
    return launch_status();
}

// q float [rows, q_stride]: per head D unrotated then R rotated-part values; w_uk [heads * D, C] and w_uv [heads * V, C]
// of `w_dtype`, which is also the type of out [rows, heads * V].
LLMX_EXPORT int llmx_latent_attention(const float* q, int q_stride, const void* cache, int cache_dtype, const void* w_uk,
                                      const void* w_uv, int w_dtype, void* out, const float* freq, int rot_pairs,
                                      int rot_halves, float rot_mag, const int* row_request, const int* positions, const int* block_tables,
                                      int table_stride, int rows, int heads, int D, int R, int V, int C, int page_size,
                                      int window, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || heads > 65535 || D <= 0 || R < 0 || V <= 0 || C <= 0 || 2 * rot_pairs > R || page_size <= 0)
        return LLMX_ERR_BAD_ARGUMENT;
    const int W = C + R;
    const int pl = (W + 31) / 32;
    const size_t smem = (size_t)(D + R + W + WARPS * (C + 2)) * sizeof(float);
    if (smem > 200 * 1024) return LLMX_ERR_UNSUPPORTED;
    const dim3 grid(rows, heads);
#define LLMX_GO(WT, KVT)                                                                                                  \
    return launch_attention<WT, KVT>(pl, grid, smem, stream, q, q_stride, cache, w_uk, w_uv, out, freq, rot_pairs,       \
                                     rot_halves, rot_mag, row_request, positions, block_tables, table_stride, heads, D, R, V, C, page_size,   \
                                     window, scale)
    if (w_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) LLMX_GO(__nv_bfloat16, __nv_bfloat16);
    if (w_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) LLMX_GO(__nv_bfloat16, float);
    if (w_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) LLMX_GO(float, __nv_bfloat16);
    if (w_dtype == LLMX_F32 && cache_dtype == LLMX_F32) LLMX_GO(float, float);
#undef LLMX_GO
    return LLMX_ERR_UNSUPPORTED;
}
