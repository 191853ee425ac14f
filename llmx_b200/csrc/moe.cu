// A mixture of experts whose routing is a table: token id -> the `top` experts that token uses (no router product), or
// row of the step -> experts, as a router (`llmx_moe_router`) wrote it on the device.
//
// A step's rows are sorted by expert on the device, so that nothing about the routing is read on the host and a step
// can be recorded and replayed.  A *pair* is (row, k): row r with the k-th expert of its token, numbered r * top + k.
//   llmx_moe_route       one block an expert walks the pairs in order and lists those that name it (so a list is in
//                        row order, whatever else the launch holds); then one block cuts the lists into tiles of
//                        32 or 128 pairs (as the products' form wants): (expert, first place in the list), compactly,
//                        with their number.
//   llmx_moe_gate_up     act[pair, f] = silu(h[row] . Wg_e[f]) * (h[row] . Wu_e[f])         (gate and up rows stacked per expert)
//   llmx_moe_down        y[pair, c]   = act[pair] . Wd_e[c]                                 (32-bit)
//   llmx_moe_combine     x[row]      += weight * sum_k y[row * top + k]                      (k in order: one order of sums)
// The products run one block a (tile of an expert's pairs, tile of output columns): rows are gathered through the
// list, the expert's weights are read once a tile.  Two forms: on the CUDA cores with explicit fmaf and k in
// increasing order (32-bit weights and rows: the true 32-bit path; also bfloat16 shapes the tensor-core form does not
// take), and on the tensor cores (mma.sync m16n8k16, bfloat16 in, 32-bit sums) for bfloat16 with K a multiple of 32.
// A third form serves steps of a few pairs (decoding), where the products are the experts' weights streamed once.
// The CUDA-core form checks its tiles' size against what the routing wrote (tiles[1]).
#include "common.cuh"
#include <math.h>

namespace {
constexpr int TILE_ROWS = 32;     // pairs a tile holds

__global__ void __launch_bounds__(256)
route_kernel(const int* __restrict__ token_ids, const int* __restrict__ table, int top, int rows, int experts, int vocab,
             int* __restrict__ lists, int* __restrict__ counts) {
    pdl_trigger();
    pdl_wait();
    __shared__ int warp_count[8];
    __shared__ int base;
    const int e = blockIdx.x;
    const int pairs = rows * top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int p0 = 0; p0 < pairs; p0 += 256) {
        const int p = p0 + threadIdx.x;
        bool mine = false;
        if (p < pairs) {
            const int tok = token_ids ? token_ids[p / top] : p / top;      // no ids: the table has a row for each row of the step
            mine = tok >= 0 && tok < vocab && table[(size_t)tok * top + p % top] == e;
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_count[warp] = __popc(ballot);
        __syncthreads();
        int before = base;
        for (int w = 0; w < warp; ++w) before += warp_count[w];
        if (mine) lists[(size_t)e * pairs + before + __popc(ballot & ((1u << lane) - 1u))] = p;
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < 8; ++w) total += warp_count[w];
            base += total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = base;
}

// tiles: [0] their number, then (expert, first place) pairs from tiles[2] on.
__global__ void tiles_kernel(const int* __restrict__ counts, int experts, int* __restrict__ tiles, int tile_rows) {
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x != 0) return;
    int n = 0;
    for (int e = 0; e < experts; ++e)
        for (int at = 0; at < counts[e]; at += tile_rows) {
            tiles[2 + 2 * n] = e;
            tiles[3 + 2 * n] = at;
            ++n;
        }
    tiles[0] = n;
    tiles[1] = tile_rows;
}

// ---- the product on the CUDA cores ---------------------------------------------------------------------------------
// A block: TILE_ROWS pairs x 64 output columns, K in steps of 16; a thread owns 2 pairs x 4 columns (and, GATED, the
// same of the up rows).  A's rows are gathered: pair p reads row p / a_div of `a`.
constexpr int CC_COLS = 64, CC_K = 16;

template <typename T, bool GATED, typename OutT>
__global__ void __launch_bounds__(256)
moe_cores_kernel(const T* __restrict__ a, int a_div, const T* __restrict__ w, const int* __restrict__ lists,
                 const int* __restrict__ counts, const int* __restrict__ tiles, int pairs, OutT* __restrict__ out, int N,
                 int K) {
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x >= tiles[0] || tiles[1] != TILE_ROWS) return;
    const int e = tiles[2 + 2 * blockIdx.x], at = tiles[3 + 2 * blockIdx.x];
    const int n_here = min(TILE_ROWS, counts[e] - at);
    const int* list = lists + (size_t)e * pairs + at;
    const int col0 = blockIdx.y * CC_COLS;
    __shared__ float As[CC_K][TILE_ROWS + 1];
    __shared__ float Ws[GATED ? 2 : 1][CC_K][CC_COLS + 1];
    __shared__ int src_pair[TILE_ROWS];
    if (threadIdx.x < TILE_ROWS) src_pair[threadIdx.x] = threadIdx.x < n_here ? list[threadIdx.x] : -1;
    __syncthreads();
    const int tr = threadIdx.x / 16, tc = threadIdx.x % 16;        // pairs 2 tr, 2 tr + 1; columns tc + 16 j
    float acc[2][4] = {}, acc2[2][4] = {};
    const T* wbase = w + (size_t)e * (GATED ? 2 : 1) * N * K;
    for (int k0 = 0; k0 < K; k0 += CC_K) {
        for (int i = threadIdx.x; i < TILE_ROWS * CC_K; i += 256) {
            const int r = i / CC_K, kk = i % CC_K;
            const int p = src_pair[r];
            As[kk][r] = (p >= 0 && k0 + kk < K) ? to_float(a[(size_t)(p / a_div) * K + k0 + kk]) : 0.0f;
        }
        for (int i = threadIdx.x; i < CC_COLS * CC_K; i += 256) {
            const int c = i / CC_K, kk = i % CC_K;
            const bool ok = col0 + c < N && k0 + kk < K;
            Ws[0][kk][c] = ok ? to_float(wbase[(size_t)(col0 + c) * K + k0 + kk]) : 0.0f;
            if (GATED) Ws[1][kk][c] = ok ? to_float(wbase[(size_t)(N + col0 + c) * K + k0 + kk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < CC_K; ++kk) {
            const float a0 = As[kk][2 * tr], a1 = As[kk][2 * tr + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = Ws[0][kk][tc + 16 * j];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
                if (GATED) {
                    const float b2 = Ws[1][kk][tc + 16 * j];
                    acc2[0][j] = fmaf(a0, b2, acc2[0][j]);
                    acc2[1][j] = fmaf(a1, b2, acc2[1][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int p = src_pair[2 * tr + i];
        if (p < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + tc + 16 * j;
            if (c >= N) continue;
            float v = acc[i][j];
            if (GATED) v = v / (1.0f + expf(-v)) * acc2[i][j];
            out[(size_t)p * N + c] = from_float<OutT>(v);
        }
    }
}

// ---- the product on the tensor cores -------------------------------------------------------------------------------
// A block of eight warps: a tile of 128 pairs (the routing cut the lists into tiles of 128 for this form) x 128 weight
// rows, K in steps of 32 through four stages of cp.async copies (16-byte pieces; rows that do not exist are filled with
// zeros by the copy itself).  The 128 weight rows are two halves of 64: gated, the gate rows and the up rows of the
// same 64 output columns, so that a thread holds both of an output and writes silu(gate) * up; else 128 output columns.
// The weights are the A operand of mma.sync m16n8k16 and the gathered rows the B operand, both read by ldmatrix from
// rows padded by 8 values (no two of a read's eight rows in one bank).  Warp (wm, wn), wm < 4, wn < 2: weight rows
// 16 wm .. of both halves x pairs 64 wn .. 64 wn + 63.
constexpr int TC_ROWS = 128, TC_HALF = 64, TC_K = 32, TC_PAD = 8, TC_STAGES = 4, TC_LD = TC_K + TC_PAD;
constexpr int TC_STAGE_ELEMS = (2 * TC_HALF + TC_ROWS) * TC_LD;
constexpr size_t TC_SMEM = (size_t)TC_STAGES * TC_STAGE_ELEMS * 2;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async_16_or_zeros(void* dst, const void* src, bool real) {
    const int bytes = real ? 16 : 0;                 // fewer source bytes than 16: the rest of the piece is zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}

template <bool GATED, typename OutT>
__global__ void __launch_bounds__(256)
moe_tc_kernel(const __nv_bfloat16* __restrict__ a, int a_div, const __nv_bfloat16* __restrict__ w,
              const int* __restrict__ lists, const int* __restrict__ counts, const int* __restrict__ tiles, int pairs,
              OutT* __restrict__ out, int N, int K) {
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x >= tiles[0] || tiles[1] != TC_ROWS) return;
    extern __shared__ __align__(16) unsigned char tc_smem[];
    __nv_bfloat16* stages = reinterpret_cast<__nv_bfloat16*>(tc_smem);
    __shared__ int src_pair[TC_ROWS];
    const int e = tiles[2 + 2 * blockIdx.x], at = tiles[3 + 2 * blockIdx.x];
    const int n_here = min(TC_ROWS, counts[e] - at);
    const int* list = lists + (size_t)e * pairs + at;
    if (threadIdx.x < TC_ROWS) src_pair[threadIdx.x] = (int)threadIdx.x < n_here ? list[threadIdx.x] : -1;
    __syncthreads();
    const int out_cols = GATED ? TC_HALF : 2 * TC_HALF;           // output columns a block makes
    const int col0 = blockIdx.y * out_cols;
    const __nv_bfloat16* wbase = w + (size_t)e * (GATED ? 2 : 1) * N * K;
    // What this thread copies a stage: pieces t and t + 256 of the weights (row piece / 4, 8 values at 8 * (piece % 4)),
    // and the same of the gathered rows.  The rows' addresses do not change from stage to stage.
    const __nv_bfloat16* wsrc[2];
    const __nv_bfloat16* bsrc[2];
    bool wreal[2], breal[2];
    int dst_off[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int piece = threadIdx.x + 256 * i;
        const int row = piece >> 2, kp = piece & 3;
        const int half = row >> 6, rr = row & 63;
        const int col = col0 + (GATED ? rr : row);                // the output column this weight row belongs to
        wreal[i] = col < N;
        const size_t wrow = GATED ? (size_t)half * N + col : (size_t)col;
        wsrc[i] = wreal[i] ? wbase + wrow * K + 8 * kp : wbase;
        const int p = src_pair[row];
        breal[i] = p >= 0;
        bsrc[i] = breal[i] ? a + (size_t)(p / a_div) * K + 8 * kp : a;
        dst_off[i] = row * TC_LD + 8 * kp;
    }
    auto load = [&](int kt, int stage) {
        __nv_bfloat16* ws = stages + (size_t)stage * TC_STAGE_ELEMS;
        __nv_bfloat16* bs = ws + 2 * TC_HALF * TC_LD;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            cp_async_16_or_zeros(ws + dst_off[i], wsrc[i] + (size_t)kt * TC_K, wreal[i]);
            cp_async_16_or_zeros(bs + dst_off[i], bsrc[i] + (size_t)kt * TC_K, breal[i]);
        }
    };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp & 3, wn = warp >> 2;
    const int gid = lane >> 2, tig = lane & 3;
    float acc[2][8][4];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int t = 0; t < 8; ++t) acc[h][t][0] = acc[h][t][1] = acc[h][t][2] = acc[h][t][3] = 0.0f;
    const int KT = K / TC_K;
#pragma unroll
    for (int s = 0; s < TC_STAGES - 1; ++s) {
        if (s < KT) load(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // ldmatrix addresses inside a stage: A (weights): row lane % 16, k offset 8 * (lane / 16); B (pairs): two tiles of 8
    // pairs a read: pair (lane % 8) + 8 * (lane / 16), k offset 8 * ((lane / 8) % 2).
    const int a_row = lane & 15, a_k = (lane >> 4) * 8;
    const int b_row = (lane & 7) + ((lane >> 4) << 3), b_k = ((lane >> 3) & 1) * 8;
    for (int kt = 0; kt < KT; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(TC_STAGES - 2) : "memory");
        __syncthreads();                             // stage kt has landed; everyone has left the stage that is filled next
        if (kt + TC_STAGES - 1 < KT) load(kt + TC_STAGES - 1, (kt + TC_STAGES - 1) % TC_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const __nv_bfloat16* ws = stages + (size_t)(kt % TC_STAGES) * TC_STAGE_ELEMS;
        const __nv_bfloat16* bs = ws + 2 * TC_HALF * TC_LD;
#pragma unroll
        for (int ks = 0; ks < TC_K; ks += 16) {
            uint32_t af[2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const __nv_bfloat16* p = ws + (size_t)(h * TC_HALF + 16 * wm + a_row) * TC_LD + ks + a_k;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(af[h][0]), "=r"(af[h][1]), "=r"(af[h][2]), "=r"(af[h][3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
            }
            // All of the step's fragments are asked for before the first product, so that the reads overlap the products
            // of the step before (the statements keep their order; a warp's products do not wait for one another).
            uint32_t b[4][4];
#pragma unroll
            for (int t2 = 0; t2 < 4; ++t2) {
                const __nv_bfloat16* p = bs + (size_t)(64 * wn + 16 * t2 + b_row) * TC_LD + ks + b_k;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b[t2][0]), "=r"(b[t2][1]), "=r"(b[t2][2]), "=r"(b[t2][3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
            }
#pragma unroll
            for (int t2 = 0; t2 < 4; ++t2)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    mma_bf16(acc[h][2 * t2], af[h], b[t2][0], b[t2][1]);
                    mma_bf16(acc[h][2 * t2 + 1], af[h], b[t2][2], b[t2][3]);
                }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // d[0], d[1]: weight row 16 wm + gid of a half, pairs 64 wn + 8 t + 2 tig, + 1;  d[2], d[3]: weight row + 8.
#pragma unroll
    for (int t = 0; t < 8; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int p = src_pair[64 * wn + 8 * t + 2 * tig + (i & 1)];
            const int rr = 16 * wm + gid + (i >> 1) * 8;
            if (p < 0) continue;
            if (GATED) {
                const int c = col0 + rr;
                if (c < N) {
                    const float g = acc[0][t][i];
                    out[(size_t)p * N + c] = from_float<OutT>(g / (1.0f + expf(-g)) * acc[1][t][i]);
                }
            } else {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int c = col0 + h * TC_HALF + rr;
                    if (c < N) out[(size_t)p * N + c] = from_float<OutT>(acc[h][t][i]);
                }
            }
        }
}

// ---- steps of a few pairs -------------------------------------------------------------------------------------------
// With a handful of pairs (decoding) nearly every pair has an expert of its own and the products are the experts'
// weights streamed once: a block takes one pair and 16 output columns, its row lies in shared memory, and a warp makes
// two columns, each lane reading 16-byte pieces of the weight rows (several in flight) and the lanes' sums meeting by
// shuffles in a fixed order.  The pair's expert is read from the table; no lists are needed.
constexpr int GV_COLS = 16;

__device__ __forceinline__ void fma8(float& acc, const uint4& w, const uint4& x) {
    const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&w);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 a = __bfloat1622float2(wp[i]), b = __bfloat1622float2(xp[i]);
        acc = fmaf(a.x, b.x, acc);
        acc = fmaf(a.y, b.y, acc);
    }
}

template <bool GATED, typename OutT>
__global__ void __launch_bounds__(256)
moe_few_kernel(const __nv_bfloat16* __restrict__ a, int a_div, const __nv_bfloat16* __restrict__ w,
               const int* __restrict__ token_ids, const int* __restrict__ table, int top, int vocab, int experts,
               OutT* __restrict__ out, int N, int K) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char few_smem[];
    uint4* row = reinterpret_cast<uint4*>(few_smem);                 // the pair's row, K bfloat16
    const int p = blockIdx.x;
    const int tok = token_ids ? token_ids[p / top] : p / top;
    const int e = (tok >= 0 && tok < vocab) ? table[(size_t)tok * top + p % top] : -1;
    if (e < 0 || e >= experts) return;
    const uint4* src = reinterpret_cast<const uint4*>(a + (size_t)(p / a_div) * K);
    for (int i = threadIdx.x; i < K / 8; i += 256) row[i] = src[i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const __nv_bfloat16* wbase = w + (size_t)e * (GATED ? 2 : 1) * N * K;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int c = blockIdx.y * GV_COLS + 2 * warp + j;
        if (c >= N) continue;
        const uint4* w0 = reinterpret_cast<const uint4*>(wbase + (size_t)c * K);
        const uint4* w1 = reinterpret_cast<const uint4*>(wbase + (size_t)(N + c) * K);
        float s0 = 0.0f, s1 = 0.0f;
#pragma unroll 4
        for (int i = lane; i < K / 8; i += 32) {
            const uint4 x = row[i];
            fma8(s0, w0[i], x);
            if (GATED) fma8(s1, w1[i], x);
        }
        s0 = warp_sum(s0);
        if (GATED) s1 = warp_sum(s1);
        if (lane == 0) out[(size_t)p * N + c] = from_float<OutT>(GATED ? s0 / (1.0f + expf(-s0)) * s1 : s0);
    }
}

__global__ void combine_kernel(const float* __restrict__ y, float* __restrict__ x, int top, int width, float weight,
                               long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long row = i / width;
    const int c = (int)(i % width);
    float s = 0.0f;
    for (int k = 0; k < top; ++k) s += y[((size_t)row * top + k) * width + c];
    x[i] = fmaf(weight, s, x[i]);
}

// x[row] += factor * sum_k pair_weight[row * top + k] * y[row * top + k], k in increasing order.
__global__ void combine_weighted_kernel(const float* __restrict__ y, float* __restrict__ x, const float* __restrict__ pair_weight,
                                        int top, int width, float factor, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long row = i / width;
    const int c = (int)(i % width);
    float s = 0.0f;
    for (int k = 0; k < top; ++k) s = fmaf(pair_weight[row * top + k], y[((size_t)row * top + k) * width + c], s);
    x[i] = fmaf(factor, s, x[i]);
}

// A router: logits z = h W^T + b in 32-bit (h may be bfloat16; the weights are 32-bit), the `top` largest (the lower index
// first among equals), and as weights the softmax over the chosen logits alone.  `extra` more rows of W after the experts'
// give one number a row each through a sigmoid (a gate on a part that runs beside the experts).  A block takes R rows of
// the step (1 when the rows are few, so that they spread over the SMs; 8 when they are many, so that a weight row is read
// once for 8 rows); a row's logits do not depend on what else the step holds.
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
}

template <typename T, int R, int VEC>
__global__ void __launch_bounds__(256)
router_kernel(const T* __restrict__ h, const float* __restrict__ w, const float* __restrict__ bias, int rows, int K, int experts,
              int top, int extra, int* __restrict__ choice, float* __restrict__ weight, float* __restrict__ gate) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float router_z[];                    // [R][experts + extra], then the warps' parts [8][experts + extra][R]
    const int row0 = blockIdx.x * R, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int outs = experts + extra;
    float* part = router_z + R * outs;
    // The inner width is cut into runs of VEC values, run p going to thread p mod 256: a warp holds every eighth group of
    // 32 runs, for all logits, so its loads of one turn (a run of each row, a run of each of four weight rows) do not wait
    // for one another.  Parts are summed lane tree first, then warps in order: one order whatever the step holds.
    constexpr int EC = R == 1 ? 8 : 4;                       // few rows: more weight rows a turn, so that more loads are in flight
    for (int e0 = 0; e0 < outs; e0 += EC) {
        float s[EC][R];
#pragma unroll
        for (int j = 0; j < EC; ++j)
#pragma unroll
            for (int r = 0; r < R; ++r) s[j][r] = 0.0f;
#pragma unroll(R == 1 ? 2 : 1)
        for (int k = VEC * (int)threadIdx.x; k < K; k += VEC * 256) {
            float xv[R][VEC];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (row0 + r < rows) {
                    if constexpr (VEC == 4) load4(h + (size_t)(row0 + r) * K + k, xv[r]);
                    else xv[r][0] = to_float(h[(size_t)(row0 + r) * K + k]);
                } else {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) xv[r][i] = 0.0f;
                }
            }
#pragma unroll
            for (int j = 0; j < EC; ++j) {
                if (e0 + j >= outs) break;
                float wv[VEC];
                if constexpr (VEC == 4) load4(w + (size_t)(e0 + j) * K + k, wv);
                else wv[0] = w[(size_t)(e0 + j) * K + k];
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int i = 0; i < VEC; ++i) s[j][r] = fmaf(xv[r][i], wv[i], s[j][r]);
            }
        }
#pragma unroll
        for (int j = 0; j < EC; ++j) {
            if (e0 + j >= outs) break;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float t = warp_sum(s[j][r]);
                if (lane == 0) part[((size_t)warp * outs + e0 + j) * R + r] = t;
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < R * outs; i += blockDim.x) {
        const int r = i / outs, e = i - r * outs;
        float t = 0.0f;
        for (int wp = 0; wp < 8; ++wp) t += part[((size_t)wp * outs + e) * R + r];
        router_z[i] = t + ((bias && e < experts) ? bias[e] : 0.0f);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < R * extra; i += blockDim.x) {
        const int r = i / extra, x = i - r * extra;
        if (row0 + r < rows) gate[(size_t)(row0 + r) * extra + x] = 1.0f / (1.0f + expf(-router_z[r * outs + experts + x]));
    }
    if (threadIdx.x >= R || row0 + (int)threadIdx.x >= rows) return;
    // One thread a row picks: the largest logit left, `top` times (a chosen one is struck out in shared memory; the chosen
    // logits wait in the warps' parts, which nobody reads any more), then the softmax over the chosen.
    float* z = router_z + threadIdx.x * outs;
    float* picked = part + (size_t)threadIdx.x * top;
    int* mine = choice + (size_t)(row0 + threadIdx.x) * top;
    float* wt = weight + (size_t)(row0 + threadIdx.x) * top;
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float bz = -INFINITY;
        for (int e = 0; e < experts; ++e) {
            const float ze = z[e];
            if (ze > bz) best = e, bz = ze;                  // the lower index first among equals; no number is never larger
        }
        if (best < 0) {                                      // nothing left that is a number
            for (int e = 0; e < experts && best < 0; ++e)
                if (z[e] != z[e]) best = e;
            best = best < 0 ? 0 : best;
        }
        z[best] = -INFINITY;
        mine[k] = best;
        picked[k] = bz;
    }
    const float zmax = picked[0];
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
        const float e = zmax == -INFINITY ? 1.0f : expf(picked[k] - zmax);
        picked[k] = e;
        sum += e;
    }
    for (int k = 0; k < top; ++k) wt[k] = picked[k] / sum;
}

inline int max_tiles(int pairs, int experts, int tile_rows) { return (pairs + tile_rows - 1) / tile_rows + experts; }
}  // namespace

// h [rows, K] of `dtype`; w float32 [experts + extra, K]; bias float32 [experts] or null; choice int32 [rows, top]; weight float32
// [rows, top]; gate float32 [rows, extra] (extra 0: not used).
LLMX_EXPORT int llmx_moe_router(const void* h, int dtype, const float* w, const float* bias, int rows, int K, int experts, int top,
                                int extra, int* choice, float* weight, float* gate, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (K <= 0 || experts <= 0 || top <= 0 || top > experts || extra < 0 || extra > 128 || (extra > 0 && gate == nullptr) ||
        experts + extra > 1024)
        return LLMX_ERR_BAD_ARGUMENT;
    // Eight rows a block when the rows are many (a weight row is then read once for eight rows), one when they are few.
    const bool vec = (K & 3) == 0 && !((uintptr_t)h & 15) && !((uintptr_t)w & 15);
    int R = rows > 64 ? 8 : 1;
    size_t smem = (size_t)9 * R * (experts + extra) * sizeof(float);
    if (smem > 40 * 1024) R = 1, smem = (size_t)9 * (experts + extra) * sizeof(float);
    if (smem > 40 * 1024) return LLMX_ERR_UNSUPPORTED;
    const dim3 grid((rows + R - 1) / R);
#define LLMX_ROUTER(T, RR, V) \
    launch_kernel(router_kernel<T, RR, V>, grid, dim3(256), smem, stream, (const T*)h, w, bias, rows, K, experts, top, extra, choice, weight, gate)
#define LLMX_ROUTER_T(T)                      \
    do {                                      \
        if (R == 8 && vec) LLMX_ROUTER(T, 8, 4); \
        else if (R == 8) LLMX_ROUTER(T, 8, 1);   \
        else if (vec) LLMX_ROUTER(T, 1, 4);      \
        else LLMX_ROUTER(T, 1, 1);               \
    } while (0)
    if (dtype == LLMX_BF16) LLMX_ROUTER_T(__nv_bfloat16);
    else if (dtype == LLMX_F32) LLMX_ROUTER_T(float);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_ROUTER_T
#undef LLMX_ROUTER
    return launch_status();
}

// x [rows, width] += factor * sum over k of pair_weight[rows * top] * y [rows * top, width], k in increasing order.
LLMX_EXPORT int llmx_moe_combine_weighted(const float* y, float* x, const float* pair_weight, int rows, int top, int width,
                                          float factor, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (pair_weight == nullptr) return LLMX_ERR_BAD_ARGUMENT;
    const long long n = (long long)rows * width;
    launch_kernel(combine_weighted_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, y, x, pair_weight, top, width, factor, n);
    return launch_status();
}

// The pairs a tile holds for the products' two forms: the routing cuts the lists for the form that will run.
LLMX_EXPORT int llmx_moe_tile_rows(int tensor_cores) { return tensor_cores ? TC_ROWS : TILE_ROWS; }

// Whether the tensor-core form takes a product of these sizes and type.
LLMX_EXPORT int llmx_moe_tensor_cores_fit(int dtype, int K) { return dtype == LLMX_BF16 && K > 0 && K % TC_K == 0; }

// token_ids int32 [rows]; table int32 [vocab, top]; lists int32 [experts, rows * top]; counts int32 [experts]; tiles int32
// [2 + 2 * (ceil(rows * top / tile_rows) + experts)].
LLMX_EXPORT int llmx_moe_route(const int* token_ids, const int* table, int top, int rows, int experts, int vocab, int* lists,
                               int* counts, int* tiles, int tile_rows, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (top <= 0 || experts <= 0 || experts > 65535 || (tile_rows != TILE_ROWS && tile_rows != TC_ROWS)) return LLMX_ERR_BAD_ARGUMENT;
    launch_kernel(route_kernel, dim3(experts), dim3(256), 0, stream, token_ids, table, top, rows, experts, vocab, lists, counts);
    int status = launch_status();
    if (status) return status;
    launch_kernel(tiles_kernel, dim3(1), dim3(32), 0, stream, (const int*)counts, experts, tiles, tile_rows);
    return launch_status();
}

// a [rows of `a_div` pairs each, K] and w [experts, (gated ? 2 : 1) * N, K] of `dtype`; out [pairs, N] of `out_dtype`
// (gated: silu(gate) * up; else the plain product, float32).  `tensor_cores`: the form to run; the routing must have cut
// the lists into tiles of `llmx_moe_tile_rows(tensor_cores)` pairs.
LLMX_EXPORT int llmx_moe_product(const void* a, int a_div, const void* w, int dtype, const int* lists, const int* counts,
                                 const int* tiles, int pairs, int experts, void* out, int out_dtype, int N, int K,
                                 int gated, int tensor_cores, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (N <= 0 || K <= 0 || a_div <= 0) return LLMX_ERR_BAD_ARGUMENT;
    if (!gated && out_dtype != LLMX_F32) return LLMX_ERR_UNSUPPORTED;
    if (tensor_cores) {
        if (!llmx_moe_tensor_cores_fit(dtype, K) || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return LLMX_ERR_UNSUPPORTED;
        const int out_cols = gated ? TC_HALF : 2 * TC_HALF;
        dim3 grid(max_tiles(pairs, experts, TC_ROWS), (N + out_cols - 1) / out_cols);
        if (grid.y > 65535) return LLMX_ERR_UNSUPPORTED;
        const __nv_bfloat16* ab = (const __nv_bfloat16*)a;
        const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
#define LLMX_MOE_TC(G, O)                                                                                              \
    do {                                                                                                                \
        cudaFuncSetAttribute(moe_tc_kernel<G, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);          \
        launch_kernel(moe_tc_kernel<G, O>, dim3(grid), dim3(256), TC_SMEM, stream, ab, a_div, wb, lists, counts, tiles, \
                      pairs, (O*)out, N, K);                                                                            \
    } while (0)
        if (gated && out_dtype == LLMX_BF16) LLMX_MOE_TC(true, __nv_bfloat16);
        else if (gated) LLMX_MOE_TC(true, float);
        else LLMX_MOE_TC(false, float);
#undef LLMX_MOE_TC
        return launch_status();
    }
    dim3 grid(max_tiles(pairs, experts, TILE_ROWS), (N + CC_COLS - 1) / CC_COLS);
    if (grid.y > 65535) return LLMX_ERR_UNSUPPORTED;
#define LLMX_MOE(T, G, O) \
    launch_kernel(moe_cores_kernel<T, G, O>, dim3(grid), dim3(256), 0, stream, (const T*)a, a_div, (const T*)w, lists, counts, tiles, pairs, (O*)out, N, K)
    if (dtype == LLMX_BF16 && gated && out_dtype == LLMX_BF16) LLMX_MOE(__nv_bfloat16, true, __nv_bfloat16);
    else if (dtype == LLMX_BF16 && gated && out_dtype == LLMX_F32) LLMX_MOE(__nv_bfloat16, true, float);
    else if (dtype == LLMX_BF16 && !gated) LLMX_MOE(__nv_bfloat16, false, float);
    else if (dtype == LLMX_F32 && gated && out_dtype == LLMX_F32) LLMX_MOE(float, true, float);
    else if (dtype == LLMX_F32 && !gated) LLMX_MOE(float, false, float);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_MOE
    return launch_status();
}

// The same products for steps of a few pairs, without lists: a [rows of `a_div` pairs each, K] and w bfloat16 with K a
// multiple of 8; the pair's expert is read from the table.
LLMX_EXPORT int llmx_moe_product_few(const void* a, int a_div, const void* w, const int* token_ids, const int* table,
                                     int top, int vocab, int pairs, int experts, void* out, int out_dtype, int N, int K,
                                     int gated, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (N <= 0 || K <= 0 || K % 8 || a_div <= 0 || top <= 0 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return LLMX_ERR_UNSUPPORTED;
    if (!gated && out_dtype != LLMX_F32) return LLMX_ERR_UNSUPPORTED;
    const size_t smem = (size_t)K * 2;
    if (smem > 200 * 1024) return LLMX_ERR_UNSUPPORTED;
    dim3 grid(pairs, (N + GV_COLS - 1) / GV_COLS);
    if (grid.y > 65535) return LLMX_ERR_UNSUPPORTED;
#define LLMX_FEW(G, O)                                                                                                  \
    do {                                                                                                                \
        if (smem > 48 * 1024) cudaFuncSetAttribute(moe_few_kernel<G, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_kernel(moe_few_kernel<G, O>, dim3(grid), dim3(256), smem, stream, (const __nv_bfloat16*)a, a_div,       \
                      (const __nv_bfloat16*)w, token_ids, table, top, vocab, experts, (O*)out, N, K);                   \
    } while (0)
    if (gated && out_dtype == LLMX_BF16) LLMX_FEW(true, __nv_bfloat16);
    else if (gated) LLMX_FEW(true, float);
    else LLMX_FEW(false, float);
#undef LLMX_FEW
    return launch_status();
}

// x [rows, width] += weight * sum over k of y [rows * top, width], k in increasing order.
LLMX_EXPORT int llmx_moe_combine(const float* y, float* x, int rows, int top, int width, float weight, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const long long n = (long long)rows * width;
    launch_kernel(combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, y, x, top, width, weight, n);
    return launch_status();
}
