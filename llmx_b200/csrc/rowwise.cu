// Row-wise kernels: embedding gather, RMSNorm, per-head norm + rotation + cache write, SwiGLU.
//
// All arithmetic is 32-bit: sums of squares, the reciprocal root, the rotation
// and the activation.  Only what is stored for a matrix product or in the cache
// is rounded to bfloat16 on the bfloat16 path.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: x[r, :] = table[ids[r], :] widened to 32-bit.
// Reference: llmx_gather (src/backends/gpu/kernels/f32.gpu:747-751).  Ids are checked
// on the host before the step; an id outside the table writes a zero row here.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ x,
                             int width, int table_rows) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int id = ids[r];
    float* dst = x + (size_t)r * width;
    if (id < 0 || id >= table_rows) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = 0.0f;
        return;
    }
    const T* src = table + (size_t)id * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = to_float(src[i]);
}

LLMX_EXPORT int llmx_embed(const void* table, int table_dtype, const int* ids, float* x, int rows, int width,
                           int table_rows, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (table_dtype == LLMX_BF16)
        launch_kernel(embed_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, (const __nv_bfloat16*)table, ids, x, width, table_rows);
    else
        launch_kernel(embed_kernel<float>, dim3(rows), dim3(256), 0, stream, (const float*)table, ids, x, width, table_rows);
    return launch_status();
}

// ---------------------------------------------------------------------------
// RMSNorm: s = sum x_i^2; r = 1 / sqrt(s / n + eps); y_i = x_i * (r * w_i)
// (the grouping x * (r * w) is the reference's, src/backends/cpu/cpu_backend.hpp:1437-1459).
// `row_index` (optional) picks the source rows: y[i] = norm(x[row_index[i]]), which folds
// the head's row gather (src/model/arch/blocks.hpp:267-272) into its norm.
// ---------------------------------------------------------------------------
template <typename OutT>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, OutT* __restrict__ y,
                               const int* __restrict__ row_index, int width, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const float* src = x + (size_t)(row_index ? row_index[r] : r) * width;
    float s = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = src[i];
        s = fmaf(v, v, s);
    }
    s = block_sum(s, scratch);
    const float rr = 1.0f / sqrtf(s / (float)width + eps);
    OutT* dst = y + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_float<OutT>(src[i] * (rr * w[i]));
}

// The same for widths that are a multiple of 4 and at most 4 * VEC_MAX * blockDim: each thread keeps its
// values in registers (one read of the row, 16-byte loads all issued before the first is used).
constexpr int NORM_VEC_MAX = 8;

__device__ __forceinline__ void store4(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = v;
}

// `zero` (optional): a float buffer of `zero_count` values (a multiple of 4, 16-byte aligned) that the launch
// clears with blocks of its own (those beyond `rows`): the output of the product that follows, when that product
// adds its pieces with atomics.
template <typename OutT>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, OutT* __restrict__ y,
                                   const int* __restrict__ row_index, int rows, int width, float eps,
                                   float* __restrict__ zero, long long zero_count) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    if (r >= rows) {
        // Blocks beyond the rows only clear: with a few rows, a few blocks would store for longer than the norm takes.
        float4* z = reinterpret_cast<float4*>(zero);
        const long long n4 = zero_count >> 2;
        const long long blocks = gridDim.x - rows;
        for (long long i = (long long)(r - rows) * blockDim.x + threadIdx.x; i < n4; i += blocks * blockDim.x)
            z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(row_index ? row_index[r] : r) * width);
    const float4* wv = reinterpret_cast<const float4*>(w);
    const int n4 = width >> 2;
    float4 v[NORM_VEC_MAX];
#pragma unroll
    for (int k = 0; k < NORM_VEC_MAX; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        v[k] = i < n4 ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < NORM_VEC_MAX; ++k) {
        s = fmaf(v[k].x, v[k].x, s);
        s = fmaf(v[k].y, v[k].y, s);
        s = fmaf(v[k].z, v[k].z, s);
        s = fmaf(v[k].w, v[k].w, s);
    }
    s = block_sum(s, scratch);
    const float rr = 1.0f / sqrtf(s / (float)width + eps);
    OutT* dst = y + (size_t)r * width;
#pragma unroll
    for (int k = 0; k < NORM_VEC_MAX; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < n4) {
            const float4 ww = wv[i];
            store4(dst + 4 * i, v[k].x * (rr * ww.x), v[k].y * (rr * ww.y), v[k].z * (rr * ww.z), v[k].w * (rr * ww.w));
        }
    }
}

LLMX_EXPORT int llmx_rmsnorm(const float* x, const float* w, void* y, int out_dtype, const int* row_index, int rows,
                             int width, float eps, float* zero, long long zero_count, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (zero && (zero_count % 4 || ((uintptr_t)zero & 15))) return LLMX_ERR_BAD_ARGUMENT;
    const bool aligned = width % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)w & 15) && !((uintptr_t)y & 15);
    if (aligned && width <= 4 * NORM_VEC_MAX * 256) {
        const int n4 = width / 4;
        // The block width depends on the row width alone, so a row's sum has one order whatever the batch.
        int threads = ((n4 + 3) / 4 + 31) / 32 * 32;
        threads = threads < 32 ? 32 : threads > 256 ? 256 : threads;
        // Clearing: blocks of their own, each about 16 KB (four 16-byte stores a thread), at most 1,024 of them.
        long long zero_blocks = zero ? (zero_count / 4 + 4 * threads - 1) / (4 * threads) : 0;
        zero_blocks = zero_blocks > 1024 ? 1024 : zero_blocks;
        const dim3 grid((unsigned)(rows + zero_blocks));
        if (out_dtype == LLMX_BF16)
            launch_kernel(rmsnorm_vec_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, x, w, (__nv_bfloat16*)y, row_index, rows, width, eps, zero, zero_count);
        else
            launch_kernel(rmsnorm_vec_kernel<float>, grid, dim3(threads), 0, stream, x, w, (float*)y, row_index, rows, width, eps, zero, zero_count);
        return launch_status();
    }
    if (zero && cudaMemsetAsync(zero, 0, (size_t)zero_count * sizeof(float), stream) != cudaSuccess) return launch_status();
    const int threads = width >= 1024 ? 256 : 128;
    if (out_dtype == LLMX_BF16)
        launch_kernel(rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, x, w, (__nv_bfloat16*)y, row_index, width, eps);
    else
        launch_kernel(rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, stream, x, w, (float*)y, row_index, width, eps);
    return launch_status();
}

// ---------------------------------------------------------------------------
// Per-head norm, rotation and cache write, one warp per (row, head).
//
// For a query head: RMSNorm over the head's D values with q_weight (skipped when null),
// rotate the first 2*rot_half values by the row's position, store to q_out.
// For a key head: the same with k_weight, stored to the key plane of the row's cache
// slot; the value head is stored raw to the value plane.
// Rotation pairs (i, i + rot_half), i < rot_half ("rotate half"):
//   a' = fma(-b, sin_i, a * cos_i);  b' = fma(a, sin_i, b * cos_i)
// (src/backends/cpu/cpu_backend.hpp:1461-1480, fused form f32.gpu:722-744).
// Cache layout: [page][plane][kv_head][slot][D]; `slots[row]` = page * page_size + slot,
// or negative to skip the write (a layer that reads another layer's cache).
// ---------------------------------------------------------------------------
template <typename QT, typename KVT>
__global__ void head_norm_rope_kernel(const float* __restrict__ qkv, int qkv_stride, int k_offset, int v_offset,
                                      const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                      float eps, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                      int rot_half, const int* __restrict__ positions, const int* __restrict__ slots,
                                      QT* __restrict__ q_out, KVT* __restrict__ cache, int rows, int heads, int kv_heads,
                                      int head_dim, int page_size) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_row = heads + kv_heads;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)rows * per_row) return;
    const int row = (int)(item / per_row), j = (int)(item % per_row);
    const bool is_q = j < heads;
    const int g = is_q ? 0 : j - heads;
    float* buf = smem + warp * head_dim;
    const float* src = qkv + (size_t)row * qkv_stride + (is_q ? j * head_dim : k_offset + g * head_dim);
    const float* weight = is_q ? q_weight : k_weight;

    int slot = 0;
    if (!is_q) {
        slot = slots[row];
        if (slot < 0) return;
    }
    float s = 0.0f;
    for (int d = lane; d < head_dim; d += 32) {
        const float v = src[d];
        buf[d] = v;
        s = fmaf(v, v, s);
    }
    if (weight) {
        s = warp_sum(s);
        const float rr = 1.0f / sqrtf(s / (float)head_dim + eps);
        __syncwarp();
        for (int d = lane; d < head_dim; d += 32) buf[d] = buf[d] * (rr * weight[d]);
    }
    __syncwarp();
    size_t key_base = 0, value_base = 0;
    if (!is_q) {
        const int page = slot / page_size, off = slot % page_size;
        key_base = ((((size_t)page * 2 + 0) * kv_heads + g) * page_size + off) * head_dim;
        value_base = ((((size_t)page * 2 + 1) * kv_heads + g) * page_size + off) * head_dim;
    }
    const float* cs = cos_table ? cos_table + (size_t)positions[row] * rot_half : nullptr;
    const float* sn = cos_table ? sin_table + (size_t)positions[row] * rot_half : nullptr;
    for (int d = lane; d < head_dim; d += 32) {
        float out;
        if (cs && d < 2 * rot_half) {
            const int i = d < rot_half ? d : d - rot_half;
            const float a = buf[i], b = buf[i + rot_half];
            out = d < rot_half ? fmaf(-b, sn[i], a * cs[i]) : fmaf(a, sn[i], b * cs[i]);
        } else {
            out = buf[d];
        }
        if (is_q) q_out[(size_t)row * heads * head_dim + j * head_dim + d] = from_float<QT>(out);
        else cache[key_base + d] = from_float<KVT>(out);
    }
    if (!is_q) {
        const float* vsrc = qkv + (size_t)row * qkv_stride + v_offset + g * head_dim;
        for (int d = lane; d < head_dim; d += 32) cache[value_base + d] = from_float<KVT>(vsrc[d]);
    }
}

// The same for the common shape -- a head of 128 values rotated whole (64 pairs) -- with each lane holding
// four consecutive values (16-byte loads, 8-byte stores); a pair's partner sits 16 lanes away.  A warp takes
// U consecutive (row, head) items of one row (U divides heads + kv_heads): their loads are all asked for
// before the first is used, and the row's position, cosines and sines are fetched once.
template <typename QT, typename KVT, int U>
__global__ void head_norm_rope_128_kernel(const float* __restrict__ qkv, int qkv_stride, int k_offset, int v_offset,
                                          const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                          float eps, const float* __restrict__ cos_table,
                                          const float* __restrict__ sin_table, const int* __restrict__ positions,
                                          const int* __restrict__ slots, QT* __restrict__ q_out, KVT* __restrict__ cache,
                                          int rows, int heads, int kv_heads, int page_size) {
    pdl_trigger();
    pdl_wait();
    constexpr int D = 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_row = heads + kv_heads;
    // 32-bit arithmetic (the launcher sees to it that rows * per_row fits): a 64-bit division costs this
    // kernel, which is bound by the instructions it issues, a tenth of its time.
    const unsigned first = (blockIdx.x * (blockDim.x >> 5) + warp) * U;
    if (first >= (unsigned)rows * (unsigned)per_row) return;
    const int row = (int)(first / (unsigned)per_row), j0 = (int)(first - (unsigned)row * (unsigned)per_row);
    const float* row_src = qkv + (size_t)row * qkv_stride;
    const int slot = slots[row];
    float4 v[U], raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int j = j0 + u;
        const bool is_q = j < heads;
        const int g = is_q ? 0 : j - heads;
        v[u] = reinterpret_cast<const float4*>(row_src + (is_q ? j * D : k_offset + g * D))[lane];
        if (!is_q && slot >= 0) raw[u] = reinterpret_cast<const float4*>(row_src + v_offset + g * D)[lane];
    }
    float4 c = make_float4(1.f, 1.f, 1.f, 1.f), sn = make_float4(0.f, 0.f, 0.f, 0.f);
    if (cos_table) {
        // Lane l < 16 holds a = x[4l..4l+3], lane l + 16 holds b = x[64 + 4l ..]; both need cos/sin[4 (l % 16) ..].
        const size_t base = (size_t)positions[row] * 64 + 4 * (lane & 15);
        c = *reinterpret_cast<const float4*>(cos_table + base);
        sn = *reinterpret_cast<const float4*>(sin_table + base);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int j = j0 + u;
        const bool is_q = j < heads;
        const int g = is_q ? 0 : j - heads;
        if (!is_q && slot < 0) continue;
        const float* weight = is_q ? q_weight : k_weight;
        float4 x = v[u];
        if (weight) {
            float s = fmaf(x.x, x.x, fmaf(x.y, x.y, fmaf(x.z, x.z, x.w * x.w)));
            s = warp_sum(s);
            const float rr = 1.0f / sqrtf(s / (float)D + eps);
            const float4 w4 = reinterpret_cast<const float4*>(weight)[lane];
            x.x *= rr * w4.x; x.y *= rr * w4.y; x.z *= rr * w4.z; x.w *= rr * w4.w;
        }
        if (cos_table) {
            float4 o;
            o.x = __shfl_xor_sync(0xffffffffu, x.x, 16); o.y = __shfl_xor_sync(0xffffffffu, x.y, 16);
            o.z = __shfl_xor_sync(0xffffffffu, x.z, 16); o.w = __shfl_xor_sync(0xffffffffu, x.w, 16);
            if (lane < 16) {        // a' = fma(-b, sin, a cos)
                x.x = fmaf(-o.x, sn.x, x.x * c.x); x.y = fmaf(-o.y, sn.y, x.y * c.y);
                x.z = fmaf(-o.z, sn.z, x.z * c.z); x.w = fmaf(-o.w, sn.w, x.w * c.w);
            } else {                // b' = fma(a, sin, b cos)
                x.x = fmaf(o.x, sn.x, x.x * c.x); x.y = fmaf(o.y, sn.y, x.y * c.y);
                x.z = fmaf(o.z, sn.z, x.z * c.z); x.w = fmaf(o.w, sn.w, x.w * c.w);
            }
        }
        if (is_q) {
            store4(q_out + ((size_t)row * heads + j) * D + 4 * lane, x.x, x.y, x.z, x.w);
        } else {
            const int page = slot / page_size, off = slot % page_size;
            const size_t key_base = ((((size_t)page * 2 + 0) * kv_heads + g) * page_size + off) * D;
            const size_t value_base = ((((size_t)page * 2 + 1) * kv_heads + g) * page_size + off) * D;
            store4(cache + key_base + 4 * lane, x.x, x.y, x.z, x.w);
            store4(cache + value_base + 4 * lane, raw[u].x, raw[u].y, raw[u].z, raw[u].w);
        }
    }
}

template <typename T, int U>
static void launch_head_norm_rope_128(const float* qkv, int qkv_stride, int k_offset, int v_offset, const float* q_weight,
                                      const float* k_weight, float eps, const float* cos_table, const float* sin_table,
                                      const int* positions, const int* slots, void* q_out, void* cache, int rows,
                                      int heads, int kv_heads, int page_size, cudaStream_t stream) {
    const int warps = 4;
    const long long groups = (long long)rows * (heads + kv_heads) / U;
    launch_kernel(head_norm_rope_128_kernel<T, T, U>, dim3((unsigned)((groups + warps - 1) / warps)), dim3(warps * 32), 0,
                  stream, qkv, qkv_stride, k_offset, v_offset, q_weight, k_weight, eps, cos_table, sin_table, positions,
                  slots, (T*)q_out, (T*)cache, rows, heads, kv_heads, page_size);
}

LLMX_EXPORT int llmx_head_norm_rope_kv(const float* qkv, int qkv_stride, int k_offset, int v_offset,
                                       const float* q_weight, const float* k_weight, float eps,
                                       const float* cos_table, const float* sin_table, int rot_half,
                                       const int* positions, const int* slots, void* q_out, int q_dtype, void* cache,
                                       int cache_dtype, int rows, int heads, int kv_heads, int head_dim,
                                       int page_size, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (head_dim <= 0 || rot_half < 0 || 2 * rot_half > head_dim) return LLMX_ERR_BAD_ARGUMENT;
    const int warps = 4;
    const long long items = (long long)rows * (heads + kv_heads);
    const unsigned blocks = (unsigned)((items + warps - 1) / warps);
    const bool fast = q_dtype == cache_dtype && head_dim == 128 && (!cos_table || rot_half == 64) && qkv_stride % 4 == 0 && k_offset % 4 == 0 &&
                      v_offset % 4 == 0 && !((uintptr_t)qkv & 15) && !((uintptr_t)q_out & 15) && !((uintptr_t)cache & 15) &&
                      !((uintptr_t)q_weight & 15) && !((uintptr_t)k_weight & 15) && !((uintptr_t)cos_table & 15) &&
                      !((uintptr_t)sin_table & 15);
    if (fast) {
        // Many rows: two items a warp (measured at 2,048 rows of 48 heads: one 24, two 20.5, four 22 us: more items
        // a warp cost registers, and with them resident warps); few rows: one item a warp keeps more warps busy.
        const int per_row = heads + kv_heads;
        if ((long long)rows * per_row >= (1ll << 31)) return LLMX_ERR_UNSUPPORTED;
        const int u = rows >= 64 && per_row % 2 == 0 ? 2 : 1;
#define LLMX_HNR(T, U) launch_head_norm_rope_128<T, U>(qkv, qkv_stride, k_offset, v_offset, q_weight, k_weight, eps, cos_table, \
                                                       sin_table, positions, slots, q_out, cache, rows, heads, kv_heads, page_size, stream)
        if (q_dtype == LLMX_BF16) {
            if (u == 2) LLMX_HNR(__nv_bfloat16, 2); else LLMX_HNR(__nv_bfloat16, 1);
        } else {
            if (u == 2) LLMX_HNR(float, 2); else LLMX_HNR(float, 1);
        }
#undef LLMX_HNR
        return launch_status();
    }
    const size_t shmem = (size_t)warps * head_dim * sizeof(float);
    // The general form takes queries and cache of different types (bfloat16 products over a float32 cache, or the reverse).
#define LLMX_HNR_ANY(QT, KVT)                                                                                           \
    launch_kernel(head_norm_rope_kernel<QT, KVT>, dim3(blocks), dim3(warps * 32), shmem, stream, qkv, qkv_stride,      \
                  k_offset, v_offset, q_weight, k_weight, eps, cos_table, sin_table, rot_half, positions, slots,       \
                  (QT*)q_out, (KVT*)cache, rows, heads, kv_heads, head_dim, page_size)
    if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) LLMX_HNR_ANY(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) LLMX_HNR_ANY(__nv_bfloat16, float);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) LLMX_HNR_ANY(float, __nv_bfloat16);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_F32) LLMX_HNR_ANY(float, float);
    else return LLMX_ERR_BAD_ARGUMENT;
#undef LLMX_HNR_ANY
    return launch_status();
}

// ---------------------------------------------------------------------------
// SwiGLU: act = silu(g) * u, silu(g) = g / (1 + exp(-g))
// (src/backends/cpu/cpu_backend.hpp:1677; f32.gpu:596-631).  `gu` holds a row's gate
// values then its up values ([rows, 2 * width]).
// ---------------------------------------------------------------------------
template <typename OutT>
__global__ void swiglu_kernel(const float* __restrict__ gu, OutT* __restrict__ act, long long total, int width) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / width;
    const int c = (int)(i % width);
    const float g = gu[r * 2 * width + c], u = gu[r * 2 * width + width + c];
    act[i] = from_float<OutT>(g / (1.0f + expf(-g)) * u);
}

LLMX_EXPORT int llmx_swiglu(const float* gu, void* act, int out_dtype, int rows, int width, cudaStream_t stream) {
    const long long total = (long long)rows * width;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == LLMX_BF16) launch_kernel(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, gu, (__nv_bfloat16*)act, total, width);
    else launch_kernel(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, gu, (float*)act, total, width);
    return launch_status();
}

// ---------------------------------------------------------------------------
// Embedding with a factor: x[r, :] = table[ids[r], :] * scale, the product made in 32-bit.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_scaled_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ x,
                                    int width, int table_rows, float scale) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int id = ids[r];
    float* dst = x + (size_t)r * width;
    if (id < 0 || id >= table_rows) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = 0.0f;
        return;
    }
    const T* src = table + (size_t)id * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = to_float(src[i]) * scale;
}

LLMX_EXPORT int llmx_embed_scaled(const void* table, int table_dtype, const int* ids, float* x, int rows, int width,
                                  int table_rows, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (table_dtype == LLMX_BF16)
        launch_kernel(embed_scaled_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, (const __nv_bfloat16*)table, ids, x, width, table_rows, scale);
    else
        launch_kernel(embed_scaled_kernel<float>, dim3(rows), dim3(256), 0, stream, (const float*)table, ids, x, width, table_rows, scale);
    return launch_status();
}

// x[i] *= s over a flat float buffer (a model whose logits carry a factor).
__global__ void scale_kernel(float* __restrict__ x, long long n, float s) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= s;
}

LLMX_EXPORT int llmx_scale(float* x, long long n, float s, cudaStream_t stream) {
    if (n <= 0) return 0;
    launch_kernel(scale_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, s);
    return launch_status();
}

// ---------------------------------------------------------------------------
// LayerNorm with a weight and no bias: m = mean x; v = mean (x - m)^2; y_i = (x_i - m) / sqrt(v + eps) * w_i.
// Two passes over the row's values (kept in registers when the row fits, else read again): the variance is the
// mean of squared deviations, not a difference of means.  `row_index` as in RMSNorm.
// ---------------------------------------------------------------------------
constexpr int LN_MAX = 16;   // values a thread keeps (rows up to 16 * 256 wide); wider rows are read three times

// `zero` (optional): a float buffer of `zero_count` values (a multiple of 4, 16-byte aligned) that the launch clears with
// blocks of its own (those beyond `rows`): the outputs of products that follow and add their pieces with atomics.
template <typename OutT>
__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ in_bias, const float* __restrict__ w,
                                 const float* __restrict__ b, OutT* __restrict__ y, float* __restrict__ add_to, float mult,
                                 const int* __restrict__ row_index, int rows, int width, float eps,
                                 float* __restrict__ zero, long long zero_count) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    if (r >= rows) {
        float4* z = reinterpret_cast<float4*>(zero);
        const long long n4 = zero_count >> 2;
        const long long blocks = gridDim.x - rows;
        for (long long i = (long long)(r - rows) * blockDim.x + threadIdx.x; i < n4; i += blocks * blockDim.x)
            z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    const float* src = x + (size_t)(row_index ? row_index[r] : r) * width;
    OutT* dst = y + (size_t)r * width;
    float* sum = add_to ? add_to + (size_t)r * width : nullptr;
    const float n = (float)width;            // divided by, not multiplied with a rounded 1 / n: a row of equal values has deviations of exactly 0
    if (width <= LN_MAX * (int)blockDim.x) {
        float v[LN_MAX];
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < LN_MAX; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            v[k] = i < width ? src[i] + (in_bias ? in_bias[i] : 0.0f) : 0.0f;
            s += v[k];
        }
        const float mean = block_sum(s, scratch) / n;
        float q = 0.0f;
#pragma unroll
        for (int k = 0; k < LN_MAX; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            const float d = i < width ? v[k] - mean : 0.0f;
            v[k] = d;
            q = fmaf(d, d, q);
        }
        const float rr = 1.0f / sqrtf(block_sum(q, scratch) / n + eps);
#pragma unroll
        for (int k = 0; k < LN_MAX; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < width) {
                const float o = v[k] * rr * w[i] + (b ? b[i] : 0.0f);
                if (sum) sum[i] = fmaf(mult, o, sum[i]);
                else dst[i] = from_float<OutT>(o);
            }
        }
        return;
    }
    float s = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) s += src[i] + (in_bias ? in_bias[i] : 0.0f);
    const float mean = block_sum(s, scratch) / n;
    float q = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float d = src[i] + (in_bias ? in_bias[i] : 0.0f) - mean;
        q = fmaf(d, d, q);
    }
    const float rr = 1.0f / sqrtf(block_sum(q, scratch) / n + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float o = (src[i] + (in_bias ? in_bias[i] : 0.0f) - mean) * rr * w[i] + (b ? b[i] : 0.0f);
        if (sum) sum[i] = fmaf(mult, o, sum[i]);
        else dst[i] = from_float<OutT>(o);
    }
}

// The centred norm in its general form: y = ((x + in_bias) - mean) / sqrt(var + eps) * w + b.  `in_bias` and `b` may be
// null.  With `add_to` (float [rows, width]) nothing is written to `y`; instead add_to += mult * y in 32-bit: the norm
// after a sublayer and the sublayer's weighted entry into the residual stream in one pass.
LLMX_EXPORT int llmx_layernorm_affine(const float* x, const float* in_bias, const float* w, const float* b, void* y, int out_dtype,
                                      float* add_to, float mult, const int* row_index, int rows, int width, float eps,
                                      float* zero, long long zero_count, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || (!y && !add_to)) return LLMX_ERR_BAD_ARGUMENT;
    if (zero && (zero_count % 4 || ((uintptr_t)zero & 15))) return LLMX_ERR_BAD_ARGUMENT;
    // The block width follows the row width alone, so a row's sums have one order whatever the batch.
    int threads = (width + LN_MAX - 1) / LN_MAX;
    threads = (threads + 31) / 32 * 32;
    threads = threads < 64 ? 64 : threads > 256 ? 256 : threads;
    // Clearing: blocks of their own, each about four 16-byte stores a thread, at most 1,024 of them.
    long long zero_blocks = zero ? (zero_count / 4 + 4 * threads - 1) / (4 * threads) : 0;
    zero_blocks = zero_blocks > 1024 ? 1024 : zero_blocks;
    const dim3 grid((unsigned)(rows + zero_blocks));
    if (out_dtype == LLMX_BF16 && !add_to)
        launch_kernel(layernorm_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, x, in_bias, w, b, (__nv_bfloat16*)y, add_to, mult,
                      row_index, rows, width, eps, zero, zero_count);
    else
        launch_kernel(layernorm_kernel<float>, grid, dim3(threads), 0, stream, x, in_bias, w, b, (float*)y, add_to, mult, row_index, rows,
                      width, eps, zero, zero_count);
    return launch_status();
}

LLMX_EXPORT int llmx_layernorm(const float* x, const float* w, void* y, int out_dtype, const int* row_index, int rows,
                               int width, float eps, float* zero, long long zero_count, cudaStream_t stream) {
    return llmx_layernorm_affine(x, nullptr, w, nullptr, y, out_dtype, nullptr, 0.0f, row_index, rows, width, eps, zero, zero_count,
                                 stream);
}

// ---------------------------------------------------------------------------
// A gate on rows: o[r, c] *= sigmoid(gate[r, c]) in 32-bit, o of the path's type in place; `gate` is float and has a
// row stride of its own (it lies inside a wider product's output).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ o, const float* __restrict__ gate, int gate_stride, int width, long long total) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float g = gate[(i / width) * gate_stride + (i % width)];
    o[i] = from_float<T>(to_float(o[i]) / (1.0f + expf(-g)));
}

LLMX_EXPORT int llmx_sigmoid_gate(void* o, int dtype, const float* gate, int gate_stride, int rows, int width, cudaStream_t stream) {
    const long long total = (long long)rows * width;
    if (total <= 0) return 0;
    if (gate_stride < width) return LLMX_ERR_BAD_ARGUMENT;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == LLMX_BF16) launch_kernel(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)o, gate, gate_stride, width, total);
    else launch_kernel(sigmoid_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)o, gate, gate_stride, width, total);
    return launch_status();
}

// ---------------------------------------------------------------------------
// x[r, c] += bias[c]: the bias of a product whose result was added into x.
// ---------------------------------------------------------------------------
__global__ void add_bias_kernel(float* __restrict__ x, const float* __restrict__ bias, int width, long long total) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] += bias[i % width];
}

LLMX_EXPORT int llmx_add_bias(float* x, const float* bias, int rows, int width, cudaStream_t stream) {
    const long long total = (long long)rows * width;
    if (total <= 0) return 0;
    launch_kernel(add_bias_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, bias, width, total);
    return launch_status();
}

// ---------------------------------------------------------------------------
// Clamped gated unit: g = min(gate, limit); u = clamp(up, -limit, limit); act = g * sigmoid(alpha * g) * (u + 1).
// `gu` holds a row's gate values then its up values ([rows, 2 * width]); 32-bit arithmetic.
// ---------------------------------------------------------------------------
template <typename OutT>
__global__ void clamped_glu_kernel(const float* __restrict__ gu, OutT* __restrict__ act, long long total, int width,
                                   float limit, float alpha) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / width;
    const int c = (int)(i % width);
    const float g = fminf(gu[r * 2 * width + c], limit);
    const float u = fminf(fmaxf(gu[r * 2 * width + width + c], -limit), limit);
    act[i] = from_float<OutT>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
}

LLMX_EXPORT int llmx_clamped_glu(const float* gu, void* act, int out_dtype, int rows, int width, float limit, float alpha,
                                 cudaStream_t stream) {
    const long long total = (long long)rows * width;
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == LLMX_BF16) launch_kernel(clamped_glu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, gu, (__nv_bfloat16*)act, total, width, limit, alpha);
    else launch_kernel(clamped_glu_kernel<float>, dim3(blocks), dim3(256), 0, stream, gu, (float*)act, total, width, limit, alpha);
    return launch_status();
}

// ---------------------------------------------------------------------------
// In-place activation of a column range of a float matrix: x[r, c0 .. c0 + n) = silu(x).  (A mixer whose
// projections pass an activation before a recurrence reads them.)
// ---------------------------------------------------------------------------
__global__ void silu_columns_kernel(float* __restrict__ x, int stride, int c0, int n, long long total) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float* p = x + (i / n) * stride + c0 + (i % n);
    const float v = *p;
    *p = v / (1.0f + expf(-v));
}

LLMX_EXPORT int llmx_silu_columns(float* x, int rows, int stride, int c0, int n, cudaStream_t stream) {
    const long long total = (long long)rows * n;
    if (total <= 0) return 0;
    if (c0 < 0 || c0 + n > stride) return LLMX_ERR_BAD_ARGUMENT;
    launch_kernel(silu_columns_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, stride, c0, n, total);
    return launch_status();
}

// ---------------------------------------------------------------------------
// RMS norm over groups of a row, times a gate: for group j of `group` values,
//   y = o / sqrt(mean_group(o^2) + eps) * w[(j * group + i) % w_len] * act(gate),  act = sigmoid (0) or silu (1).
// One group is the whole row (a norm over all heads together, weight as long as the row) or one head (weight as
// long as a head and shared by the heads).  `gate` has its own row stride (it lies inside a wider product's output).
// One block per (row, group); the block width follows the group width alone.
// ---------------------------------------------------------------------------
template <typename OutT>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_stride,
                                     const float* __restrict__ w, int w_len, OutT* __restrict__ y, int groups, int group,
                                     float eps, int gate_kind, int gate_first) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x, j = blockIdx.y;
    const size_t base = ((size_t)r * groups + j) * group;
    const float* src = o + base;
    const float* gsrc = gate + (size_t)r * gate_stride + (size_t)j * group;
    auto act = [&](float g) {
        const float sg = 1.0f / (1.0f + expf(-g));
        return gate_kind == 0 ? sg : g * sg;
    };
    float s = 0.0f;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const float x = gate_first ? src[i] * act(gsrc[i]) : src[i];
        s = fmaf(x, x, s);
    }
    const float rr = 1.0f / sqrtf(block_sum(s, scratch) / (float)group + eps);
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        const float a = act(gsrc[i]);
        const float wi = w[(j * group + i) % w_len];
        y[base + i] = from_float<OutT>(gate_first ? (src[i] * a) * rr * wi : src[i] * rr * wi * a);
    }
}

// `gate_first` 0: y = o / rms(o) * w * act(gate).  1: the gate comes before the norm: z = o * act(gate), y = z / rms(z) * w.
LLMX_EXPORT int llmx_gated_rmsnorm(const float* o, const float* gate, int gate_stride, const float* w, int w_len, void* y,
                                   int out_dtype, int rows, int groups, int group, float eps, int gate_kind, int gate_first,
                                   cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (groups <= 0 || group <= 0 || w_len <= 0 || groups > 65535 || (gate_kind != 0 && gate_kind != 1)) return LLMX_ERR_BAD_ARGUMENT;
    int threads = (group + 3) / 4;
    threads = (threads + 31) / 32 * 32;
    threads = threads < 32 ? 32 : threads > 256 ? 256 : threads;
    if (out_dtype == LLMX_BF16)
        launch_kernel(gated_rmsnorm_kernel<__nv_bfloat16>, dim3(rows, groups), dim3(threads), 0, stream, o, gate, gate_stride, w, w_len, (__nv_bfloat16*)y, groups, group, eps, gate_kind, gate_first);
    else
        launch_kernel(gated_rmsnorm_kernel<float>, dim3(rows, groups), dim3(threads), 0, stream, o, gate, gate_stride, w, w_len, (float*)y, groups, group, eps, gate_kind, gate_first);
    return launch_status();
}

// ---------------------------------------------------------------------------
// Two mixers side by side: x[r] += factor * (a[r] / rms(a[r]) * wa + b[r] / rms(b[r]) * wb), each side normed over
// the whole row with a plain weight of its own.  One block a row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
pair_norm_add_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ wa,
                     const float* __restrict__ wb, float* __restrict__ x, int width, float eps, float factor) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * width;
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        sa = fmaf(a[base + i], a[base + i], sa);
        sb = fmaf(b[base + i], b[base + i], sb);
    }
    const float ra = 1.0f / sqrtf(block_sum(sa, scratch) / (float)width + eps);
    const float rb = 1.0f / sqrtf(block_sum(sb, scratch) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        x[base + i] += factor * (a[base + i] * ra * wa[i] + b[base + i] * rb * wb[i]);
}

LLMX_EXPORT int llmx_pair_norm_add(const float* a, const float* b, const float* wa, const float* wb, float* x, int rows,
                                   int width, float eps, float factor, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return LLMX_ERR_BAD_ARGUMENT;
    launch_kernel(pair_norm_add_kernel, dim3(rows), dim3(256), 0, stream, a, b, wa, wb, x, width, eps, factor);
    return launch_status();
}

// x[i] += y[i] over flat float buffers (a model that adds its embedding output to the stream again).
__global__ void add_kernel(float* __restrict__ x, const float* __restrict__ y, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += y[i];
}

LLMX_EXPORT int llmx_add(float* x, const float* y, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    launch_kernel(add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, y, n);
    return launch_status();
}

// ---------------------------------------------------------------------------
// RMS norm in groups, with the mixer's input filter in the same launch.
//   h[c]  = x[c] / sqrt(mean(part(c)^2) + eps) * w[c]        the row in `groups` equal consecutive parts, each with its own
//                                                            root mean square
//   hm[c] = h[c] + sum_j taps_w[j, c] h_(t - taps + 1 + j)[c]  a causal filter over the request's rows, per channel; the last
//                                                            tap lies on the row itself, rows before the request's first
//                                                            token are zeros
// A block makes one row.  The filter needs the normed values of the taps - 1 rows before: those of the same step are made
// again from x (the same arithmetic, so the same bits), those of earlier steps lie in the request's state slot, which
// holds its last taps - 1 normed rows ([taps - 1][width] floats at `state_off`); the step's last ones go to the slot the
// step writes.  One warp makes the sum of squares of one (row, part), lanes in a fixed order.  Blocks beyond the rows:
// one a request, copying what the new state keeps of the old one when the step brings fewer than taps - 1 rows; then
// blocks that clear `zero`.  With `row_index` the rows are gathered (no filter then).
struct GroupNormConv {
    const float* x;
    const float* w;
    int width, groups;
    float eps;
    const int* row_index;
    int rows;
    const float* taps_w;
    int taps;
    float* state;
    long long slot_floats, state_off;
    const int *row_request, *row_start, *row_count, *history, *slot_in, *slot_out;
    int requests;
    float* zero;
    long long zero_count;
};

template <int VEC> __device__ __forceinline__ void load_run(const float* p, float (&v)[VEC]) {
    if constexpr (VEC == 4) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    } else {
        v[0] = p[0];
    }
}
template <typename T, int VEC> __device__ __forceinline__ void store_run(T* p, const float (&v)[VEC]) {
    if constexpr (VEC == 4) store4(p, v[0], v[1], v[2], v[3]);
    else p[0] = from_float<T>(v[0]);
}

template <typename OutT, int VEC>
__global__ void __launch_bounds__(256)
group_norm_conv_kernel(GroupNormConv a, OutT* __restrict__ h, OutT* __restrict__ hm) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float gnc_rstd[];                    // [taps][groups]
    const int keep = a.taps - 1, width = a.width;
    const int state_blocks = keep > 0 ? a.requests : 0;
    if ((int)blockIdx.x >= a.rows + state_blocks) {
        float4* z = reinterpret_cast<float4*>(a.zero);
        const long long n4 = a.zero_count >> 2;
        const long long blocks = gridDim.x - a.rows - state_blocks;
        for (long long i = (long long)(blockIdx.x - a.rows - state_blocks) * blockDim.x + threadIdx.x; i < n4; i += blocks * blockDim.x)
            z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        return;
    }
    if ((int)blockIdx.x >= a.rows) {
        const int q = blockIdx.x - a.rows;
        const int n = a.row_count[q], hist = a.history[q];
        if (n <= 0 || n >= keep) return;
        const float* old = a.state + (size_t)a.slot_in[q] * a.slot_floats + a.state_off;
        float* fresh = a.state + (size_t)a.slot_out[q] * a.slot_floats + a.state_off;
        for (int s = 0; s < keep - n; ++s) {
            const int ii = n - keep + s;                    // < 0: a row of an earlier step, or before the request
            for (int c = threadIdx.x; c < width; c += blockDim.x)
                fresh[(size_t)s * width + c] = hist + ii >= 0 ? old[(size_t)(keep + ii) * width + c] : 0.0f;
        }
        return;
    }
    const int r = blockIdx.x;
    const int src_row = a.row_index ? a.row_index[r] : r;
    int first = 0, i0 = 0, hist = 0, n = 0;
    const float* old = nullptr;
    float* fresh = nullptr;
    if (keep > 0) {
        const int q = a.row_request[r];
        first = a.row_start[q];
        i0 = r - first;
        hist = a.history[q];
        n = a.row_count[q];
        old = a.state + (size_t)a.slot_in[q] * a.slot_floats + a.state_off;
        fresh = a.state + (size_t)a.slot_out[q] * a.slot_floats + a.state_off;
    }
    const int part = width / a.groups;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const bool vec = (part & 3) == 0 && !((uintptr_t)a.x & 15);             // 16-byte pieces (one order of sums a width)
    for (int item = warp; item < a.taps * a.groups; item += warps) {
        const int j = item / a.groups, g = item - j * a.groups;
        const int ii = i0 - keep + j;
        if (j < keep && ii < 0) continue;                    // not a row of this step
        const float* xr = a.x + (size_t)(j == keep ? src_row : first + ii) * width + (size_t)g * part;
        float ss = 0.0f;
        if (vec) {
            for (int c = 4 * lane; c < part; c += 128) {
                const float4 v = *reinterpret_cast<const float4*>(xr + c);
                ss = fmaf(v.x, v.x, ss);
                ss = fmaf(v.y, v.y, ss);
                ss = fmaf(v.z, v.z, ss);
                ss = fmaf(v.w, v.w, ss);
            }
        } else
            for (int c = lane; c < part; c += 32) ss = fmaf(xr[c], xr[c], ss);
        ss = warp_sum(ss);
        if (lane == 0) gnc_rstd[item] = 1.0f / sqrtf(ss / (float)part + a.eps);
    }
    __syncthreads();
    const float* xrow = a.x + (size_t)src_row * width;
    const int s_new = i0 - (n - keep);                       // the place of this row in the state the step leaves
    // VEC channels a thread and turn (4 where rows, weights and outputs can be read and written in 16-byte pieces: the
    // channels of a piece lie in one part).
    for (int c = VEC * threadIdx.x; c < width; c += VEC * blockDim.x) {
        const int g = c / part;
        float xv[VEC], wc[VEC], cur[VEC];
        load_run<VEC>(xrow + c, xv);
        load_run<VEC>(a.w + c, wc);
        const float rr = gnc_rstd[keep * a.groups + g];
#pragma unroll
        for (int i = 0; i < VEC; ++i) cur[i] = xv[i] * rr * wc[i];
        store_run<OutT, VEC>(h + (size_t)r * width + c, cur);
        if (a.taps_w != nullptr) {
            float acc[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
            for (int j = 0; j < keep; ++j) {
                const int ii = i0 - keep + j;
                float v[VEC];
                if (ii >= 0) {
                    load_run<VEC>(a.x + (size_t)(first + ii) * width + c, v);
                    const float rj = gnc_rstd[j * a.groups + g];
#pragma unroll
                    for (int i = 0; i < VEC; ++i) v[i] = v[i] * rj * wc[i];
                } else if (hist + ii >= 0) {
                    load_run<VEC>(old + (size_t)(keep + ii) * width + c, v);
                } else {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) v[i] = 0.0f;
                }
                {
                    float tw[VEC];
                    load_run<VEC>(a.taps_w + (size_t)j * width + c, tw);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[i] = fmaf(tw[i], v[i], acc[i]);
                }
            }
            float out[VEC], tw[VEC];
            load_run<VEC>(a.taps_w + (size_t)keep * width + c, tw);
#pragma unroll
            for (int i = 0; i < VEC; ++i) out[i] = cur[i] + fmaf(tw[i], cur[i], acc[i]);
            store_run<OutT, VEC>(hm + (size_t)r * width + c, out);
            if (keep > 0 && s_new >= 0) store_run<float, VEC>(fresh + (size_t)s_new * width + c, cur);
        }
    }
}

// x float32 [*, width]; w float32 [width]; h (and hm, with a filter) [rows, width] of `out_dtype`; taps_w float32 [taps, width]
// (tap by tap, so that a tap of neighbouring channels is one piece) or null (no filter; a filter of one tap keeps no state); state float32 [slots, slot_floats]; the step's row ranges, histories and slots as a step gives them;
// zero: a float buffer of zero_count values (a multiple of 4, 16-byte aligned) cleared in passing, or null.
LLMX_EXPORT int llmx_group_norm_conv(const float* x, const float* w, int width, int groups, float eps, const int* row_index,
                                     int rows, void* h, void* hm, int out_dtype, const float* taps_w, int taps, float* state,
                                     long long slot_floats, long long state_off, const int* row_request, const int* row_start,
                                     const int* row_count, const int* history, const int* slot_in, const int* slot_out,
                                     int requests, float* zero, long long zero_count, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || groups <= 0 || width % groups || taps < 1 || taps * groups > 8192) return LLMX_ERR_BAD_ARGUMENT;
    if (zero && (zero_count % 4 || ((uintptr_t)zero & 15))) return LLMX_ERR_BAD_ARGUMENT;
    if ((taps_w != nullptr) != (hm != nullptr) || (taps > 1 && taps_w == nullptr)) return LLMX_ERR_BAD_ARGUMENT;
    if (taps > 1 && (state == nullptr || row_index != nullptr || row_request == nullptr ||
                     state_off + (long long)(taps - 1) * width > slot_floats))
        return LLMX_ERR_BAD_ARGUMENT;
    GroupNormConv a{x, w, width, groups, eps, row_index, rows, taps_w, taps, state, slot_floats, state_off, row_request, row_start,
                    row_count, history, slot_in, slot_out, requests, zero, zero_count};
    long long zero_blocks = zero ? (zero_count / 4 + 4 * 256 - 1) / (4 * 256) : 0;
    zero_blocks = zero_blocks > 1024 ? 1024 : zero_blocks;
    const dim3 grid((unsigned)(rows + (taps > 1 ? requests : 0) + zero_blocks));
    const size_t smem = (size_t)taps * groups * sizeof(float);
    // 16-byte pieces where every row, weight, output and state row starts on one and a piece lies within one part.
    const bool vec = (width / groups) % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)w & 15) && !((uintptr_t)taps_w & 15) && !((uintptr_t)h & 15) && !((uintptr_t)hm & 15) &&
                     (taps == 1 || (!((uintptr_t)state & 15) && slot_floats % 4 == 0 && state_off % 4 == 0));
    if (out_dtype == LLMX_BF16 && vec)
        launch_kernel(group_norm_conv_kernel<__nv_bfloat16, 4>, grid, dim3(256), smem, stream, a, (__nv_bfloat16*)h, (__nv_bfloat16*)hm);
    else if (out_dtype == LLMX_BF16)
        launch_kernel(group_norm_conv_kernel<__nv_bfloat16, 1>, grid, dim3(256), smem, stream, a, (__nv_bfloat16*)h, (__nv_bfloat16*)hm);
    else if (out_dtype == LLMX_F32 && vec)
        launch_kernel(group_norm_conv_kernel<float, 4>, grid, dim3(256), smem, stream, a, (float*)h, (float*)hm);
    else if (out_dtype == LLMX_F32)
        launch_kernel(group_norm_conv_kernel<float, 1>, grid, dim3(256), smem, stream, a, (float*)h, (float*)hm);
    else
        return LLMX_ERR_UNSUPPORTED;
    return launch_status();
}

// ---------------------------------------------------------------------------
// Token embedding times a factor, plus a row of a second table chosen by the pair (token before, token):
//   x[r] = table[id] * scale + pair_table[(before * mul_prev + id * mul_cur) mod buckets]
// and row `buckets` of the pair table for a request's first token.  The token before a step's first row is the
// request's state (one int32 in its slot); the step's last token goes to the slot the step writes (blocks beyond the rows,
// one a request).
template <typename T>
__global__ void embed_pairs_kernel(const T* __restrict__ table, const T* __restrict__ pair_table, const int* __restrict__ ids,
                                   float* __restrict__ x, int rows, int width, int vocab, float scale, int buckets,
                                   long long mul_prev, long long mul_cur, const int* __restrict__ row_request,
                                   const int* __restrict__ row_start, const int* __restrict__ row_count,
                                   const int* __restrict__ history, int* __restrict__ state, long long slot_ints,
                                   const int* __restrict__ slot_in, const int* __restrict__ slot_out) {
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x >= rows) {
        const int q = blockIdx.x - rows;
        const int n = row_count[q];
        if (threadIdx.x == 0 && n > 0) state[(size_t)slot_out[q] * slot_ints] = ids[row_start[q] + n - 1];
        return;
    }
    const int r = blockIdx.x;
    const int q = row_request[r];
    const int i0 = r - row_start[q];
    int id = ids[r];
    id = id < 0 ? 0 : id >= vocab ? vocab - 1 : id;
    int before = -1;
    if (i0 > 0) before = ids[r - 1];
    else if (history[q] > 0) before = state[(size_t)slot_in[q] * slot_ints];
    const long long pair = before < 0 ? (long long)buckets : ((long long)before * mul_prev + (long long)id * mul_cur) % (long long)buckets;
    const T* src = table + (size_t)id * width;
    const T* psrc = pair_table + (size_t)pair * width;
    float* dst = x + (size_t)r * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = fmaf(to_float(src[c]), scale, to_float(psrc[c]));
}

LLMX_EXPORT int llmx_embed_pairs(const void* table, const void* pair_table, int table_dtype, const int* ids, float* x, int rows,
                                 int width, int vocab, float scale, int buckets, long long mul_prev, long long mul_cur,
                                 const int* row_request, const int* row_start, const int* row_count, const int* history,
                                 int* state, long long slot_ints, const int* slot_in, const int* slot_out, int requests,
                                 cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (buckets <= 0 || width <= 0 || vocab <= 0 || state == nullptr || slot_ints <= 0) return LLMX_ERR_BAD_ARGUMENT;
    const dim3 grid(rows + requests);
    if (table_dtype == LLMX_BF16)
        launch_kernel(embed_pairs_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pair_table,
                      ids, x, rows, width, vocab, scale, buckets, mul_prev, mul_cur, row_request, row_start, row_count, history, state,
                      slot_ints, slot_in, slot_out);
    else if (table_dtype == LLMX_F32)
        launch_kernel(embed_pairs_kernel<float>, grid, dim3(256), 0, stream, (const float*)table, (const float*)pair_table, ids, x, rows,
                      width, vocab, scale, buckets, mul_prev, mul_cur, row_request, row_start, row_count, history, state, slot_ints,
                      slot_in, slot_out);
    else
        return LLMX_ERR_UNSUPPORTED;
    return launch_status();
}

// ---------------------------------------------------------------------------
// x[r, c] += factor * row_factor[r] * y[r, c]   (row_factor null: 1), float32.
__global__ void add_rows_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ row_factor,
                                float factor, int width, long long total) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float f = row_factor ? factor * row_factor[i / width] : factor;
    x[i] = fmaf(f, y[i], x[i]);
}

__global__ void add_rows_vec_kernel(float4* __restrict__ x, const float4* __restrict__ y, const float* __restrict__ row_factor,
                                    float factor, int width4, long long total4) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const float f = row_factor ? factor * row_factor[i / width4] : factor;
    float4 a = x[i];
    const float4 b = y[i];
    a.x = fmaf(f, b.x, a.x);
    a.y = fmaf(f, b.y, a.y);
    a.z = fmaf(f, b.z, a.z);
    a.w = fmaf(f, b.w, a.w);
    x[i] = a;
}

LLMX_EXPORT int llmx_add_rows(float* x, const float* y, const float* row_factor, float factor, int rows, int width,
                              cudaStream_t stream) {
    if (rows <= 0) return 0;
    const long long total = (long long)rows * width;
    if (width % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)y & 15)) {
        launch_kernel(add_rows_vec_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream, (float4*)x, (const float4*)y,
                      row_factor, factor, width / 4, total / 4);
        return launch_status();
    }
    launch_kernel(add_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, y, row_factor, factor, width, total);
    return launch_status();
}

// x <- cap * tanh(x / cap), float32.
__global__ void softcap_kernel(float* __restrict__ x, long long n, float cap) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

LLMX_EXPORT int llmx_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.0f)) return LLMX_ERR_BAD_ARGUMENT;
    launch_kernel(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, n, cap);
    return launch_status();
}
