// Softmax attention whose keys and values have widths of their own, over pages that hold one [key ; value] row per
// token and key/value head: cache [pages, 1, kv_heads, page_size, D + V].
//
// Two kernels.  `llmx_qk_norm_rope_write` finishes the rows of the stacked q/k/v product: an RMS norm per head with a
// weight of D values shared by the heads (optional), a rotation of the first 2 * rot_half values of every query and
// key head (value i pairs with value i + rot_half; the angle is position * freq[i], made in 32-bit here, so there is
// no table whose length bounds the context), queries to `q_out`, keys and values to the row's cache slot.
// Designs vary the softmax (`AttnExtras`: a cap on the scores, a sink in the denominator, values rotated by position).
// `llmx_attention_split` is the plain form of the attention: one block per (row, head); a row at position p reads the
// keys lo..p of its own request, where lo is the larger of p - window + 1 (window > 0) and the start of p's chunk,
// floor(p / chunk) * chunk (chunk > 0: positions are counted from the start of the request, so chunks do not move
// with the way a prompt was cut); query head h reads key/value head h / (heads / kv_heads).
//   s_t = dot(q, k_t) * scale;  m = max s;  e_t = exp(s_t - m);  l = sum e_t;  o = sum_t (e_t / l) v_t
// in the online form, 32-bit.  Each warp walks every fourth key in increasing order and the four partial states are
// merged in warp order, so the order of a row's sums depends on its own keys only.
#include "common.cuh"
#include <math.h>
#include <algorithm>

namespace {
constexpr int WARPS = 4;
constexpr int MAX_PER_LANE = 16;  // key and value widths up to 512

template <typename QT, typename KVT>
__global__ void __launch_bounds__(128)
qk_write_kernel(const float* __restrict__ proj, int stride, const float* __restrict__ q_weight,
                const float* __restrict__ k_weight, float eps, const float* __restrict__ freq, int rot_half,
                const int* __restrict__ positions, const int* __restrict__ slots, QT* __restrict__ q_out,
                KVT* __restrict__ cache, int heads, int kv_heads, int D, int V, int page_size) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const float pos = (float)positions[row];
    const int slot = slots[row];
    const float* src = proj + (size_t)row * stride;
    const int v_off = (heads + kv_heads) * D;
    for (int item = warp; item < heads + kv_heads; item += warps) {
        const bool is_q = item < heads;
        const float* x = src + (size_t)item * D;                     // q heads, then k heads, lie one after the other
        const float* w = is_q ? q_weight : k_weight;
        float val[MAX_PER_LANE];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            val[i] = d < D ? x[d] : 0.0f;
            ss = fmaf(val[i], val[i], ss);
        }
        QT* qdst = is_q ? q_out + ((size_t)row * heads + item) * D : nullptr;
        KVT* kdst = nullptr;
        if (!is_q) {
            if (slot < 0) continue;                                  // a row whose cache write is skipped
            const int g = item - heads;
            kdst = cache + (((size_t)(slot / page_size) * kv_heads + g) * page_size + slot % page_size) * (size_t)(D + V);
        }
        // A rotated value needs its partner, which another lane holds: each lane reads the partner from the input again
        // and norms it with the head's factor (through shared memory would cost a barrier a head).
        float rr = 1.0f;
        if (w != nullptr) rr = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d >= D) continue;
            float out = w != nullptr ? val[i] * rr * w[d] : val[i];
            if (d < 2 * rot_half) {
                const bool low = d < rot_half;
                const int fi = low ? d : d - rot_half;
                const int pd = low ? d + rot_half : d - rot_half;
                float partner = x[pd];
                if (w != nullptr) partner = partner * rr * w[pd];
                float s, c;
                sincosf(pos * freq[fi], &s, &c);
                out = low ? out * c - partner * s : out * c + partner * s;
            }
            if (is_q) qdst[d] = from_float<QT>(out);
            else kdst[d] = from_float<KVT>(out);
        }
        if (!is_q) {
            const float* vsrc = src + v_off + (size_t)(item - heads) * V;
            for (int d = lane; d < V; d += 32) kdst[D + d] = from_float<KVT>(vsrc[d]);
        }
    }
}

// The general finishing of the rows of a q/k/v product, for designs that put more between the product and the attention:
//   u = proj + bias                                   (bias may be null)
//   y[t] = sum_j taps_w[c, j] u[t - taps + 1 + j]      a short causal filter per channel, zeros before the request's first
//                                                     token; inputs of earlier steps come from the request's state slot,
//                                                     which holds the last taps - 1 values of u ([taps - 1][channels] at
//                                                     `conv_off`); the step's last ones go to the slot the step writes
//   q, k: a norm per head (RMS over D, weights of D values or none) before the rotation (norm 1) or after it (norm 2), or
//         one RMS norm over all of a row's queries and one over all of its keys, before they are split into heads and
//         rotated, with weights of heads * D and kv_heads * D values (norm 3),
//         a rotation of pair i < rot_pairs by position * freq[i]: the pair is (i, i + rot_pairs), or with `neighbours`
//         (2i, 2i + 1)
//   q -> q_out, [k ; v] -> the row's cache slot (kv_heads 0: the rows hold queries only, another layer's keys are read)
// A row's heads are spread over the blocks (x, 0..gridDim.y - 1), a warp per head; blocks whose x lies beyond the rows write
// the requests' new filter inputs, the channels spread likewise.
struct QkvFinish {
    const float* proj;
    int stride;
    const float* bias;
    const float* taps_w;
    int taps;
    float* state;
    long long slot_floats, conv_off;
    const int *row_request, *row_start, *row_count, *history, *slot_in, *slot_out;
    const float *q_weight, *k_weight;
    int norm;
    float eps;
    const float* freq;
    int rot_pairs, neighbours;
    const int *positions, *slots;
    int heads, kv_heads, D, V, page_size, rows;
    int planes;   // 1: a slot holds [key ; value] in one row of D + V; 2: keys and values in planes of their own (D = V)
    float rot_mag;        // a factor on the cosines and sines of the q/k rotation
    const float* vfreq;   // [V / 2] or null: values are rotated by their position over all of V, in the q/k pairing
};

template <typename QT, typename KVT>
__global__ void __launch_bounds__(128)
qkv_finish_kernel(QkvFinish a, QT* __restrict__ q_out, KVT* __restrict__ cache) {
    pdl_trigger();
    pdl_wait();
    __shared__ float stage[4][32 * MAX_PER_LANE];
    __shared__ float turn[2][16 * MAX_PER_LANE];
    const int keep = a.taps - 1;
    const int D = a.D, V = a.V;
    const int channels = (a.heads + a.kv_heads) * D + a.kv_heads * V;
    if ((int)blockIdx.x >= a.rows) {
        // The filter's inputs a later step needs: the last `keep` values of u of the request, from this step's rows or,
        // when the step brings fewer, from the slot read (the slot written is another one).
        const int r = blockIdx.x - a.rows;
        const int n = a.row_count[r], a0 = a.row_start[r], hist = a.history[r];
        if (n <= 0) return;
        const float* old = a.state + (size_t)a.slot_in[r] * a.slot_floats + a.conv_off;
        float* fresh = a.state + (size_t)a.slot_out[r] * a.slot_floats + a.conv_off;
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x)
            for (int s = 0; s < keep; ++s) {
                const int ii = n - keep + s;
                float x = 0.0f;
                if (ii >= 0) x = a.proj[(size_t)(a0 + ii) * a.stride + c] + (a.bias ? a.bias[c] : 0.0f);
                else if (hist + ii >= 0) x = old[(size_t)(keep + ii) * channels + c];
                fresh[(size_t)s * channels + c] = x;
            }
        return;
    }
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int r = a.row_request[row];
    const int first = a.row_start[r], i0 = row - first, hist = a.history[r];
    const float* old = keep > 0 ? a.state + (size_t)a.slot_in[r] * a.slot_floats + a.conv_off : nullptr;
    const float pos = (float)a.positions[row];
    const int slot = a.slots ? a.slots[row] : -1;                  // rows of queries alone have no cache slot
    auto filtered = [&](int c) -> float {
        const float b = a.bias ? a.bias[c] : 0.0f;
        if (a.taps_w == nullptr) return a.proj[(size_t)row * a.stride + c] + b;
        float y = 0.0f;
        for (int jt = 0; jt <= keep; ++jt) {
            const int ii = i0 - keep + jt;
            float x = 0.0f;
            if (ii >= 0) x = a.proj[(size_t)(first + ii) * a.stride + c] + b;
            else if (hist + ii >= 0) x = old[(size_t)(keep + ii) * channels + c];
            y = fmaf(a.taps_w[(size_t)c * a.taps + jt], x, y);
        }
        return y;
    };
    // The row's cosines and sines once for all of its heads.
    for (int i = threadIdx.x; i < a.rot_pairs; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * a.freq[i], &sn, &cs);
        turn[0][i] = cs * a.rot_mag;
        turn[1][i] = sn * a.rot_mag;
    }
    // Norm 3: the root mean square of all of the row's queries, and of all of its keys.  Every block of the row makes both,
    // with the same threads in the same order.
    __shared__ float whole[2], whole_part[4];
    if (a.norm == 3) {
        for (int which = 0; which < (a.kv_heads > 0 ? 2 : 1); ++which) {
            const int c_lo = which == 0 ? 0 : a.heads * D, c_hi = which == 0 ? a.heads * D : (a.heads + a.kv_heads) * D;
            float ss = 0.0f;
            for (int c = c_lo + threadIdx.x; c < c_hi; c += blockDim.x) {
                const float v = filtered(c);
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0) whole_part[warp] = ss;
            __syncthreads();
            if (threadIdx.x == 0) {
                float t = 0.0f;
                for (int w = 0; w < warps; ++w) t += whole_part[w];
                whole[which] = 1.0f / sqrtf(t / (float)(c_hi - c_lo) + a.eps);
            }
            __syncthreads();
        }
    }
    __syncthreads();
    float* st = stage[warp];
    const int v_off = (a.heads + a.kv_heads) * D;
    for (int item = blockIdx.y * warps + warp; item < a.heads + a.kv_heads; item += gridDim.y * warps) {
        const bool is_q = item < a.heads;
        if (!is_q && slot < 0) continue;                              // a row whose cache write is skipped
        const float* w = is_q ? a.q_weight : a.k_weight;
        for (int d = lane; d < D; d += 32) st[d] = filtered(item * D + d);
        __syncwarp();
        if (a.norm == 1) {
            float ss = 0.0f;
            for (int d = lane; d < D; d += 32) ss = fmaf(st[d], st[d], ss);
            const float rr = 1.0f / sqrtf(warp_sum(ss) / (float)D + a.eps);
            for (int d = lane; d < D; d += 32) st[d] = st[d] * rr * (w ? w[d] : 1.0f);
            __syncwarp();
        } else if (a.norm == 3) {
            const float rr = whole[is_q ? 0 : 1];
            const float* wh = w ? w + (size_t)(is_q ? item : item - a.heads) * D : nullptr;
            for (int d = lane; d < D; d += 32) st[d] = st[d] * rr * (wh ? wh[d] : 1.0f);
            __syncwarp();
        }
        for (int i = lane; i < a.rot_pairs; i += 32) {
            const int ia = a.neighbours ? 2 * i : i, ib = a.neighbours ? 2 * i + 1 : i + a.rot_pairs;
            const float u = st[ia], v = st[ib];
            const float cs = turn[0][i], sn = turn[1][i];
            st[ia] = u * cs - v * sn;
            st[ib] = v * cs + u * sn;
        }
        __syncwarp();
        float rr = 1.0f;
        if (a.norm == 2) {
            float ss = 0.0f;
            for (int d = lane; d < D; d += 32) ss = fmaf(st[d], st[d], ss);
            rr = 1.0f / sqrtf(warp_sum(ss) / (float)D + a.eps);
        }
        if (is_q) {
            QT* dst = q_out + ((size_t)row * a.heads + item) * D;
            for (int d = lane; d < D; d += 32) dst[d] = from_float<QT>(a.norm == 2 ? st[d] * rr * (w ? w[d] : 1.0f) : st[d]);
        } else {
            const int g = item - a.heads;
            const size_t page = slot / a.page_size, off = slot % a.page_size;
            KVT* dst = a.planes == 2 ? cache + (((page * 2) * a.kv_heads + g) * a.page_size + off) * (size_t)D
                                     : cache + ((page * a.kv_heads + g) * a.page_size + off) * (size_t)(D + V);
            KVT* vdst = a.planes == 2 ? dst + (size_t)a.kv_heads * a.page_size * D : dst + D;
            for (int d = lane; d < D; d += 32) dst[d] = from_float<KVT>(a.norm == 2 ? st[d] * rr * (w ? w[d] : 1.0f) : st[d]);
            if (a.vfreq == nullptr) {
                for (int d = lane; d < V; d += 32) vdst[d] = from_float<KVT>(filtered(v_off + g * V + d));
            } else {
                __syncwarp();                                         // the key has left the stage
                for (int d = lane; d < V; d += 32) st[d] = filtered(v_off + g * V + d);
                __syncwarp();
                for (int i = lane; i < V / 2; i += 32) {
                    const int ia = a.neighbours ? 2 * i : i, ib = a.neighbours ? 2 * i + 1 : i + V / 2;
                    float sn, cs;
                    sincosf(pos * a.vfreq[i], &sn, &cs);
                    const float u = st[ia], v = st[ib];
                    vdst[ia] = from_float<KVT>(u * cs - v * sn);
                    vdst[ib] = from_float<KVT>(v * cs + u * sn);
                }
            }
        }
        __syncwarp();                                                 // the stage is written again for the warp's next head
    }
}

// What a design may add to the softmax attention below.
//   softcap > 0: score <- softcap * tanh(score / softcap), after the scale
//   sink_mode 1: exp(sink[head]) joins the softmax's denominator (a learned number per head that has no key and no value);
//             2: the same with 0 for every head (one is added to the denominator)
//   vfreq [V / 2]: the cached values were rotated by their positions over all of V (pair m by position * vfreq[m]; pairs
//             (m, m + V / 2), or with v_neighbours (2m, 2m + 1)); a row's output is turned back by its own position
struct AttnExtras {
    float softcap;
    const float* sink;
    int sink_mode;
    const float* vfreq;
    int v_neighbours;
};

// The factor on the weighted sum and the whole denominator, given the keys' maximum m and sum l (relative to m).
__device__ __forceinline__ float finish_softmax(float m, float l, const AttnExtras& x, int head) {
    if (x.sink_mode == 0) return 1.0f / l;
    const float sk = x.sink_mode == 1 ? x.sink[head] : 0.0f;
    const float top = fmaxf(m, sk);
    const float f = m == -INFINITY ? 0.0f : expf(m - top);
    return f / (l * f + expf(sk - top));
}

// The row's output in `o` (float, V values, written by this warp's lanes) turned back by the row's position, to `orow`.
template <typename QT>
__device__ __forceinline__ void write_turned_back(const float* o, QT* orow, int V, float pos, const AttnExtras& x, int lane) {
    for (int i = lane; i < V / 2; i += 32) {
        const int ia = x.v_neighbours ? 2 * i : i, ib = x.v_neighbours ? 2 * i + 1 : i + V / 2;
        float sn, cs;
        sincosf(pos * x.vfreq[i], &sn, &cs);
        const float u = o[ia], v = o[ib];
        orow[ia] = from_float<QT>(u * cs + v * sn);
        orow[ib] = from_float<QT>(v * cs - u * sn);
    }
}

template <typename QT, typename KVT>
__global__ void __launch_bounds__(WARPS * 32)
attention_split_kernel(const QT* __restrict__ q, const KVT* __restrict__ cache, QT* __restrict__ out,
                       const int* __restrict__ row_request, const int* __restrict__ positions,
                       const int* __restrict__ block_tables, int table_stride, int heads, int kv_heads, int D, int V,
                       int page_size, int window, int chunk, float scale, int splits, float* __restrict__ partial,
                       AttnExtras extras) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];  // WARPS * (V + 2), then V for the output before it is turned back
    const int row = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = h / (heads / kv_heads);
    const int pos = positions[row];
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
    const int* table = block_tables + (size_t)row_request[row] * table_stride;
    const int W = D + V;

    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
    const QT* qrow = q + ((size_t)row * heads + h) * D;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < D ? to_float(qrow[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    // With `splits` > 1 the row's keys are cut into that many equal ranges, one a block (blockIdx.z); each leaves its
    // partial state (sum, maximum, weight) and a second kernel merges them in range order.
    int first = lo, last = pos;
    if (splits > 1) {
        const int per = (pos - lo + splits) / splits;
        first = lo + (int)blockIdx.z * per;
        last = min(pos, first + per - 1);
    }
    for (int t = first + warp; t <= last; t += WARPS) {
        const int page = table[t / page_size], off = t % page_size;
        const KVT* kp = cache + (((size_t)page * kv_heads + g) * page_size + off) * (size_t)W;
        const KVT* vp = kp + D;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < D) s = fmaf(qv[i], to_float(kp[d]), s);
        }
        s = warp_sum(s) * scale;
        if (extras.softcap > 0.0f) s = extras.softcap * tanhf(s / extras.softcap);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
        const float e = expf(s - m_new);
        l = l * corr + e;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < V) acc[i] = fmaf(e, to_float(vp[d]), acc[i] * corr);
        }
        m = m_new;
    }
    float* mine = smem + warp * (V + 2);
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < V) mine[d] = acc[i];
    }
    if (lane == 0) {
        mine[V] = m;
        mine[V + 1] = l;
    }
    __syncthreads();
    if (warp == 0) {
        float mm = -INFINITY;
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, smem[w * (V + 2) + V]);
        float ll = 0.0f;
        float f[WARPS];
        for (int w = 0; w < WARPS; ++w) {
            const float mw = smem[w * (V + 2) + V];
            f[w] = mw == -INFINITY ? 0.0f : expf(mw - mm);
            ll += smem[w * (V + 2) + V + 1] * f[w];
        }
        if (splits > 1) {
            float* prow = partial + (((size_t)row * heads + h) * splits + blockIdx.z) * (size_t)(V + 2);
            for (int d = lane; d < V; d += 32) {
                float o = 0.0f;
                for (int w = 0; w < WARPS; ++w) o += smem[w * (V + 2) + d] * f[w];
                prow[d] = o;
            }
            if (lane == 0) {
                prow[V] = mm;
                prow[V + 1] = ll;
            }
            return;
        }
        QT* orow = out + ((size_t)row * heads + h) * V;
        const float inv = finish_softmax(mm, ll, extras, h);
        float* turned = smem + WARPS * (V + 2);
        for (int d = lane; d < V; d += 32) {
            float o = 0.0f;
            for (int w = 0; w < WARPS; ++w) o += smem[w * (V + 2) + d] * f[w];
            if (extras.vfreq) turned[d] = o * inv;
            else orow[d] = from_float<QT>(o * inv);
        }
        if (extras.vfreq) {
            __syncwarp();
            write_turned_back(turned, orow, V, (float)pos, extras, lane);
        }
    }
}

// The ranges' partial states of one (row, head), merged in range order.  One warp a (row, head).
template <typename QT>
__global__ void __launch_bounds__(128)
attention_merge_kernel(const float* __restrict__ partial, QT* __restrict__ out, int items, int V, int splits, int heads,
                       const int* __restrict__ positions, AttnExtras extras) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float merge_smem[];            // 4 * V: a warp's output before it is turned back
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= items) return;
    float* turned = merge_smem + (threadIdx.x >> 5) * V;
    const float* p = partial + (size_t)item * splits * (V + 2);
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, p[(size_t)s * (V + 2) + V]);
    float ll = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float ms = p[(size_t)s * (V + 2) + V];
        ll += ms == -INFINITY ? 0.0f : p[(size_t)s * (V + 2) + V + 1] * expf(ms - mm);
    }
    const float inv = finish_softmax(mm, ll, extras, item % heads);
    for (int d = lane; d < V; d += 32) {
        float o = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float ms = p[(size_t)s * (V + 2) + V];
            if (ms != -INFINITY) o += p[(size_t)s * (V + 2) + d] * expf(ms - mm);
        }
        if (extras.vfreq) turned[d] = o * inv;
        else out[(size_t)item * V + d] = from_float<QT>(o * inv);
    }
    if (extras.vfreq) {
        __syncwarp();
        write_turned_back(turned, out + (size_t)item * V, V, (float)positions[item / heads], extras, lane);
    }
}

// ---- the staged form, for rows that are few -------------------------------------------------------------------------------
// A block of four warps takes one row, one key/value head and one of `splits` ranges of the row's keys, and serves all
// query heads of the group from one read of the keys: tiles of TK [key ; value] rows are copied from their pages into two
// buffers of shared memory by cp.async (16-byte pieces, the next tile in flight while this one is used; rows padded by
// one piece, so that lanes reading 16-byte pieces of 32 different rows meet in no bank).  Warp w serves heads w, w + 4, ...:
// a lane makes the whole score of one key (no shuffles within a key), the tile's maximum and sum meet once a tile, the
// 32-bit weights lie in shared memory and every lane adds them over its columns of the values.  Every (row, head, range)
// leaves sum, maximum and weight in `partial`, which the merge kernel above finishes (sink, division, turning back).
template <typename T> struct Piece;
template <> struct Piece<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    }
};
template <> struct Piece<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            v[2 * i] = f.x, v[2 * i + 1] = f.y;
        }
    }
};

template <typename T, int HPW, int VPL>
__global__ void __launch_bounds__(128)
attention_staged_kernel(const T* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ row_request,
                        const int* __restrict__ positions, const int* __restrict__ block_tables, int table_stride, int heads,
                        int kv_heads, int D, int V, int page_size, int window, int chunk, float scale, int splits, int TK,
                        float softcap, float* __restrict__ partial) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char st_smem[];
    constexpr int EP = Piece<T>::N;
    const int row = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int ratio = heads / kv_heads, W = D + V, ws = W + EP, pieces = W / EP;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* qs = reinterpret_cast<float*>(st_smem);               // [ratio][D]
    float* ps = qs + (size_t)ratio * D;                          // [ratio][TK]
    T* kv = reinterpret_cast<T*>(ps + (size_t)ratio * TK);       // [2][TK][ws]
    const int pos = positions[row];
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
    const int per = (pos - lo + splits) / splits;
    const int first = lo + split * per, last = min(pos, first + per - 1);
    const int n_tiles = first <= last ? (last - first + TK) / TK : 0;
    const int* table = block_tables + (size_t)row_request[row] * table_stride;
    auto issue = [&](int tile, int which) {
        T* buf = kv + (size_t)which * TK * ws;
        const int kt0 = first + tile * TK;
        for (int i = threadIdx.x; i < TK * pieces; i += 128) {
            const int j = i / pieces, c = i - j * pieces;
            const int t = kt0 + j;
            const bool real = t <= last;
            const T* src = cache;
            if (real) src = cache + (((size_t)table[t / page_size] * kv_heads + g) * page_size + t % page_size) * (size_t)W + (size_t)c * EP;
            const int bytes = real ? 16 : 0;                         // no key here: the piece is filled with zeros
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(buf + (size_t)j * ws + c * EP)),
                         "l"(src), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n_tiles > 0) issue(0, 0);
    for (int i = threadIdx.x; i < ratio * D; i += 128) qs[i] = to_float(q[((size_t)row * heads + (size_t)g * ratio) * D + i]);
    float m[HPW], l[HPW], acc[HPW][VPL];
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        m[hh] = -INFINITY;
        l[hh] = 0.0f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) acc[hh][i] = 0.0f;
    }
    for (int tile = 0; tile < n_tiles; ++tile) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                 // this tile has landed (and the queries); everyone has left the other buffer
        if (tile + 1 < n_tiles) issue(tile + 1, (tile + 1) & 1);
        const T* buf = kv + (size_t)(tile & 1) * TK * ws;
        const int kt0 = first + tile * TK;
        const int n_here = min(TK, last - kt0 + 1);
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) {
            const int hl = warp + 4 * hh;                // the head of the group this warp serves now
            if (hl >= ratio) break;
            const float* qh = qs + (size_t)hl * D;
            float* ph = ps + (size_t)hl * TK;
            float mx = -INFINITY;
            for (int kt = lane; kt < TK; kt += 32) {
                const T* kr = buf + (size_t)kt * ws;
                float s = 0.0f;
                for (int d = 0; d < D; d += EP) {
                    float kvv[EP];
                    Piece<T>::load(kr + d, kvv);
#pragma unroll
                    for (int i = 0; i < EP; i += 4) {
                        const float4 qv = *reinterpret_cast<const float4*>(qh + d + i);
                        s = fmaf(qv.x, kvv[i], s);
                        s = fmaf(qv.y, kvv[i + 1], s);
                        s = fmaf(qv.z, kvv[i + 2], s);
                        s = fmaf(qv.w, kvv[i + 3], s);
                    }
                }
                s *= scale;
                if (softcap > 0.0f) s = softcap * tanhf(s / softcap);
                s = kt < n_here ? s : -INFINITY;
                ph[kt] = s;
                mx = fmaxf(mx, s);
            }
            mx = warp_max(mx);
            const float m_new = fmaxf(m[hh], mx);        // finite: a tile holds at least one key
            const float corr = expf(m[hh] - m_new);      // exp(-inf) = 0 before the first tile
            m[hh] = m_new;
            float lsum = 0.0f;
            for (int kt = lane; kt < TK; kt += 32) {
                const float e = expf(ph[kt] - m_new);
                ph[kt] = e;
                lsum += e;
            }
            l[hh] = l[hh] * corr + lsum;                 // per lane; the lanes meet at the end
#pragma unroll
            for (int i = 0; i < VPL; ++i) acc[hh][i] *= corr;
            __syncwarp();
            for (int key = 0; key < n_here; ++key) {
                const float e = ph[key];
                const T* vr = buf + (size_t)key * ws + D;
#pragma unroll
                for (int i = 0; i < VPL; ++i) {
                    const int c = lane + 32 * i;
                    if (c < V) acc[hh][i] = fmaf(e, to_float(vr[c]), acc[hh][i]);
                }
            }
            __syncwarp();                                // the weights are written again at the next tile
        }
    }
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int hl = warp + 4 * hh;
        if (hl >= ratio) break;
        const float lt = warp_sum(l[hh]);
        float* prow = partial + (((size_t)row * heads + (size_t)g * ratio + hl) * splits + split) * (size_t)(V + 2);
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int c = lane + 32 * i;
            if (c < V) prow[c] = acc[hh][i];
        }
        if (lane == 0) {
            prow[V] = m[hh];
            prow[V + 1] = lt;
        }
    }
}

// The tile of keys the staged form takes for these sizes (the largest of 64, 32, 16 whose buffers fit), or 0 when it does
// not take them: equal types of queries and cache, key and whole-row widths in 16-byte pieces, at most 16 heads a group.
static int staged_tile(int q_dtype, int cache_dtype, int heads, int kv_heads, int D, int V, size_t* smem_out) {
    if (q_dtype != cache_dtype || (q_dtype != LLMX_BF16 && q_dtype != LLMX_F32)) return 0;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || heads / kv_heads > 16 || D <= 0 || V <= 0 || V > 512 || D > 512) return 0;
    const int ep = q_dtype == LLMX_BF16 ? 8 : 4, es = q_dtype == LLMX_BF16 ? 2 : 4;
    if (D % ep || (D + V) % ep) return 0;
    const int ratio = heads / kv_heads;
    for (int tk = 64; tk >= 16; tk /= 2) {
        const size_t smem = ((size_t)ratio * D + (size_t)ratio * tk) * 4 + 2 * (size_t)tk * (D + V + ep) * es;
        if (smem <= 72 * 1024) {
            if (smem_out) *smem_out = smem;
            return tk;
        }
    }
    return 0;
}

// ---- the tiled form, on the tensor cores ----------------------------------------------------------------------------
// bfloat16 queries and cache, D and V multiples of 16.  A block of four warps takes 64 rows that share their keys: TOK
// tokens in a row of one request times the R_PAD heads (the group's head count rounded up to a power of two) of one
// key/value head; warp w owns rows 16 w .. 16 w + 15 for all keys (mma.sync m16n8k16, 32-bit sums).  Keys come in tiles
// of 64, whole [key ; value] rows copied from their pages by cp.async into two buffers, the next tile in flight while
// this one is multiplied.  Scores and the online softmax are 32-bit; a weight enters the second product as the sum
// of three bfloat16 values, each the rounding of what the ones before left over, so that the weights keep their 32-bit
// value (three products instead of one; their sums are 32-bit).  Values are read as the B operand through
// ldmatrix.trans.  A block finds its tile from its index by walking the requests' row counts, so nothing is planned on
// the host and a recorded step holds for any histories.
constexpr int TL_ROWS = 64, TL_KEYS = 64, TL_PAD = 8;

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Three bfloat16 values whose sum is x to 24 bits, for two neighbouring weights at once.
__device__ __forceinline__ void split3(float x, float y, uint32_t& a, uint32_t& b, uint32_t& c) {
    const __nv_bfloat16 x0 = __float2bfloat16_rn(x), y0 = __float2bfloat16_rn(y);
    const float xr = x - __bfloat162float(x0), yr = y - __bfloat162float(y0);
    const __nv_bfloat16 x1 = __float2bfloat16_rn(xr), y1 = __float2bfloat16_rn(yr);
    const __nv_bfloat16 x2 = __float2bfloat16_rn(xr - __bfloat162float(x1)), y2 = __float2bfloat16_rn(yr - __bfloat162float(y1));
    __nv_bfloat162 p0(x0, y0), p1(x1, y1), p2(x2, y2);
    a = *reinterpret_cast<uint32_t*>(&p0);
    b = *reinterpret_cast<uint32_t*>(&p1);
    c = *reinterpret_cast<uint32_t*>(&p2);
}

template <int VN_MAX>
__global__ void __launch_bounds__(128)
attention_tiled_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                       __nv_bfloat16* __restrict__ out, const int* __restrict__ row_start, const int* __restrict__ row_count,
                       const int* __restrict__ history, const int* __restrict__ block_tables, int table_stride, int requests,
                       int heads, int kv_heads, int D, int V, int page_size, int window, int chunk, float scale, int r_pad,
                       AttnExtras extras) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char tl_smem[];
    const int ratio = heads / kv_heads, tok = TL_ROWS / r_pad;
    // Which tile: the requests' tiles are numbered one request after the other.
    int idx = blockIdx.x, r = 0, tiles_r = 0;
    for (; r < requests; ++r) {
        tiles_r = (row_count[r] + tok - 1) / tok;
        if (idx < tiles_r) break;
        idx -= tiles_r;
    }
    if (r >= requests) return;
    idx = tiles_r - 1 - idx;                         // a request's last tiles have the most keys: they start first
    const int g = blockIdx.y;
    const int t0 = idx * tok, n_rows = row_count[r], a0 = row_start[r], hist = history[r];
    const int n_tok = min(tok, n_rows - t0);
    const int W = D + V, qs = D + TL_PAD, ws = W + TL_PAD;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(tl_smem);
    __nv_bfloat16* KV = Qs + (size_t)TL_ROWS * qs;               // [2][TL_KEYS][ws]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    auto lowest = [&](int p) {
        int lo = window > 0 ? max(0, p - window + 1) : 0;
        if (chunk > 0) lo = max(lo, (p / chunk) * chunk);
        return lo;
    };
    const int p_first = hist + t0, p_last = hist + t0 + n_tok - 1;
    const int key0 = lowest(p_first);
    const int n_tiles = (p_last - key0 + TL_KEYS) / TL_KEYS;
    const int* table = block_tables + (size_t)r * table_stride;
    const int w8 = W / 8;
    auto issue = [&](int tile, int which) {
        __nv_bfloat16* buf = KV + (size_t)which * TL_KEYS * ws;
        const int kt0 = key0 + tile * TL_KEYS;
        for (int i = threadIdx.x; i < TL_KEYS * w8; i += 128) {
            const int j = i / w8, c = i - j * w8;
            const int t = kt0 + j;
            __nv_bfloat16* dst = buf + (size_t)j * ws + 8 * c;
            if (t <= p_last) {
                const int page = table[t / page_size];
                const __nv_bfloat16* src = cache + (((size_t)page * kv_heads + g) * page_size + t % page_size) * (size_t)W + 8 * c;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);      // no key here: a zero weight must meet a finite value
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue(0, 0);
    // The tile's queries: row i is token t0 + i / r_pad, head g * ratio + i % r_pad (rows past the heads or the tokens are zeros).
    const int d8 = D / 8;
    for (int i = threadIdx.x; i < TL_ROWS * d8; i += 128) {
        const int row = i / d8, c = i - row * d8;
        const int tk = row / r_pad, hd = row % r_pad;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tk < n_tok && hd < ratio)
            v = *reinterpret_cast<const uint4*>(q + ((size_t)(a0 + t0 + tk) * heads + (size_t)g * ratio + hd) * D + 8 * c);
        *reinterpret_cast<uint4*>(Qs + (size_t)row * qs + 8 * c) = v;
    }
    bool valid[2];
    int pos[2], lo[2];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        const int row = 16 * warp + gid + 8 * hf;
        const int tk = row / r_pad, hd = row % r_pad;
        valid[hf] = tk < n_tok && hd < ratio;
        pos[hf] = hist + t0 + tk;
        lo[hf] = lowest(pos[hf]);
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float o[VN_MAX][4];
#pragma unroll
    for (int i = 0; i < VN_MAX; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    const int vn = V / 8;
    for (int tile = 0; tile < n_tiles; ++tile) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                 // this tile has landed (and the queries); everyone has left the other buffer
        if (tile + 1 < n_tiles) issue(tile + 1, (tile + 1) & 1);
        const __nv_bfloat16* buf = KV + (size_t)(tile & 1) * TL_KEYS * ws;
        const int kt0 = key0 + tile * TL_KEYS;
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
        for (int kk = 0; kk < D; kk += 16) {
            uint32_t a[4];
            const __nv_bfloat16* qa = Qs + (size_t)(16 * warp + gid) * qs + kk + 2 * tig;
            a[0] = *reinterpret_cast<const uint32_t*>(qa);
            a[1] = *reinterpret_cast<const uint32_t*>(qa + 8 * qs);
            a[2] = *reinterpret_cast<const uint32_t*>(qa + 8);
            a[3] = *reinterpret_cast<const uint32_t*>(qa + 8 * qs + 8);
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const __nv_bfloat16* kb = buf + (size_t)(8 * n + gid) * ws + kk + 2 * tig;
                mma_bf16_16816(s[n], a, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int hf = i >> 1, key = kt0 + 8 * n + 2 * tig + (i & 1);
                const bool seen = valid[hf] && key >= lo[hf] && key <= pos[hf];
                float sc = s[n][i] * scale;
                if (extras.softcap > 0.0f) sc = extras.softcap * tanhf(sc / extras.softcap);
                s[n][i] = seen ? sc : -INFINITY;
                mx[hf] = fmaxf(mx[hf], s[n][i]);
            }
        float corr[2], base[2];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 1));
            mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 2));
            const float m_new = fmaxf(m[hf], mx[hf]);
            base[hf] = m_new == -INFINITY ? 0.0f : m_new;
            corr[hf] = expf(m[hf] - base[hf]);           // exp(-inf) = 0 before the row's first key
            m[hf] = m_new;
            l[hf] *= corr[hf];
        }
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                s[n][i] = expf(s[n][i] - base[i >> 1]);
                l[i >> 1] += s[n][i];
            }
#pragma unroll
        for (int nv = 0; nv < VN_MAX; ++nv) {
            o[nv][0] *= corr[0];
            o[nv][1] *= corr[0];
            o[nv][2] *= corr[1];
            o[nv][3] *= corr[1];
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t p0[4], p1[4], p2[4];
            split3(s[2 * ks][0], s[2 * ks][1], p0[0], p1[0], p2[0]);
            split3(s[2 * ks][2], s[2 * ks][3], p0[1], p1[1], p2[1]);
            split3(s[2 * ks + 1][0], s[2 * ks + 1][1], p0[2], p1[2], p2[2]);
            split3(s[2 * ks + 1][2], s[2 * ks + 1][3], p0[3], p1[3], p2[3]);
            const __nv_bfloat16* vrow = buf + (size_t)(16 * ks + (lane & 15)) * ws + D;
#pragma unroll
            for (int nv = 0; nv < VN_MAX; ++nv) {
                if (nv < vn) {
                    uint32_t b0, b1;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                                 : "=r"(b0), "=r"(b1) : "r"((uint32_t)__cvta_generic_to_shared(vrow + 8 * nv)));
                    mma_bf16_16816(o[nv], p2, b0, b1);   // the smallest parts first
                    mma_bf16_16816(o[nv], p1, b0, b1);
                    mma_bf16_16816(o[nv], p0, b0, b1);
                }
            }
        }
    }
    if (extras.vfreq) {
        // Rotated values: the normed outputs meet in shared memory (the key buffers are free now), and every row is turned
        // back by its own position on the way out.
        __syncthreads();
        float* fo = reinterpret_cast<float*>(KV);                    // [TL_ROWS][V]
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            l[hf] += __shfl_xor_sync(0xffffffffu, l[hf], 1);
            l[hf] += __shfl_xor_sync(0xffffffffu, l[hf], 2);
            const int row = 16 * warp + gid + 8 * hf;
            const float inv = valid[hf] ? finish_softmax(m[hf], l[hf], extras, g * ratio + row % r_pad) : 0.0f;
#pragma unroll
            for (int nv = 0; nv < VN_MAX; ++nv)
                if (nv < vn) {
                    fo[(size_t)row * V + 8 * nv + 2 * tig] = o[nv][2 * hf] * inv;
                    fo[(size_t)row * V + 8 * nv + 2 * tig + 1] = o[nv][2 * hf + 1] * inv;
                }
        }
        __syncthreads();
        const int half = V / 2;
        for (int i = threadIdx.x; i < TL_ROWS * half; i += 128) {
            const int row = i / half, pm = i - row * half;
            const int tk = row / r_pad, hd = row % r_pad;
            if (tk >= n_tok || hd >= ratio) continue;
            const int ia = extras.v_neighbours ? 2 * pm : pm, ib = extras.v_neighbours ? 2 * pm + 1 : pm + half;
            float sn, cs;
            sincosf((float)(hist + t0 + tk) * extras.vfreq[pm], &sn, &cs);
            const float u = fo[(size_t)row * V + ia], v = fo[(size_t)row * V + ib];
            __nv_bfloat16* orow = out + ((size_t)(a0 + t0 + tk) * heads + (size_t)g * ratio + hd) * V;
            orow[ia] = __float2bfloat16_rn(u * cs + v * sn);
            orow[ib] = __float2bfloat16_rn(v * cs - u * sn);
        }
        return;
    }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        l[hf] += __shfl_xor_sync(0xffffffffu, l[hf], 1);
        l[hf] += __shfl_xor_sync(0xffffffffu, l[hf], 2);
        if (!valid[hf]) continue;
        const int row = 16 * warp + gid + 8 * hf;
        const int tk = row / r_pad, hd = row % r_pad;
        const float inv = finish_softmax(m[hf], l[hf], extras, g * ratio + hd);
        __nv_bfloat16* orow = out + ((size_t)(a0 + t0 + tk) * heads + (size_t)g * ratio + hd) * V;
#pragma unroll
        for (int nv = 0; nv < VN_MAX; ++nv)
            if (nv < vn)
                *reinterpret_cast<uint32_t*>(orow + 8 * nv + 2 * tig) = pack_bf16(o[nv][2 * hf] * inv, o[nv][2 * hf + 1] * inv);
    }
}
}  // namespace

// proj float32 [rows, stride]: queries (heads * D), keys (kv_heads * D), values (kv_heads * V) in this order.
// q_weight, k_weight float32 [D] or null (no norm); freq float32 [rot_half]; q_out [rows, heads * D] of `q_dtype`;
// cache [pages, 1, kv_heads, page_size, D + V] of `cache_dtype`; slots int32 [rows] (page * page_size + offset; negative
// skips the row's cache write).
LLMX_EXPORT int llmx_qk_norm_rope_write(const float* proj, int stride, const float* q_weight, const float* k_weight,
                                        float eps, const float* freq, int rot_half, const int* positions,
                                        const int* slots, void* q_out, int q_dtype, void* cache, int cache_dtype, int rows,
                                        int heads, int kv_heads, int D, int V, int page_size, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (D <= 0 || V <= 0 || D > 32 * MAX_PER_LANE || 2 * rot_half > D || rot_half < 0 || (rot_half > 0 && freq == nullptr) ||
        (q_weight == nullptr) != (k_weight == nullptr))
        return LLMX_ERR_UNSUPPORTED;
#define LLMX_QKW(QT, KVT)                                                                                              \
    launch_kernel(qk_write_kernel<QT, KVT>, dim3(rows), dim3(128), 0, stream, proj, stride, q_weight, k_weight, eps,   \
                  freq, rot_half, positions, slots, (QT*)q_out, (KVT*)cache, heads, kv_heads, D, V, page_size)
    if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) LLMX_QKW(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) LLMX_QKW(__nv_bfloat16, float);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) LLMX_QKW(float, __nv_bfloat16);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_F32) LLMX_QKW(float, float);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_QKW
    return launch_status();
}

// The general form of the above (see `QkvFinish`): proj float32 [rows, stride] = q (heads * D) | k (kv_heads * D) | v (kv_heads
// * V), kv_heads 0 for rows of queries alone (then `cache` and `slots` are not used); bias float32 [channels] or null; taps_w
// float32 [channels, taps] or null (taps 1: no filter); state float32 [slots, slot_floats] with the filter's inputs at
// conv_off; norm 0 / 1 / 2 = none / before / after the rotation, q_weight and k_weight float32 [D] or null; norm 3 = over the
// whole of a row's queries and of its keys before the rotation, weights float32 [heads * D] and [kv_heads * D]; freq float32
// [rot_pairs], cosines and sines times rot_mag; vfreq float32 [V / 2] or null: values rotated over all of V by their position;
// the rows' requests, their row ranges, histories and the slots read and written as a step gives them.
// planes 1: cache [pages, 1, kv_heads, page_size, D + V]; planes 2 (D = V): cache [pages, 2, kv_heads, page_size, D], the
// layout of the paged kernels with key and value planes.
LLMX_EXPORT int llmx_qkv_finish(const float* proj, int stride, const float* bias, const float* taps_w, int taps, float* state,
                                long long slot_floats, long long conv_off, const int* row_request, const int* row_start,
                                const int* row_count, const int* history, const int* slot_in, const int* slot_out,
                                const float* q_weight, const float* k_weight, int norm, float eps, const float* freq, int rot_pairs,
                                int neighbours, const int* positions, const int* slots, void* q_out, int q_dtype, void* cache,
                                int cache_dtype, int rows, int requests, int heads, int kv_heads, int D, int V, int page_size,
                                int planes, float rot_mag, const float* vfreq, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (planes != 1 && !(planes == 2 && D == V)) return LLMX_ERR_BAD_ARGUMENT;
    if (D <= 0 || V <= 0 || heads <= 0 || kv_heads < 0 || D > 32 * MAX_PER_LANE || 2 * rot_pairs > D || rot_pairs < 0 ||
        (rot_pairs > 0 && freq == nullptr) || norm < 0 || norm > 3 || taps < 1 || (vfreq != nullptr && (V % 2 || V > 32 * MAX_PER_LANE)) || (taps > 1 && (taps_w == nullptr || state == nullptr)) ||
        (kv_heads > 0 && (cache == nullptr || slots == nullptr || page_size <= 0)))
        return LLMX_ERR_BAD_ARGUMENT;
    const long long channels = (long long)(heads + kv_heads) * D + (long long)kv_heads * V;
    if (taps > 1 && conv_off + (taps - 1) * channels > slot_floats) return LLMX_ERR_BAD_ARGUMENT;
    QkvFinish a{proj, stride, bias, taps_w, taps, state, slot_floats, conv_off, row_request, row_start, row_count, history, slot_in,
                slot_out, q_weight, k_weight, norm, eps, freq, rot_pairs, neighbours, positions, slots, heads, kv_heads, D, V,
                page_size > 0 ? page_size : 1, rows, planes, rot_mag, vfreq};
    const dim3 grid(rows + (taps > 1 ? requests : 0), std::min((heads + kv_heads + 3) / 4, 64));
    const bool cache16 = kv_heads > 0 && cache_dtype == LLMX_BF16;
    if (kv_heads > 0 && cache_dtype != LLMX_BF16 && cache_dtype != LLMX_F32) return LLMX_ERR_UNSUPPORTED;
    if (q_dtype == LLMX_BF16 && cache16) launch_kernel(qkv_finish_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(128), 0, stream, a, (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache);
    else if (q_dtype == LLMX_BF16) launch_kernel(qkv_finish_kernel<__nv_bfloat16, float>, grid, dim3(128), 0, stream, a, (__nv_bfloat16*)q_out, (float*)cache);
    else if (q_dtype == LLMX_F32 && cache16) launch_kernel(qkv_finish_kernel<float, __nv_bfloat16>, grid, dim3(128), 0, stream, a, (float*)q_out, (__nv_bfloat16*)cache);
    else if (q_dtype == LLMX_F32) launch_kernel(qkv_finish_kernel<float, float>, grid, dim3(128), 0, stream, a, (float*)q_out, (float*)cache);
    else return LLMX_ERR_UNSUPPORTED;
    return launch_status();
}

// q [rows, heads, D] and out [rows, heads, V] of `q_dtype`; the cache as above, of `cache_dtype`.  `splits` > 1: a row's
// keys are cut into that many ranges (a matter of speed only: steps of few rows over long histories), which meet in
// `partial`, float32 [rows, heads, splits, V + 2].
LLMX_EXPORT int llmx_attention_split(const void* q, int q_dtype, const void* cache, int cache_dtype, void* out,
                                     const int* row_request, const int* positions, const int* block_tables,
                                     int table_stride, int rows, int heads, int kv_heads, int D, int V, int page_size,
                                     int window, int chunk, float scale, int splits, float* partial, float softcap,
                                     const float* sink, int sink_mode, const float* vfreq, int v_neighbours, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (sink_mode < 0 || sink_mode > 2 || (sink_mode == 1 && sink == nullptr) || (vfreq != nullptr && V % 2)) return LLMX_ERR_BAD_ARGUMENT;
    const AttnExtras extras{softcap, sink, sink_mode, vfreq, v_neighbours};
    if (D <= 0 || V <= 0 || D > 32 * MAX_PER_LANE || V > 32 * MAX_PER_LANE || heads % kv_heads || heads > 65535)
        return LLMX_ERR_UNSUPPORTED;
    if (splits < 1 || splits > 64 || (splits > 1 && partial == nullptr)) return LLMX_ERR_BAD_ARGUMENT;
    dim3 grid(rows, heads, splits);
    const size_t shmem = ((size_t)WARPS * (V + 2) + V) * sizeof(float);
#define LLMX_SPLIT(QT, KVT)                                                                                            \
    launch_kernel(attention_split_kernel<QT, KVT>, dim3(grid), dim3(WARPS * 32), shmem, stream, (const QT*)q,         \
                  (const KVT*)cache, (QT*)out, row_request, positions, block_tables, table_stride, heads, kv_heads, D, \
                  V, page_size, window, chunk, scale, splits, partial, extras)
    if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) LLMX_SPLIT(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) LLMX_SPLIT(__nv_bfloat16, float);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) LLMX_SPLIT(float, __nv_bfloat16);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_F32) LLMX_SPLIT(float, float);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_SPLIT
    int status = launch_status();
    if (status || splits == 1) return status;
    const int items = rows * heads;
    if (q_dtype == LLMX_BF16)
        launch_kernel(attention_merge_kernel<__nv_bfloat16>, dim3((items + 3) / 4), dim3(128), (size_t)4 * V * sizeof(float), stream, (const float*)partial, (__nv_bfloat16*)out, items, V, splits, heads, positions, extras);
    else
        launch_kernel(attention_merge_kernel<float>, dim3((items + 3) / 4), dim3(128), (size_t)4 * V * sizeof(float), stream, (const float*)partial, (float*)out, items, V, splits, heads, positions, extras);
    return launch_status();
}

// Whether the tiled form takes these sizes (bfloat16 queries and cache are the caller's to check).
LLMX_EXPORT int llmx_attention_tiled_fits(int heads, int kv_heads, int D, int V) {
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || heads / kv_heads > TL_ROWS) return 0;
    if (D <= 0 || V <= 0 || D % 16 || V % 16 || D > 256 || V > 256) return 0;
    const size_t smem = ((size_t)TL_ROWS * (D + TL_PAD) + 2 * (size_t)TL_KEYS * (D + V + TL_PAD)) * 2;
    return smem <= 200 * 1024;
}

// The tiled form: q [rows, heads, D], out [rows, heads, V] and the cache bfloat16; the step's row ranges and histories
// on the device; `rows`: the step's rows (for the grid's size only).
LLMX_EXPORT int llmx_attention_tiled(const void* q, const void* cache, void* out, const int* row_start, const int* row_count,
                                     const int* history, const int* block_tables, int table_stride, int rows, int requests,
                                     int heads, int kv_heads, int D, int V, int page_size, int window, int chunk, float scale,
                                     float softcap, const float* sink, int sink_mode, const float* vfreq, int v_neighbours,
                                     cudaStream_t stream) {
    if (rows <= 0 || requests <= 0) return 0;
    if (sink_mode < 0 || sink_mode > 2 || (sink_mode == 1 && sink == nullptr)) return LLMX_ERR_BAD_ARGUMENT;
    const AttnExtras extras{softcap, sink, sink_mode, vfreq, v_neighbours};
    if (!llmx_attention_tiled_fits(heads, kv_heads, D, V) || kv_heads > 65535) return LLMX_ERR_UNSUPPORTED;
    int r_pad = 1;
    while (r_pad < heads / kv_heads) r_pad *= 2;
    const int tok = TL_ROWS / r_pad;
    dim3 grid((rows + tok - 1) / tok + requests, kv_heads);
    const size_t smem = ((size_t)TL_ROWS * (D + TL_PAD) + 2 * (size_t)TL_KEYS * (D + V + TL_PAD)) * 2;
#define LLMX_TILED(VN)                                                                                                   \
    do {                                                                                                                  \
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_tiled_kernel<VN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_kernel(attention_tiled_kernel<VN>, dim3(grid), dim3(128), smem, stream, (const __nv_bfloat16*)q,          \
                      (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, row_start, row_count, history, block_tables,    \
                      table_stride, requests, heads, kv_heads, D, V, page_size, window, chunk, scale, r_pad, extras);   \
        return launch_status();                                                                                           \
    } while (0)
    if (V <= 64) LLMX_TILED(8);
    if (V <= 128) LLMX_TILED(16);
    LLMX_TILED(32);
#undef LLMX_TILED
}

// Whether the staged form takes these types and sizes.
LLMX_EXPORT int llmx_attention_staged_fits(int q_dtype, int cache_dtype, int heads, int kv_heads, int D, int V) {
    return staged_tile(q_dtype, cache_dtype, heads, kv_heads, D, V, nullptr) > 0;
}

// The staged form with its merge: arguments as `llmx_attention_split`; `partial` float32 [rows, heads, splits, V + 2] is
// needed whatever `splits` is.
LLMX_EXPORT int llmx_attention_staged(const void* q, int q_dtype, const void* cache, int cache_dtype, void* out,
                                      const int* row_request, const int* positions, const int* block_tables, int table_stride,
                                      int rows, int heads, int kv_heads, int D, int V, int page_size, int window, int chunk,
                                      float scale, int splits, float* partial, float softcap, const float* sink, int sink_mode,
                                      const float* vfreq, int v_neighbours, cudaStream_t stream) {
    if (rows <= 0) return 0;
    size_t smem = 0;
    const int tk = staged_tile(q_dtype, cache_dtype, heads, kv_heads, D, V, &smem);
    if (tk == 0 || kv_heads > 65535 || ((uintptr_t)cache & 15)) return LLMX_ERR_UNSUPPORTED;
    if (splits < 1 || splits > 64 || partial == nullptr || page_size <= 0) return LLMX_ERR_BAD_ARGUMENT;
    if (sink_mode < 0 || sink_mode > 2 || (sink_mode == 1 && sink == nullptr) || (vfreq != nullptr && V % 2)) return LLMX_ERR_BAD_ARGUMENT;
    const AttnExtras extras{softcap, sink, sink_mode, vfreq, v_neighbours};
    const dim3 grid(rows, kv_heads, splits);
    const int hpw = (heads / kv_heads + 3) / 4;
#define LLMX_STAGED(T, H, VL)                                                                                              \
    do {                                                                                                                    \
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_staged_kernel<T, H, VL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_kernel(attention_staged_kernel<T, H, VL>, grid, dim3(128), smem, stream, (const T*)q, (const T*)cache, row_request, \
                      positions, block_tables, table_stride, heads, kv_heads, D, V, page_size, window, chunk, scale, splits, tk, \
                      softcap, partial);                                                                                    \
    } while (0)
#define LLMX_STAGED_T(T)                                                                                                   \
    do {                                                                                                                    \
        if (V <= 128) {                                                                                                     \
            if (hpw == 1) LLMX_STAGED(T, 1, 4);                                                                             \
            else if (hpw == 2) LLMX_STAGED(T, 2, 4);                                                                        \
            else LLMX_STAGED(T, 4, 4);                                                                                      \
        } else {                                                                                                            \
            if (hpw == 1) LLMX_STAGED(T, 1, 16);                                                                            \
            else if (hpw == 2) LLMX_STAGED(T, 2, 16);                                                                       \
            else LLMX_STAGED(T, 4, 16);                                                                                     \
        }                                                                                                                   \
    } while (0)
    if (q_dtype == LLMX_BF16) LLMX_STAGED_T(__nv_bfloat16);
    else LLMX_STAGED_T(float);
#undef LLMX_STAGED_T
#undef LLMX_STAGED
    int status = launch_status();
    if (status) return status;
    const int items = rows * heads;
    if (q_dtype == LLMX_BF16)
        launch_kernel(attention_merge_kernel<__nv_bfloat16>, dim3((items + 3) / 4), dim3(128), (size_t)4 * V * sizeof(float), stream, (const float*)partial, (__nv_bfloat16*)out, items, V, splits, heads, positions, extras);
    else
        launch_kernel(attention_merge_kernel<float>, dim3((items + 3) / 4), dim3(128), (size_t)4 * V * sizeof(float), stream, (const float*)partial, (float*)out, items, V, splits, heads, positions, extras);
    return launch_status();
}
