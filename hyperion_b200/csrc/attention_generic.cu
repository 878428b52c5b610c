// Causal grouped-query attention over the paged cache for any head size up to 256, any number of
// heads and groups, and an optional window: the kernel of the 32-bit path (and of float tests of the
// bfloat16 kernels). One block serves one token and up to 8 query heads of one key/value head.
// Keys are walked in tiles of 64 absolute positions (tile t covers positions 64t..64t+63), with a
// running maximum and sum in float, so a token's result does not depend on how its request was cut
// into steps or on the rest of the batch. The formula is the reference's: q head h reads kv head
// h / group, scores (q.k) * scale for key position <= query position, softmax, weighted sum of values
// (helios/crates/helios-hal/src/reference.rs:118-156; kernels/elementwise.cu:64-118).
// Beyond the reference: keys and values may have different sizes per head and lie anywhere in a page
// (the launcher gets their two base pointers and the strides of a page, a head and a token), and a
// score may be capped smoothly, s <- cap * tanh(s / cap), before the softmax (cap 0 = no cap); a learned bias per head and
// distance may be added to the score, and the result may pass a sigmoid gate.  Further options, each absent unless its
// argument is given: a factor per head on the scaled score; a slope per head, slope * (query position - key position)
// being taken off the score; sight limited to the query's own chunk of positions (chunks of `chunk` positions counted
// from position 0); a sink per head, one more term exp(sink) in the softmax's denominator that has no key and no value.
// Heads of up to 640 entries take the kernel's second size (more shared memory and registers).
#include "common.cuh"

namespace {
constexpr int TILE = 64, THREADS = 128, GMAX = 8;

struct ScoreExtras {
    const float* head_scale;  // [heads] or null
    const float* slopes;      // [heads] or null
    const float* sinks;       // [heads] or null
    int chunk;                // 0: no chunks
};

template <typename T, int DMAX>
__global__ void __launch_bounds__(THREADS) attention_generic_kernel(
    const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride, const T* __restrict__ k_cache,
    const T* __restrict__ v_cache, size_t page_stride, size_t head_stride, int token_stride,
    const int* __restrict__ block_table, int table_width, const int* __restrict__ token_row,
    const int* __restrict__ positions, int heads, int kv_heads, int head_dim, int v_dim, int page_size, int pages, float scale,
    float softcap, int window, const float* __restrict__ dist_bias, int bias_span, const float* __restrict__ gate, int gate_stride,
    int gate_off, float out_scale, const ScoreExtras extras, int* status) {
    __shared__ float qs[GMAX][DMAX];
    __shared__ float score[GMAX][TILE];
    __shared__ float m_run[GMAX], l_run[GMAX], alpha[GMAX];
    __shared__ int tile_page[TILE];

    const int t = blockIdx.x, kvh = blockIdx.y;
    const int group = heads / kv_heads;
    const int g0 = blockIdx.z * GMAX;
    const int g = min(GMAX, group - g0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = positions[t];
    const int row = token_row[t];
    const int* table = block_table + (size_t)row * table_width;

    for (int e = tid; e < g * head_dim; e += THREADS) {
        const int hh = e / head_dim, d = e - hh * head_dim;
        qs[hh][d] = to_float(q[(size_t)t * q_stride + (size_t)(kvh * group + g0 + hh) * head_dim + d]);
    }
    if (tid < GMAX) {  // a sink enters as a key whose score is the sink itself and whose value is nothing
        const bool sunk = extras.sinks && tid < g;
        m_run[tid] = sunk ? extras.sinks[kvh * group + g0 + tid] : -INFINITY;
        l_run[tid] = sunk ? 1.f : 0.f;
    }
    float acc[GMAX][DMAX / THREADS];
#pragma unroll
    for (int hh = 0; hh < GMAX; ++hh)
#pragma unroll
        for (int c = 0; c < DMAX / THREADS; ++c) acc[hh][c] = 0.f;

    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (extras.chunk > 0) lo = max(lo, (pos / extras.chunk) * extras.chunk);
    bool bad_page = false;
    __syncthreads();

    for (int base = (lo / TILE) * TILE; base <= pos; base += TILE) {
        // pages of the tile's keys
        if (tid < TILE) {
            const int j = base + tid;
            int page = -1;
            if (j >= lo && j <= pos) {
                const int block = j / page_size;
                page = block < table_width ? table[block] : -1;
                if (page < 0 || page >= pages) { bad_page = true; page = -1; }
            }
            tile_page[tid] = page;
        }
        __syncthreads();
        // scores: one warp per key, lanes across the head dimension
        for (int jj = warp; jj < TILE; jj += THREADS / 32) {
            const int j = base + jj;
            const int page = tile_page[jj];
            float part[GMAX];
#pragma unroll
            for (int hh = 0; hh < GMAX; ++hh) part[hh] = 0.f;
            if (page >= 0) {
                const T* kp = k_cache + (size_t)page * page_stride + (size_t)kvh * head_stride + (size_t)(j % page_size) * token_stride;
                for (int d = lane; d < head_dim; d += 32) {
                    const float kv = to_float(kp[d]);
#pragma unroll
                    for (int hh = 0; hh < GMAX; ++hh)
                        if (hh < g) part[hh] = fmaf(qs[hh][d], kv, part[hh]);
                }
            }
#pragma unroll
            for (int hh = 0; hh < GMAX; ++hh) {
                if (hh < g) {
                    const float s = warp_sum(part[hh]);
                    if (lane == 0) {
                        float capped = s * scale;
                        if (extras.head_scale) capped *= extras.head_scale[kvh * group + g0 + hh];
                        if (softcap > 0.f) capped = softcap * tanhf(capped / softcap);
                        if (dist_bias) capped += dist_bias[(size_t)(kvh * group + g0 + hh) * bias_span + min(pos - j, bias_span - 1)];
                        if (extras.slopes) capped -= extras.slopes[kvh * group + g0 + hh] * (float)(pos - j);
                        score[hh][jj] = page >= 0 ? capped : -INFINITY;
                    }
                }
            }
        }
        __syncthreads();
        // new running maximum and the rescale factor, one thread per head
        if (tid < g) {
            float m = m_run[tid];
            for (int jj = 0; jj < TILE; ++jj) m = fmaxf(m, score[tid][jj]);
            alpha[tid] = (m == -INFINITY) ? 1.f : expf(m_run[tid] - m);
            m_run[tid] = m;
        }
        __syncthreads();
        for (int e = tid; e < g * TILE; e += THREADS) {
            const int hh = e / TILE, jj = e - hh * TILE;
            const float m = m_run[hh];
            score[hh][jj] = (m == -INFINITY) ? 0.f : expf(score[hh][jj] - m);
        }
        __syncthreads();
        if (tid < g) {
            float l = l_run[tid] * alpha[tid];
            for (int jj = 0; jj < TILE; ++jj) l += score[tid][jj];
            l_run[tid] = l;
        }
        // weighted values: thread d walks the tile's keys in order
#pragma unroll
        for (int c = 0; c < DMAX / THREADS; ++c) {
            const int d = tid + c * THREADS;
            if (d < v_dim) {
#pragma unroll
                for (int hh = 0; hh < GMAX; ++hh)
                    if (hh < g) acc[hh][c] *= alpha[hh];
                for (int jj = 0; jj < TILE; ++jj) {
                    const int page = tile_page[jj];
                    if (page < 0) continue;
                    const int j = base + jj;
                    const float vv = to_float(v_cache[(size_t)page * page_stride + (size_t)kvh * head_stride +
                                                      (size_t)(j % page_size) * token_stride + d]);
#pragma unroll
                    for (int hh = 0; hh < GMAX; ++hh)
                        if (hh < g) acc[hh][c] = fmaf(score[hh][jj], vv, acc[hh][c]);
                }
            }
        }
        __syncthreads();
    }
    if (bad_page) atomicOr(status, HB_STATUS_BAD_PAGE);
#pragma unroll
    for (int c = 0; c < DMAX / THREADS; ++c) {
        const int d = tid + c * THREADS;
        if (d < v_dim) {
#pragma unroll
            for (int hh = 0; hh < GMAX; ++hh)
                if (hh < g) {
                    const float l = l_run[hh];
                    const size_t column = (size_t)(kvh * group + g0 + hh) * v_dim + d;
                    float result = l > 0.f ? acc[hh][c] / l : 0.f;
                    if (gate) result *= out_scale / (1.f + expf(-gate[(size_t)t * gate_stride + gate_off + column]));
                    out[(size_t)t * out_stride + column] = from_float<T>(result);
                }
        }
    }
}
}  // namespace

// Keys at k_cache[page * page_stride + kv_head * head_stride + place * token_stride + i], i < head_dim; values likewise
// from v_cache with i < v_dim (strides in elements).  dist_bias [heads, bias_span] float (optional): a score of query position p and
// key position j takes dist_bias[head, min(p - j, bias_span - 1)] after scale and cap.  gate [tokens, gate_stride] float (optional): the
// result of (token, head, d) is multiplied by out_scale * sigmoid(gate[token, gate_off + head * v_dim + d]) before its one rounding.
// head_scale, slopes, sinks: [heads] float each or null; chunk: 0 or the size of the chunks of positions a query stays inside.
HB_EXPORT int hb_attention_extended(const void* q, int q_stride, void* out, int out_stride, int is_bf16, const void* k_cache,
                                    const void* v_cache, long long page_stride, long long head_stride, int token_stride,
                                    const int* block_table, int table_width, const int* token_row, const int* positions,
                                    int tokens, int heads, int kv_heads, int head_dim, int v_dim, int page_size, int pages, float scale,
                                    float softcap, int window, const float* dist_bias, int bias_span, const float* gate, int gate_stride,
                                    int gate_off, float out_scale, const float* head_scale, const float* slopes, const float* sinks, int chunk,
                                    int* status, cudaStream_t stream) {
    if ((dist_bias && bias_span <= 0) || chunk < 0) return HB_BAD_ARGUMENT;
    if (tokens <= 0) return 0;
    const int largest = head_dim > v_dim ? head_dim : v_dim;
    if (head_dim <= 0 || v_dim <= 0 || largest > 640 || kv_heads <= 0 || heads % kv_heads || page_size <= 0) return HB_UNSUPPORTED_SIZE;
    const int group = heads / kv_heads;
    dim3 grid(tokens, kv_heads, (group + GMAX - 1) / GMAX);
    if (grid.y > 65535 || grid.z > 65535) return HB_UNSUPPORTED_SIZE;
    const ScoreExtras extras{head_scale, slopes, sinks, chunk};
#define HB_ATTEND(T, DMAX)                                                                                                                       \
    attention_generic_kernel<T, DMAX><<<grid, THREADS, 0, stream>>>((const T*)q, q_stride, (T*)out, out_stride, (const T*)k_cache, (const T*)v_cache, \
                                                                    (size_t)page_stride, (size_t)head_stride, token_stride, block_table, table_width, \
                                                                    token_row, positions, heads, kv_heads, head_dim, v_dim, page_size, pages, scale,  \
                                                                    softcap, window, dist_bias, bias_span, gate, gate_stride, gate_off, out_scale,    \
                                                                    extras, status)
    if (largest <= 256) {
        if (is_bf16) HB_ATTEND(__nv_bfloat16, 256);
        else HB_ATTEND(float, 256);
    } else {
        if (is_bf16) HB_ATTEND(__nv_bfloat16, 640);
        else HB_ATTEND(float, 640);
    }
#undef HB_ATTEND
    return launch_status();
}

HB_EXPORT int hb_attention_biased(const void* q, int q_stride, void* out, int out_stride, int is_bf16, const void* k_cache,
                                  const void* v_cache, long long page_stride, long long head_stride, int token_stride,
                                  const int* block_table, int table_width, const int* token_row, const int* positions,
                                  int tokens, int heads, int kv_heads, int head_dim, int v_dim, int page_size, int pages, float scale,
                                  float softcap, int window, const float* dist_bias, int bias_span, const float* gate, int gate_stride,
                                  int gate_off, float out_scale, int* status, cudaStream_t stream) {
    if (head_dim > 256 || v_dim > 256) return HB_UNSUPPORTED_SIZE;
    return hb_attention_extended(q, q_stride, out, out_stride, is_bf16, k_cache, v_cache, page_stride, head_stride, token_stride, block_table,
                                 table_width, token_row, positions, tokens, heads, kv_heads, head_dim, v_dim, page_size, pages, scale, softcap,
                                 window, dist_bias, bias_span, gate, gate_stride, gate_off, out_scale, nullptr, nullptr, nullptr, 0, status, stream);
}

HB_EXPORT int hb_attention_general(const void* q, int q_stride, void* out, int out_stride, int is_bf16, const void* k_cache,
                                   const void* v_cache, long long page_stride, long long head_stride, int token_stride,
                                   const int* block_table, int table_width, const int* token_row, const int* positions,
                                   int tokens, int heads, int kv_heads, int head_dim, int v_dim, int page_size, int pages, float scale,
                                   float softcap, int window, int* status, cudaStream_t stream) {
    return hb_attention_biased(q, q_stride, out, out_stride, is_bf16, k_cache, v_cache, page_stride, head_stride, token_stride, block_table,
                               table_width, token_row, positions, tokens, heads, kv_heads, head_dim, v_dim, page_size, pages, scale, softcap,
                               window, nullptr, 0, nullptr, 0, 0, 1.f, status, stream);
}

// Keys and values of one size in pages of [2, kv_heads, page_size, head_dim], no cap.
HB_EXPORT int hb_attention_generic(const void* q, int q_stride, void* out, int out_stride, int is_bf16, const void* cache,
                                   const int* block_table, int table_width, const int* token_row, const int* positions,
                                   int tokens, int heads, int kv_heads, int head_dim, int page_size, int pages, float scale,
                                   int window, int* status, cudaStream_t stream) {
    const long long head_stride = (long long)page_size * head_dim;
    const size_t element = is_bf16 ? 2 : 4;
    return hb_attention_general(q, q_stride, out, out_stride, is_bf16, cache, (const char*)cache + (size_t)kv_heads * head_stride * element,
                                2 * (long long)kv_heads * head_stride, head_stride, head_dim, block_table, table_width, token_row, positions,
                                tokens, heads, kv_heads, head_dim, head_dim, page_size, pages, scale, 0.f, window, status, stream);
}
