// What happens to a token's projected heads between the q/k/v product and attention, in one pass:
//   * query and key heads: RMS norm over the head with a weight shared by all heads (optional),
//   * rotation of the first `rot_dims` dimensions of query and key heads, dimension 2i paired with 2i+1,
//     by the angle position * inv_freq[i] (optional); the rest of the head passes unchanged,
//   * values: v <- (1 - lambda) v + lambda v_first, v_first being another layer's values of the same
//     token and lambda one scalar on the device (optional),
//   * keys and (mixed) values written to their cache page; queries written back in place.
// Norm, angle, sine and cosine and the mix are float; a value is rounded once, when it is stored.
// The row is [q heads x head_dim | k heads x head_dim | v heads x v_dim].  The cache is addressed
// by two base pointers and the strides of a page, a head and a token (in elements), so keys and
// values may share a page in any arrangement.
#include "common.cuh"

namespace {
constexpr int THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(THREADS) heads_prepare_kernel(
    T* __restrict__ x, int stride, int q_heads, int kv_heads, int head_dim, int v_dim, const float* __restrict__ q_norm,
    const float* __restrict__ k_norm, float eps, const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
    const T* __restrict__ v_first, int v_first_stride, const float* __restrict__ lambda, T* __restrict__ k_cache, T* __restrict__ v_cache,
    size_t page_stride, size_t head_stride, int token_stride, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ token_row, int page_size, int pages, int* status) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, head = blockIdx.y;  // heads in the row's order: q heads, k heads, v heads
    const int pos = positions[t];
    T* row = x + (size_t)t * stride;
    int page = -1, slot = 0;
    if (k_cache && head >= q_heads) {
        const int block = pos / page_size;
        page = (pos >= 0 && block < table_width) ? block_table[(size_t)token_row[t] * table_width + block] : -1;
        if (page < 0 || page >= pages) {
            if (threadIdx.x == 0) atomicOr(status, HB_STATUS_BAD_PAGE);
            page = -1;
        }
        slot = pos - block * page_size;
    }
    if (head < q_heads + kv_heads) {
        const bool is_q = head < q_heads;
        T* p = row + (size_t)head * head_dim;
        const float* w = is_q ? q_norm : k_norm;
        float inv = 1.f;
        if (w) {
            float sum = 0.f;
            for (int i = threadIdx.x; i < head_dim; i += THREADS) {
                const float v = to_float(p[i]);
                sum = fmaf(v, v, sum);
            }
            inv = 1.0f / sqrtf(block_sum(sum, scratch) / (float)head_dim + eps);
        }
        T* dst = (is_q || !k_cache) ? p : (page >= 0 ? k_cache + (size_t)page * page_stride + (size_t)(head - q_heads) * head_stride + (size_t)slot * token_stride
                                       : nullptr);
        // pairs (2i, 2i+1): every thread handles whole pairs, so in-place writes never cross threads
        for (int i = threadIdx.x; i < (head_dim + 1) / 2; i += THREADS) {
            const int a = 2 * i, b = 2 * i + 1;
            float u = to_float(p[a]) * inv * (w ? w[a] : 1.f);
            float v = b < head_dim ? to_float(p[b]) * inv * (w ? w[b] : 1.f) : 0.f;
            if (inv_freq && b < rot_dims) {
                float s, c;
                sincosf((float)pos * inv_freq[i], &s, &c);
                const float ru = u * c - v * s, rv = v * c + u * s;
                u = ru; v = rv;
            }
            if (dst) {
                dst[a] = from_float<T>(u);
                if (b < head_dim) dst[b] = from_float<T>(v);
            }
        }
    } else {
        const int vh = head - q_heads - kv_heads;
        T* p = row + (size_t)(q_heads + kv_heads) * head_dim + (size_t)vh * v_dim;
        const T* first = v_first ? v_first + (size_t)t * v_first_stride + (size_t)vh * v_dim : nullptr;
        const float lam = first ? lambda[0] : 0.f;
        T* dst = page >= 0 ? v_cache + (size_t)page * page_stride + (size_t)vh * head_stride + (size_t)slot * token_stride : nullptr;
        for (int i = threadIdx.x; i < v_dim; i += THREADS) {
            float v = to_float(p[i]);
            if (first) v = (1.f - lam) * v + lam * to_float(first[i]);
            if (dst) dst[i] = from_float<T>(v);
        }
    }
}
}  // namespace

HB_EXPORT int hb_heads_prepare(void* x, int is_bf16, int tokens, int stride, int q_heads, int kv_heads, int head_dim, int v_dim,
                               const float* q_norm, const float* k_norm, float eps, const float* inv_freq, int rot_dims,
                               const int* positions, const void* v_first, int v_first_stride, const float* lambda, void* k_cache,
                               void* v_cache, long long page_stride, long long head_stride, int token_stride, const int* block_table,
                               int table_width, const int* token_row, int page_size, int pages, int with_values, int* status,
                               cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || v_dim <= 0 || rot_dims < 0 || rot_dims > head_dim || (rot_dims & 1)) return HB_UNSUPPORTED_SIZE;
    const int heads = q_heads + kv_heads + (with_values ? kv_heads : 0);
    if (heads <= 0 || heads > 65535) return HB_UNSUPPORTED_SIZE;
    const dim3 grid(tokens, heads);
    if (is_bf16)
        heads_prepare_kernel<<<grid, THREADS, 0, stream>>>((__nv_bfloat16*)x, stride, q_heads, kv_heads, head_dim, v_dim, q_norm, k_norm, eps,
                                                           inv_freq, rot_dims, positions, (const __nv_bfloat16*)v_first, v_first_stride, lambda,
                                                           (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (size_t)page_stride, (size_t)head_stride,
                                                           token_stride, block_table, table_width, token_row, page_size, pages, status);
    else
        heads_prepare_kernel<<<grid, THREADS, 0, stream>>>((float*)x, stride, q_heads, kv_heads, head_dim, v_dim, q_norm, k_norm, eps, inv_freq,
                                                           rot_dims, positions, (const float*)v_first, v_first_stride, lambda, (float*)k_cache,
                                                           (float*)v_cache, (size_t)page_stride, (size_t)head_stride, token_stride, block_table,
                                                           table_width, token_row, page_size, pages, status);
    return launch_status();
}

// ---------------------------------------------------------------- the same from float projections, with more choices
// The projections arrive as float rows (a product kept in float so that norms, rotations and recurrences never see a
// 16-bit value); queries go to a dense buffer of the attention's element type (or stay float, in place, for a recurrence),
// keys and values to their cache pages or to dense buffers.  Further choices:
//   * the RMS norm of queries (and of keys) may run over the whole projection, all heads at once, with a weight per
//     column of the projection (norm_whole), instead of per head with one weight for all heads,
//   * the rotation may pair dimension i with i + rot_dims / 2 (rot_half) instead of 2i with 2i + 1,
//   * keys are multiplied by k_scale after the rotation, queries by a factor per head (q_head_scale, or none).
// Every thread reads and writes whole pairs, so the float-to-float case may work in place.
namespace {
template <typename TO>
__global__ void __launch_bounds__(THREADS) heads_prepare_wide_kernel(
    const float* x, int stride, int q_off, int k_off, int v_off, int q_heads, int kv_heads, int head_dim, int v_dim,
    const float* __restrict__ q_norm, const float* __restrict__ k_norm, int norm_whole, float eps, const float* __restrict__ inv_freq,
    int rot_dims, int rot_half, const int* __restrict__ positions, float k_scale, TO* q_out, int q_out_stride, TO* k_out, int k_out_stride,
    TO* __restrict__ k_cache, TO* __restrict__ v_cache, size_t page_stride, size_t head_stride, int token_stride,
    const int* __restrict__ block_table, int table_width, const int* __restrict__ token_row, int page_size, int pages, float v_unit_eps,
    const float* __restrict__ q_head_scale, const float* __restrict__ v_inv_freq, int v_rot_dims, int v_rot_half, int* status) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, head = blockIdx.y;  // q heads, then k heads, then v heads
    const int pos = positions[t];
    const float* row = x + (size_t)t * stride;
    int page = -1, slot = 0;
    if (k_cache && head >= q_heads) {
        const int block = pos / page_size;
        page = (pos >= 0 && block < table_width) ? block_table[(size_t)token_row[t] * table_width + block] : -1;
        if (page < 0 || page >= pages) {
            if (threadIdx.x == 0) atomicOr(status, HB_STATUS_BAD_PAGE);
            page = -1;
        }
        slot = pos - block * page_size;
    }
    if (head < q_heads + kv_heads) {
        const bool is_q = head < q_heads;
        const int local = is_q ? head : head - q_heads, count = is_q ? q_heads : kv_heads;
        const float* all = row + (is_q ? q_off : k_off);
        const float* p = all + (size_t)local * head_dim;
        const float* w = is_q ? q_norm : k_norm;
        float inv = 1.f;
        if (w) {
            const float* from = norm_whole ? all : p;
            const int width = norm_whole ? count * head_dim : head_dim;
            float sum = 0.f;
            for (int i = threadIdx.x; i < width; i += THREADS) sum = fmaf(from[i], from[i], sum);
            inv = 1.0f / sqrtf(block_sum(sum, scratch) / (float)width + eps);
            if (norm_whole) w += (size_t)local * head_dim;
        }
        TO* dst;
        if (is_q) dst = q_out + (size_t)t * q_out_stride + (size_t)local * head_dim;
        else if (k_cache) dst = page >= 0 ? k_cache + (size_t)page * page_stride + (size_t)local * head_stride + (size_t)slot * token_stride : nullptr;
        else dst = k_out + (size_t)t * k_out_stride + (size_t)local * head_dim;
        if (!dst) return;
        const float post = is_q ? (q_head_scale ? q_head_scale[local] : 1.f) : k_scale;
        const int pairs = inv_freq ? rot_dims / 2 : 0;
        for (int i = threadIdx.x; i < pairs; i += THREADS) {
            const int a = rot_half ? i : 2 * i, b = rot_half ? i + pairs : 2 * i + 1;
            const float u = p[a] * inv * (w ? w[a] : 1.f), v = p[b] * inv * (w ? w[b] : 1.f);
            float s, c;
            sincosf((float)pos * inv_freq[i], &s, &c);
            dst[a] = from_float<TO>((u * c - v * s) * post);
            dst[b] = from_float<TO>((v * c + u * s) * post);
        }
        for (int i = 2 * pairs + threadIdx.x; i < head_dim; i += THREADS) dst[i] = from_float<TO>(p[i] * inv * (w ? w[i] : 1.f) * post);
    } else {
        const int vh = head - q_heads - kv_heads;
        const float* p = row + v_off + (size_t)vh * v_dim;
        TO* dst = page >= 0 ? v_cache + (size_t)page * page_stride + (size_t)vh * head_stride + (size_t)slot * token_stride : nullptr;
        float inv = 1.f;
        if (v_unit_eps >= 0.f) {  // the value head leaves with a root mean square of one
            float sum = 0.f;
            for (int i = threadIdx.x; i < v_dim; i += THREADS) sum = fmaf(p[i], p[i], sum);
            inv = 1.0f / sqrtf(block_sum(sum, scratch) / (float)v_dim + v_unit_eps);
        }
        if (!dst) return;
        const int v_pairs = v_inv_freq ? v_rot_dims / 2 : 0;  // a value may be stored turned by its own position
        for (int i = threadIdx.x; i < v_pairs; i += THREADS) {
            const int a = v_rot_half ? i : 2 * i, b = v_rot_half ? i + v_pairs : 2 * i + 1;
            float s, c;
            sincosf((float)pos * v_inv_freq[i], &s, &c);
            const float u = p[a] * inv, v = p[b] * inv;
            dst[a] = from_float<TO>(u * c - v * s);
            dst[b] = from_float<TO>(v * c + u * s);
        }
        for (int i = 2 * v_pairs + threadIdx.x; i < v_dim; i += THREADS) dst[i] = from_float<TO>(p[i] * inv);
    }
}
}  // namespace

// The same work with one block per token, for the cases in which a token's heads have something in common: a norm over the whole
// projection (its sum of squares is taken once, not once per head) and the rotation (a token's sines and cosines are taken once
// and serve every head).  Per-head norms stay with the kernel above.
namespace {
constexpr int TOKEN_THREADS = 256, MAX_PAIRS = 128;

// Heads first .. first + heads - 1 of a projection whose head 0 starts at `all`.
template <typename TO, typename Place>
__device__ __forceinline__ void prepare_heads_of_token(const float* all, int first, int heads, int head_dim, const float* w, float inv, float post,
                                                       const float* head_post, int pairs, int rot_half, const float* cs, const float* sn, Place place) {
    for (int item = threadIdx.x; item < heads * pairs; item += TOKEN_THREADS) {
        const int head = first + item / pairs, i = item % pairs;
        const int a = rot_half ? i : 2 * i, b = rot_half ? i + pairs : 2 * i + 1;
        const float* p = all + (size_t)head * head_dim;
        const float* wh = w ? w + (size_t)head * head_dim : nullptr;
        const float u = p[a] * inv * (wh ? wh[a] : 1.f), v = p[b] * inv * (wh ? wh[b] : 1.f);
        TO* dst = place(head);
        if (!dst) continue;
        const float after = head_post ? post * head_post[head] : post;
        dst[a] = from_float<TO>((u * cs[i] - v * sn[i]) * after);
        dst[b] = from_float<TO>((v * cs[i] + u * sn[i]) * after);
    }
    const int rest = head_dim - 2 * pairs;
    for (int item = threadIdx.x; item < heads * rest; item += TOKEN_THREADS) {
        const int head = first + item / rest, d = 2 * pairs + item % rest;
        TO* dst = place(head);
        if (!dst) continue;
        dst[d] = from_float<TO>(all[(size_t)head * head_dim + d] * inv * (w ? w[(size_t)head * head_dim + d] : 1.f) * (head_post ? post * head_post[head] : post));
    }
}

template <typename TO>
__global__ void __launch_bounds__(TOKEN_THREADS) heads_prepare_token_kernel(
    const float* x, int stride, int q_off, int k_off, int v_off, int q_heads, int kv_heads, int head_dim, int v_dim,
    const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps, const float* __restrict__ inv_freq, int rot_dims, int rot_half,
    const int* __restrict__ positions, float k_scale, TO* q_out, int q_out_stride, TO* k_out, int k_out_stride, TO* __restrict__ k_cache,
    TO* __restrict__ v_cache, size_t page_stride, size_t head_stride, int token_stride, const int* __restrict__ block_table, int table_width,
    const int* __restrict__ token_row, int page_size, int pages, float v_unit_eps, const float* __restrict__ q_head_scale,
    const float* __restrict__ v_inv_freq, int v_rot_dims, int v_rot_half, int* status) {
    __shared__ float scratch[32];
    __shared__ float cs[MAX_PAIRS], sn[MAX_PAIRS], vcs[MAX_PAIRS], vsn[MAX_PAIRS];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const float* row = x + (size_t)t * stride;
    const int pairs = inv_freq ? rot_dims / 2 : 0;
    const int v_pairs = (v_inv_freq && k_cache) ? v_rot_dims / 2 : 0;  // a value may be stored turned by its own position
    for (int i = threadIdx.x; i < pairs; i += TOKEN_THREADS) sincosf((float)pos * inv_freq[i], &sn[i], &cs[i]);
    for (int i = threadIdx.x; i < v_pairs; i += TOKEN_THREADS) sincosf((float)pos * v_inv_freq[i], &vsn[i], &vcs[i]);
    float inv_q = 1.f, inv_k = 1.f;
    if (q_norm) {
        float sum = 0.f;
        for (int i = threadIdx.x; i < q_heads * head_dim; i += TOKEN_THREADS) sum = fmaf(row[q_off + i], row[q_off + i], sum);
        inv_q = 1.0f / sqrtf(block_sum(sum, scratch) / (float)(q_heads * head_dim) + eps);
    }
    if (k_norm) {
        float sum = 0.f;
        for (int i = threadIdx.x; i < kv_heads * head_dim; i += TOKEN_THREADS) sum = fmaf(row[k_off + i], row[k_off + i], sum);
        inv_k = 1.0f / sqrtf(block_sum(sum, scratch) / (float)(kv_heads * head_dim) + eps);
    }
    __syncthreads();  // the sines and cosines are there
    int page = -1, slot = 0;
    if (k_cache) {
        const int block = pos / page_size;
        page = (pos >= 0 && block < table_width) ? block_table[(size_t)token_row[t] * table_width + block] : -1;
        if (page < 0 || page >= pages) {
            if (threadIdx.x == 0) atomicOr(status, HB_STATUS_BAD_PAGE);
            page = -1;
        }
        slot = pos - block * page_size;
    }
    // a step of few tokens spreads a token's heads over several blocks (blockIdx.y of gridDim.y); each takes the sums for itself
    const int parts = gridDim.y, part = blockIdx.y;
    const int q_each = (q_heads + parts - 1) / parts, k_each = (kv_heads + parts - 1) / parts;
    const int q_first = min(q_heads, part * q_each), q_count = min(q_heads, q_first + q_each) - q_first;
    const int k_first = min(kv_heads, part * k_each), k_count = min(kv_heads, k_first + k_each) - k_first;
    prepare_heads_of_token<TO>(row + q_off, q_first, q_count, head_dim, q_norm, inv_q, 1.f, q_head_scale, pairs, rot_half, cs, sn,
                               [&](int head) { return q_out + (size_t)t * q_out_stride + (size_t)head * head_dim; });
    if (k_cache) {
        TO* key_page = page >= 0 ? k_cache + (size_t)page * page_stride + (size_t)slot * token_stride : nullptr;
        prepare_heads_of_token<TO>(row + k_off, k_first, k_count, head_dim, k_norm, inv_k, k_scale, nullptr, pairs, rot_half, cs, sn,
                                   [&](int head) { return key_page ? key_page + (size_t)head * head_stride : nullptr; });
        if (page >= 0 && v_unit_eps >= 0.f) {  // every value head leaves with a root mean square of one: a warp per head
            TO* value_page = v_cache + (size_t)page * page_stride + (size_t)slot * token_stride;
            const int lane = threadIdx.x & 31;
            for (int head = k_first + (threadIdx.x >> 5); head < k_first + k_count; head += TOKEN_THREADS / 32) {
                const float* p = row + v_off + (size_t)head * v_dim;
                float sum = 0.f;
                for (int d = lane; d < v_dim; d += 32) sum = fmaf(p[d], p[d], sum);
                const float inv = 1.0f / sqrtf(warp_sum(sum) / (float)v_dim + v_unit_eps);
                for (int d = lane; d < v_dim; d += 32) value_page[(size_t)head * head_stride + d] = from_float<TO>(p[d] * inv);
            }
        } else if (page >= 0) {
            TO* value_page = v_cache + (size_t)page * page_stride + (size_t)slot * token_stride;
            for (int item = threadIdx.x; item < k_count * v_pairs; item += TOKEN_THREADS) {
                const int head = k_first + item / v_pairs, i = item % v_pairs;
                const int a = v_rot_half ? i : 2 * i, b = v_rot_half ? i + v_pairs : 2 * i + 1;
                const float* p = row + v_off + (size_t)head * v_dim;
                value_page[(size_t)head * head_stride + a] = from_float<TO>(p[a] * vcs[i] - p[b] * vsn[i]);
                value_page[(size_t)head * head_stride + b] = from_float<TO>(p[b] * vcs[i] + p[a] * vsn[i]);
            }
            const int rest = v_dim - 2 * v_pairs;
            for (int item = threadIdx.x; item < k_count * rest; item += TOKEN_THREADS) {
                const int head = k_first + item / rest, d = 2 * v_pairs + item % rest;
                value_page[(size_t)head * head_stride + d] = from_float<TO>(row[v_off + (size_t)head * v_dim + d]);
            }
        }
    } else {
        prepare_heads_of_token<TO>(row + k_off, k_first, k_count, head_dim, k_norm, inv_k, k_scale, nullptr, pairs, rot_half, cs, sn,
                                   [&](int head) { return k_out + (size_t)t * k_out_stride + (size_t)head * head_dim; });
    }
}
}  // namespace

// x [tokens, stride] float with queries at q_off, keys at k_off, values at v_off.  q_out is always given; keys go to the cache
// (k_cache and v_cache given, values too) or to k_out (values then stay where they are).
HB_EXPORT int hb_heads_prepare_wide(const float* x, int tokens, int stride, int q_off, int k_off, int v_off, int q_heads, int kv_heads, int head_dim,
                                    int v_dim, const float* q_norm, const float* k_norm, int norm_whole, float eps, const float* inv_freq, int rot_dims,
                                    int rot_half, const int* positions, float k_scale, void* q_out, int q_out_stride, void* k_out, int k_out_stride,
                                    int out_is_bf16, void* k_cache, void* v_cache, long long page_stride, long long head_stride, int token_stride,
                                    const int* block_table, int table_width, const int* token_row, int page_size, int pages, float v_unit_eps,
                                    const float* q_head_scale, const float* v_inv_freq, int v_rot_dims, int v_rot_half, int* status, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || v_dim <= 0 || rot_dims < 0 || rot_dims > head_dim || (rot_dims & 1) || !q_out || (!k_cache && !k_out)) return HB_UNSUPPORTED_SIZE;
    if (!v_inv_freq) v_rot_dims = 0;
    if (v_rot_dims < 0 || v_rot_dims > v_dim || (v_rot_dims & 1) || (v_rot_dims && (!k_cache || v_unit_eps >= 0.f))) return HB_UNSUPPORTED_SIZE;
    const int heads = q_heads + kv_heads + (k_cache ? kv_heads : 0);
    if (heads <= 0 || heads > 65535) return HB_UNSUPPORTED_SIZE;
    if ((norm_whole || (!q_norm && !k_norm)) && rot_dims / 2 <= MAX_PAIRS && v_rot_dims / 2 <= MAX_PAIRS) {  // one block per token, several when the tokens are few
        const int most = q_heads > kv_heads ? q_heads : kv_heads;
        int parts = tokens >= 256 ? 1 : 256 / tokens;
        parts = parts > most ? most : (parts > 16 ? 16 : parts);
        const dim3 token_grid(tokens, parts < 1 ? 1 : parts);
        if (out_is_bf16)
            heads_prepare_token_kernel<<<token_grid, TOKEN_THREADS, 0, stream>>>(x, stride, q_off, k_off, v_off, q_heads, kv_heads, head_dim, v_dim, q_norm, k_norm, eps,
                                                                             inv_freq, rot_dims, rot_half, positions, k_scale, (__nv_bfloat16*)q_out, q_out_stride,
                                                                             (__nv_bfloat16*)k_out, k_out_stride, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                                                                             (size_t)page_stride, (size_t)head_stride, token_stride, block_table, table_width,
                                                                             token_row, page_size, pages, v_unit_eps, q_head_scale, v_inv_freq, v_rot_dims, v_rot_half, status);
        else
            heads_prepare_token_kernel<<<token_grid, TOKEN_THREADS, 0, stream>>>(x, stride, q_off, k_off, v_off, q_heads, kv_heads, head_dim, v_dim, q_norm, k_norm, eps,
                                                                             inv_freq, rot_dims, rot_half, positions, k_scale, (float*)q_out, q_out_stride,
                                                                             (float*)k_out, k_out_stride, (float*)k_cache, (float*)v_cache, (size_t)page_stride,
                                                                             (size_t)head_stride, token_stride, block_table, table_width, token_row, page_size,
                                                                             pages, v_unit_eps, q_head_scale, v_inv_freq, v_rot_dims, v_rot_half, status);
        return launch_status();
    }
    const dim3 grid(tokens, heads);
    if (out_is_bf16)
        heads_prepare_wide_kernel<<<grid, THREADS, 0, stream>>>(x, stride, q_off, k_off, v_off, q_heads, kv_heads, head_dim, v_dim, q_norm, k_norm, norm_whole,
                                                                eps, inv_freq, rot_dims, rot_half, positions, k_scale, (__nv_bfloat16*)q_out, q_out_stride,
                                                                (__nv_bfloat16*)k_out, k_out_stride, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                                                                (size_t)page_stride, (size_t)head_stride, token_stride, block_table, table_width, token_row,
                                                                page_size, pages, v_unit_eps, q_head_scale, v_inv_freq, v_rot_dims, v_rot_half, status);
    else
        heads_prepare_wide_kernel<<<grid, THREADS, 0, stream>>>(x, stride, q_off, k_off, v_off, q_heads, kv_heads, head_dim, v_dim, q_norm, k_norm, norm_whole,
                                                                eps, inv_freq, rot_dims, rot_half, positions, k_scale, (float*)q_out, q_out_stride,
                                                                (float*)k_out, k_out_stride, (float*)k_cache, (float*)v_cache, (size_t)page_stride,
                                                                (size_t)head_stride, token_stride, block_table, table_width, token_row, page_size, pages,
                                                                v_unit_eps, q_head_scale, v_inv_freq, v_rot_dims, v_rot_half, status);
    return launch_status();
}

// ---------------------------------------------------------------- attention over a latent: what lies between its products
// A token's down-projections arrive as one float row: the query latent (q_rank entries at q_off) and, at kv_off, the key/value
// latent (kv_rank entries) followed by one key part of rot_dim entries that every head shares.  Both latents pass an RMS norm
// with a weight per entry; the first rot_dims entries of the shared key part are rotated in adjacent pairs, the rest pass as they
// are.  The query latent goes to a dense buffer (the next product's input); latent and key part go to the token's place in its
// page, the latent first: one record of kv_rank + rot_dim per token.  One block per token; sums, angles and products are float.
namespace {
template <typename TO>
__global__ void __launch_bounds__(TOKEN_THREADS) latent_prepare_kernel(
    const float* __restrict__ x, int stride, int q_off, int q_rank, int kv_off, int kv_rank, int rot_dim, int rot_dims,
    const float* __restrict__ q_norm, const float* __restrict__ kv_norm, float eps, const float* __restrict__ inv_freq,
    const int* __restrict__ positions, TO* __restrict__ cq_out, int cq_stride, TO* __restrict__ cache, size_t page_stride, int token_stride,
    const int* __restrict__ block_table, int table_width, const int* __restrict__ token_row, int page_size, int pages, int* status) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const float* row = x + (size_t)t * stride;
    float sum = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += TOKEN_THREADS) sum = fmaf(row[q_off + i], row[q_off + i], sum);
    const float inv_q = 1.0f / sqrtf(block_sum(sum, scratch) / (float)q_rank + eps);
    sum = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += TOKEN_THREADS) sum = fmaf(row[kv_off + i], row[kv_off + i], sum);
    const float inv_c = 1.0f / sqrtf(block_sum(sum, scratch) / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += TOKEN_THREADS) cq_out[(size_t)t * cq_stride + i] = from_float<TO>(row[q_off + i] * inv_q * q_norm[i]);
    const int block = pos / page_size;
    int page = (pos >= 0 && block < table_width) ? block_table[(size_t)token_row[t] * table_width + block] : -1;
    if (page < 0 || page >= pages) {
        if (threadIdx.x == 0) atomicOr(status, HB_STATUS_BAD_PAGE);
        return;
    }
    TO* dst = cache + (size_t)page * page_stride + (size_t)(pos - block * page_size) * token_stride;
    for (int i = threadIdx.x; i < kv_rank; i += TOKEN_THREADS) dst[i] = from_float<TO>(row[kv_off + i] * inv_c * kv_norm[i]);
    const float* part = row + kv_off + kv_rank;
    for (int i = threadIdx.x; i < rot_dims / 2; i += TOKEN_THREADS) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        const float u = part[2 * i], v = part[2 * i + 1];
        dst[kv_rank + 2 * i] = from_float<TO>(u * c - v * s);
        dst[kv_rank + 2 * i + 1] = from_float<TO>(v * c + u * s);
    }
    for (int i = rot_dims + threadIdx.x; i < rot_dim; i += TOKEN_THREADS) dst[kv_rank + i] = from_float<TO>(part[i]);
}

// The query that meets the cached records: per head, the query's unrotated part already carried into the latent's space
// (q_lat [head, token, kv_rank] float, the product of that part with the head's key matrix) followed by the head's rotated part,
// which is taken from the up-projected queries q [token, head, dim + rot_dim] and rotated here.  One block per (token, head).
template <typename T>
__global__ void __launch_bounds__(THREADS) latent_query_kernel(const T* __restrict__ q, int q_stride, int dim, int rot_dim, int rot_dims,
                                                                const float* __restrict__ q_lat, size_t lat_head_stride, int lat_token_stride,
                                                                int kv_rank, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                                                T* __restrict__ out, int out_stride) {
    const int t = blockIdx.x, head = blockIdx.y;
    const int pos = positions[t];
    T* dst = out + (size_t)t * out_stride + (size_t)head * (kv_rank + rot_dim);
    const float* lat = q_lat + (size_t)head * lat_head_stride + (size_t)t * lat_token_stride;
    for (int i = threadIdx.x; i < kv_rank; i += THREADS) dst[i] = from_float<T>(lat[i]);
    const T* part = q + (size_t)t * q_stride + (size_t)head * (dim + rot_dim) + dim;
    for (int i = threadIdx.x; i < rot_dims / 2; i += THREADS) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        const float u = to_float(part[2 * i]), v = to_float(part[2 * i + 1]);
        dst[kv_rank + 2 * i] = from_float<T>(u * c - v * s);
        dst[kv_rank + 2 * i + 1] = from_float<T>(v * c + u * s);
    }
    for (int i = rot_dims + threadIdx.x; i < rot_dim; i += THREADS) dst[kv_rank + i] = part[i];
}
}  // namespace

HB_EXPORT int hb_latent_prepare(const float* x, int tokens, int stride, int q_off, int q_rank, int kv_off, int kv_rank, int rot_dim, int rot_dims,
                                const float* q_norm, const float* kv_norm, float eps, const float* inv_freq, const int* positions, void* cq_out,
                                int cq_stride, int out_is_bf16, void* cache, long long page_stride, int token_stride, const int* block_table,
                                int table_width, const int* token_row, int page_size, int pages, int* status, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (q_rank <= 0 || kv_rank <= 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1) || page_size <= 0) return HB_UNSUPPORTED_SIZE;
    if (!q_norm || !kv_norm || !cq_out || !cache || (rot_dims && !inv_freq)) return HB_BAD_ARGUMENT;
    if (out_is_bf16)
        latent_prepare_kernel<<<tokens, TOKEN_THREADS, 0, stream>>>(x, stride, q_off, q_rank, kv_off, kv_rank, rot_dim, rot_dims, q_norm, kv_norm, eps, inv_freq,
                                                                    positions, (__nv_bfloat16*)cq_out, cq_stride, (__nv_bfloat16*)cache, (size_t)page_stride,
                                                                    token_stride, block_table, table_width, token_row, page_size, pages, status);
    else
        latent_prepare_kernel<<<tokens, TOKEN_THREADS, 0, stream>>>(x, stride, q_off, q_rank, kv_off, kv_rank, rot_dim, rot_dims, q_norm, kv_norm, eps, inv_freq,
                                                                    positions, (float*)cq_out, cq_stride, (float*)cache, (size_t)page_stride, token_stride,
                                                                    block_table, table_width, token_row, page_size, pages, status);
    return launch_status();
}

HB_EXPORT int hb_latent_query(const void* q, int is_bf16, int tokens, int q_stride, int heads, int dim, int rot_dim, int rot_dims, const float* q_lat,
                              long long lat_head_stride, int lat_token_stride, int kv_rank, const float* inv_freq, const int* positions, void* out,
                              int out_stride, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || dim <= 0 || kv_rank <= 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1)) return HB_UNSUPPORTED_SIZE;
    if (rot_dims && !inv_freq) return HB_BAD_ARGUMENT;
    const dim3 grid(tokens, heads);
    if (is_bf16)
        latent_query_kernel<<<grid, THREADS, 0, stream>>>((const __nv_bfloat16*)q, q_stride, dim, rot_dim, rot_dims, q_lat, (size_t)lat_head_stride,
                                                          lat_token_stride, kv_rank, inv_freq, positions, (__nv_bfloat16*)out, out_stride);
    else
        latent_query_kernel<<<grid, THREADS, 0, stream>>>((const float*)q, q_stride, dim, rot_dim, rot_dims, q_lat, (size_t)lat_head_stride, lat_token_stride,
                                                          kv_rank, inv_freq, positions, (float*)out, out_stride);
    return launch_status();
}

// ---------------------------------------------------------------- a rotation of heads in place
// Every head of the columns col0 .. col0 + heads * head_dim of a row turns by sign * position: within a head's first rot_dims entries,
// entry i with entry i + rot_dims / 2 (rot_half) or entry 2i with 2i + 1, pair i by the angle sign * position * inv_freq[i]; the rest
// of the head stays.  Values that are cached rotated by their own position and results that are turned back by the query's position
// (sign = -1) both pass through here.  The angle, its sine and cosine and the products are float; one rounding at the store.
namespace {
constexpr int ROTATE_THREADS = 256, ROTATE_PAIRS = 256;

template <typename T>
__global__ void __launch_bounds__(ROTATE_THREADS) rotate_heads_kernel(T* x, int stride, int col0, int heads, int head_dim, int rot_dims, int rot_half,
                                                                      const float* __restrict__ inv_freq, const int* __restrict__ positions, float sign) {
    __shared__ float cs[ROTATE_PAIRS], sn[ROTATE_PAIRS];
    const int t = blockIdx.x, pairs = rot_dims / 2;
    const float pos = (float)positions[t];
    const bool tabled = pairs <= ROTATE_PAIRS;
    if (tabled) {
        for (int i = threadIdx.x; i < pairs; i += ROTATE_THREADS) {
            float s, c;
            sincosf(pos * inv_freq[i], &s, &c);
            cs[i] = c;
            sn[i] = sign * s;
        }
        __syncthreads();
    }
    T* row = x + (size_t)t * stride + col0;
    for (int item = blockIdx.y * ROTATE_THREADS + threadIdx.x; item < heads * pairs; item += gridDim.y * ROTATE_THREADS) {
        const int head = item / pairs, i = item % pairs;
        const int a = rot_half ? i : 2 * i, b = rot_half ? i + pairs : 2 * i + 1;
        T* p = row + (size_t)head * head_dim;
        float s, c;
        if (tabled) { c = cs[i]; s = sn[i]; }
        else { sincosf(pos * inv_freq[i], &s, &c); s *= sign; }
        const float u = to_float(p[a]), v = to_float(p[b]);
        p[a] = from_float<T>(u * c - v * s);
        p[b] = from_float<T>(v * c + u * s);
    }
}
}  // namespace

HB_EXPORT int hb_rotate_heads(void* x, int is_bf16, int tokens, int stride, int col0, int heads, int head_dim, int rot_dims, int rot_half,
                              const float* inv_freq, const int* positions, float sign, cudaStream_t stream) {
    if (tokens <= 0 || heads <= 0 || rot_dims <= 0) return 0;
    if (head_dim <= 0 || rot_dims > head_dim || (rot_dims & 1) || !inv_freq || !positions) return HB_UNSUPPORTED_SIZE;
    const int items = heads * (rot_dims / 2);
    int parts = tokens >= 512 ? 1 : (items + ROTATE_THREADS - 1) / ROTATE_THREADS;  // few tokens: a token's pairs over several blocks
    parts = parts < 1 ? 1 : (parts > 64 ? 64 : parts);
    const dim3 grid(tokens, parts);
    if (is_bf16) rotate_heads_kernel<<<grid, ROTATE_THREADS, 0, stream>>>((__nv_bfloat16*)x, stride, col0, heads, head_dim, rot_dims, rot_half, inv_freq, positions, sign);
    else rotate_heads_kernel<<<grid, ROTATE_THREADS, 0, stream>>>((float*)x, stride, col0, heads, head_dim, rot_dims, rot_half, inv_freq, positions, sign);
    return launch_status();
}
