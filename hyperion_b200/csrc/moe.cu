// Kernels of a feed-forward made of many small experts of which every token uses a few: the router, the plan that sorts
// (token, choice) pairs by expert, the gather of the sorted rows, a grouped matrix product (every tile of rows multiplies its own
// expert's matrix) and the sum of a token's experts.  Nothing here asks the host anything: the number of rows an expert gets
// is known on the device only, so all buffers are sized by their worst case (every expert's rows padded to whole tiles) and
// tiles beyond the last used one find -1 in the tile list and return.
//
//   route:    z = W_r x in float (one sequential chain of fixed shape per logit), the `top` largest logits by selection
//             (lowest index first among equals), weight = sigmoid(z) of the chosen (not renormalised) or 1
//   plan:     per expert a run of slots, padded to a multiple of `pad`; slot_of[token, choice]; per slot its token (or -1)
//             and its weight; per tile of `pad` slots its expert (or -1) and how many of its slots are taken
//   gather:   xs[slot] = weight * x[token] (the weight multiplies what the expert reads); padding rows are left as they are
//   product:  C[slot] = A[slot] W[expert of slot's tile]^T, float accumulation in one chain over k per output
//   combine:  out[token] = base[token] + sum over choices of y[slot_of[token, choice]], in the order of the choices
//
// A second router and a second combine serve feed-forwards whose router scores are a softmax, whose choice is made on score + a
// correction inside the best groups of neighbouring experts, whose last router outputs are experts without matrices that hand
// their input on as it is, and whose weights multiply what an expert returns:
//   route_scored:      s = softmax(z) over all outputs; c = s + correction; only outputs of the `keep` groups with the largest
//                      best c can be chosen; the `top` largest c; weight = s * scale
//   plan:              a choice >= experts takes no slot (slot_of = -1); without weights every slot's weight is 1
//   combine_weighted:  out[token] = sigmoid(gate[token]) * base[token] + sum over choices of w * (y[slot] or, without a slot, x[token])
#include "common.cuh"

namespace {
constexpr int ROUTE_THREADS = 256;

// One block per token: the row in shared memory as floats, a warp per expert at a time.  A lane adds up every 32nd group of four
// columns in four chains of its own (columns beyond a multiple of four go to the first chain), the chains are added in a fixed
// order and the lanes meet in a butterfly: a logit depends on nothing but the row and the expert's weights.
template <typename T>
__device__ __forceinline__ void router_logits(const T* __restrict__ x, int x_stride, const float* __restrict__ router, int hidden, int experts, float* row,
                                              float* logit) {
    const int padded = (hidden + 3) & ~3;
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < padded; i += ROUTE_THREADS) row[i] = i < hidden ? to_float(x[(size_t)t * x_stride + i]) : 0.f;
    __syncthreads();
    const bool by_four = (hidden & 3) == 0 && (((uintptr_t)router) & 15) == 0;
    for (int e = warp; e < experts; e += ROUTE_THREADS / 32) {
        const float* w = router + (size_t)e * hidden;
        float part[4] = {0.f, 0.f, 0.f, 0.f};
        if (by_four) {
#pragma unroll 4
            for (int i = lane * 4; i < hidden; i += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(w + i), rv = *reinterpret_cast<const float4*>(row + i);
                part[0] = fmaf(rv.x, wv.x, part[0]); part[1] = fmaf(rv.y, wv.y, part[1]);
                part[2] = fmaf(rv.z, wv.z, part[2]); part[3] = fmaf(rv.w, wv.w, part[3]);
            }
        } else {
            for (int i = lane * 4; i < hidden; i += 128)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (i + j < hidden) part[j] = fmaf(row[i + j], w[i + j], part[j]);
        }
        const float sum = warp_sum((part[0] + part[1]) + (part[2] + part[3]));
        if (lane == 0) logit[e] = sum;
    }
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS) moe_route_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ router, int hidden,
                                                                  int experts, int top, int weighted, int* __restrict__ chosen,
                                                                  float* __restrict__ weights) {
    extern __shared__ __align__(16) float shared[];  // the token's row (padded to a multiple of four), then one logit per expert
    float* row = shared;
    float* logit = shared + ((hidden + 3) & ~3);
    const int t = blockIdx.x;
    router_logits(x, x_stride, router, hidden, experts, row, logit);
    if (threadIdx.x == 0) {
        for (int k = 0; k < top; ++k) {
            int best = -1;
            float value = -INFINITY;
            for (int e = 0; e < experts; ++e)
                if (logit[e] > value || (best < 0 && logit[e] == value)) { best = e; value = logit[e]; }
            if (best < 0) best = 0;  // only when every logit left is not a number
            chosen[(size_t)t * top + k] = best;
            weights[(size_t)t * top + k] = weighted ? 1.0f / (1.0f + expf(-value)) : 1.f;
            logit[best] = -INFINITY;
        }
    }
}

// The largest value among the lanes, the lowest index among equals; a lane without a candidate brings index INT_MAX.
__device__ __forceinline__ void warp_best(float& value, int& index) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, value, offset);
        const int where = __shfl_xor_sync(0xffffffffu, index, offset);
        if (where != 0x7fffffff && (index == 0x7fffffff || other > value || (other == value && where < index))) { value = other; index = where; }
    }
}

// Softmax scores over all `outputs` of the router, choice by score + correction inside the best `group_keep` of `group_count` groups of
// neighbours (a group's rank is its largest choice score; group_count <= 1: no groups), weights = plain score * scale.  The logits are
// taken as in the kernel above; everything after them is the first warp's work, sums and searches in a fixed order.
template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS) moe_route_scored_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ router,
                                                                         const float* __restrict__ correction, int hidden, int outputs, int top,
                                                                         int group_count, int group_keep, float scale, int* __restrict__ chosen,
                                                                         float* __restrict__ weights) {
    extern __shared__ __align__(16) float shared[];  // the row, then per output: logit, score, choice score, a flag; then per group: best, a flag
    float* row = shared;
    float* logit = shared + ((hidden + 3) & ~3);
    float* score = logit + outputs;
    float* choice = score + outputs;
    int* dead = reinterpret_cast<int*>(choice + outputs);
    float* group_best = reinterpret_cast<float*>(dead + outputs);
    int* group_kept = reinterpret_cast<int*>(group_best + (group_count > 0 ? group_count : 1));
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    router_logits(x, x_stride, router, hidden, outputs, row, logit);
    if (threadIdx.x >= 32) return;
    float most = -INFINITY;
    for (int e = lane; e < outputs; e += 32) most = fmaxf(most, logit[e]);
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) most = fmaxf(most, __shfl_xor_sync(0xffffffffu, most, offset));
    float sum = 0.f;
    for (int e = lane; e < outputs; e += 32) {
        const float p = expf(logit[e] - most);
        score[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < outputs; e += 32) {
        score[e] = score[e] / sum;
        choice[e] = score[e] + (correction ? correction[e] : 0.f);
        dead[e] = 0;
    }
    __syncwarp();
    if (group_count > 1 && group_keep < group_count) {
        const int per = outputs / group_count;
        for (int g = lane; g < group_count; g += 32) {
            float best = -INFINITY;
            for (int i = 0; i < per; ++i) best = fmaxf(best, choice[g * per + i]);
            group_best[g] = best;
            group_kept[g] = 0;
        }
        __syncwarp();
        for (int k = 0; k < group_keep; ++k) {
            float value = -INFINITY;
            int index = 0x7fffffff;
            for (int g = lane; g < group_count; g += 32)
                if (!group_kept[g] && (index == 0x7fffffff || group_best[g] > value)) { value = group_best[g]; index = g; }
            warp_best(value, index);
            if (lane == 0 && index != 0x7fffffff) group_kept[index] = 1;
            __syncwarp();
        }
        for (int e = lane; e < outputs; e += 32) dead[e] = !group_kept[e / per];
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float value = -INFINITY;
        int index = 0x7fffffff;
        for (int e = lane; e < outputs; e += 32)
            if (!dead[e] && (index == 0x7fffffff || choice[e] > value)) { value = choice[e]; index = e; }
        warp_best(value, index);
        if (index == 0x7fffffff) index = 0;  // only when fewer outputs can be chosen than are asked for
        if (lane == 0) {
            chosen[(size_t)t * top + k] = index;
            weights[(size_t)t * top + k] = score[index] * scale;
            dead[index] = 1;
        }
        __syncwarp();
    }
}

constexpr int PLAN_THREADS = 1024;

// One block.  counts and cursors live in shared memory (experts <= 1024).
__global__ void __launch_bounds__(PLAN_THREADS) moe_plan_kernel(const int* __restrict__ chosen, const float* __restrict__ weights, int pairs, int top,
                                                                int experts, int pad, int capacity, int* __restrict__ slot_of,
                                                                int* __restrict__ slot_token, float* __restrict__ slot_weight,
                                                                int* __restrict__ tile_expert, int* __restrict__ tile_rows) {
    __shared__ int count[1024], start[1024];
    const int tid = threadIdx.x;
    for (int e = tid; e < experts; e += PLAN_THREADS) count[e] = 0;
    for (int s = tid; s < capacity; s += PLAN_THREADS) { slot_token[s] = -1; slot_weight[s] = 0.f; }
    for (int i = tid; i < capacity / pad; i += PLAN_THREADS) { tile_expert[i] = -1; tile_rows[i] = 0; }
    __syncthreads();
    for (int i = tid; i < pairs; i += PLAN_THREADS)
        if (chosen[i] < experts) atomicAdd(&count[chosen[i]], 1);  // a choice beyond the experts with matrices takes no row
    __syncthreads();
    if (tid == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = at;
            const int tiles = (count[e] + pad - 1) / pad;
            for (int i = 0; i < tiles; ++i) {
                tile_expert[at / pad + i] = e;
                tile_rows[at / pad + i] = min(pad, count[e] - i * pad);
            }
            at += tiles * pad;
            count[e] = 0;  // from here on: the cursor inside the expert's run
        }
    }
    __syncthreads();
    // which slot of its expert's run a pair takes depends on the order of the atomics; a row's result does not depend on its slot
    for (int i = tid; i < pairs; i += PLAN_THREADS) {
        const int e = chosen[i];
        if (e >= experts) { slot_of[i] = -1; continue; }
        const int slot = start[e] + atomicAdd(&count[e], 1);
        slot_of[i] = slot;
        slot_token[slot] = i / top;
        slot_weight[slot] = weights ? weights[i] : 1.f;
    }
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, int x_stride, const int* __restrict__ slot_token, const float* __restrict__ slot_weight,
                                  T* __restrict__ out, int hidden) {
    const int slot = blockIdx.x, t = slot_token[slot];
    if (t < 0) return;  // padding: whatever the product makes of such a row, no one reads it, and rows do not meet in a product
    const float w = slot_weight[slot];
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)slot * hidden + i] = from_float<T>(to_float(x[(size_t)t * x_stride + i]) * w);
}

// C[slot, :] = A[slot, :] W[e]^T for the tile's expert e; W is [experts, n, k] dense.  Tiles of 64 x 64 outputs, 4 x 4 per thread, every
// output one sequential chain of fused multiply-adds over k = 0..K-1 in float, whatever the element type.
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const T* __restrict__ a, const T* __restrict__ w, T* __restrict__ c, const int* __restrict__ tile_expert,
                                                       int pad, int n, int k) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    const int expert = tile_expert[row0 / pad];
    if (expert < 0) return;
    const T* we = w + (size_t)expert * n * k;
    const int ty = tid / 16, tx = tid % 16;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < k; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int kk = k0 + lk + e;
            const int wr = col0 + lrow;
            as[lk + e][lrow] = kk < k ? to_float(a[(size_t)(row0 + lrow) * k + kk]) : 0.f;
            ws[lk + e][lrow] = (wr < n && kk < k) ? to_float(we[(size_t)wr * k + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = as[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wv[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = row0 + ty * TM + i;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int col = col0 + tx * TN + j;
            if (col < n) c[(size_t)r * n + col] = from_float<T>(acc[i][j]);
        }
    }
}

// The two above for bfloat16 rows that are whole 16-byte pieces: eight values per thread and access.
__global__ void moe_gather_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, int x_stride, const int* __restrict__ slot_token,
                                         const float* __restrict__ slot_weight, __nv_bfloat16* __restrict__ out, int hidden) {
    const int slot = blockIdx.x, t = slot_token[slot];
    if (t < 0) return;
    const float w = slot_weight[slot];
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)t * x_stride + i);
        const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint4 packed;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(in[j]);
            o[j] = __floats2bfloat162_rn(f.x * w, f.y * w);
        }
        *reinterpret_cast<uint4*>(out + (size_t)slot * hidden + i) = packed;
    }
}

__global__ void moe_combine_bf16x8_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ slot_of, int top,
                                          const __nv_bfloat16* __restrict__ base, __nv_bfloat16* __restrict__ out, int hidden) {
    const int t = blockIdx.x;
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
        float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (base) {
            const uint4 raw = *reinterpret_cast<const uint4*>(base + (size_t)t * hidden + i);
            const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(in[j]); sum[2 * j] = f.x; sum[2 * j + 1] = f.y; }
        }
        for (int k = 0; k < top; ++k) {
            const uint4 raw = *reinterpret_cast<const uint4*>(y + (size_t)slot_of[(size_t)t * top + k] * hidden + i);
            const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(in[j]); sum[2 * j] += f.x; sum[2 * j + 1] += f.y; }
        }
        uint4 packed;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(sum[2 * j], sum[2 * j + 1]);
        *reinterpret_cast<uint4*>(out + (size_t)t * hidden + i) = packed;
    }
}

template <typename TY, typename TB, typename TO>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ slot_of, int top, const TB* __restrict__ base, TO* __restrict__ out,
                                   int hidden) {
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float sum = base ? to_float(base[(size_t)t * hidden + i]) : 0.f;
        for (int k = 0; k < top; ++k) sum += to_float(y[(size_t)slot_of[(size_t)t * top + k] * hidden + i]);
        out[(size_t)t * hidden + i] = from_float<TO>(sum);
    }
}

// out[t] = sigmoid(base_gate[t]) * base[t] + sum_k w[t, k] * (slot_of[t, k] >= 0 ? y[slot] : x[t]), added in the order of the choices, in float.
template <typename T>
__global__ void moe_combine_weighted_kernel(const T* __restrict__ y, const int* __restrict__ slot_of, const float* __restrict__ weights, int top,
                                            const T* __restrict__ x, int x_stride, const T* __restrict__ base, const float* __restrict__ base_gate,
                                            T* __restrict__ out, int hidden) {
    const int t = blockIdx.x;
    const float share = base ? (base_gate ? 1.0f / (1.0f + expf(-base_gate[t])) : 1.f) : 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float sum = base ? share * to_float(base[(size_t)t * hidden + i]) : 0.f;
        for (int k = 0; k < top; ++k) {
            const int slot = slot_of[(size_t)t * top + k];
            const float v = slot >= 0 ? to_float(y[(size_t)slot * hidden + i]) : to_float(x[(size_t)t * x_stride + i]);
            sum = fmaf(weights[(size_t)t * top + k], v, sum);
        }
        out[(size_t)t * hidden + i] = from_float<T>(sum);
    }
}

// The same for bfloat16 rows that are whole 16-byte pieces: eight values per thread and access.
__global__ void moe_combine_weighted_bf16x8_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ slot_of, const float* __restrict__ weights,
                                                   int top, const __nv_bfloat16* __restrict__ x, int x_stride, const __nv_bfloat16* __restrict__ base,
                                                   const float* __restrict__ base_gate, __nv_bfloat16* __restrict__ out, int hidden) {
    const int t = blockIdx.x;
    const float share = base ? (base_gate ? 1.0f / (1.0f + expf(-base_gate[t])) : 1.f) : 0.f;
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
        float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (base) {
            const uint4 raw = *reinterpret_cast<const uint4*>(base + (size_t)t * hidden + i);
            const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(in[j]); sum[2 * j] = share * f.x; sum[2 * j + 1] = share * f.y; }
        }
        for (int k = 0; k < top; ++k) {
            const int slot = slot_of[(size_t)t * top + k];
            const float w = weights[(size_t)t * top + k];
            const uint4 raw = *reinterpret_cast<const uint4*>(slot >= 0 ? y + (size_t)slot * hidden + i : x + (size_t)t * x_stride + i);
            const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(in[j]); sum[2 * j] = fmaf(w, f.x, sum[2 * j]); sum[2 * j + 1] = fmaf(w, f.y, sum[2 * j + 1]); }
        }
        uint4 packed;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(sum[2 * j], sum[2 * j + 1]);
        *reinterpret_cast<uint4*>(out + (size_t)t * hidden + i) = packed;
    }
}
}  // namespace

HB_EXPORT int hb_moe_route_scored(const void* x, int is_bf16, int x_stride, const float* router, const float* correction, int tokens, int hidden,
                                  int outputs, int top, int group_count, int group_keep, float scale, int* chosen, float* weights, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (outputs <= 0 || outputs > 1024 || top <= 0 || top > outputs || hidden <= 0) return HB_UNSUPPORTED_SIZE;
    if (group_count > 1 && (outputs % group_count || group_keep <= 0 || group_keep > group_count || top > group_keep * (outputs / group_count)))
        return HB_BAD_ARGUMENT;
    const size_t shared = (size_t)(((hidden + 3) & ~3) + 4 * outputs + 2 * (group_count > 0 ? group_count : 1)) * sizeof(float);
    if (shared > 200 * 1024) return HB_UNSUPPORTED_SIZE;
    if (is_bf16) {
        if (shared > 48 * 1024) cudaFuncSetAttribute(moe_route_scored_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        moe_route_scored_kernel<<<tokens, ROUTE_THREADS, shared, stream>>>((const __nv_bfloat16*)x, x_stride, router, correction, hidden, outputs, top,
                                                                          group_count, group_keep, scale, chosen, weights);
    } else {
        if (shared > 48 * 1024) cudaFuncSetAttribute(moe_route_scored_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        moe_route_scored_kernel<<<tokens, ROUTE_THREADS, shared, stream>>>((const float*)x, x_stride, router, correction, hidden, outputs, top, group_count,
                                                                          group_keep, scale, chosen, weights);
    }
    return launch_status();
}

// y [capacity, hidden], x [tokens, x_stride] (what the feed-forward read), base [tokens, hidden] (optional, with an optional gate per token)
// and out [tokens, hidden] share an element type; weights [tokens, top] float.
HB_EXPORT int hb_moe_combine_weighted(const void* y, const int* slot_of, const float* weights, int top, const void* x, int x_stride, const void* base,
                                      const float* base_gate, void* out, int is_bf16, int tokens, int hidden, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (!weights || !x || top <= 0) return HB_BAD_ARGUMENT;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (is_bf16 && hidden % 8 == 0 && x_stride % 8 == 0 && (((uintptr_t)y | (uintptr_t)x | (uintptr_t)base | (uintptr_t)out) & 15) == 0) {
        moe_combine_weighted_bf16x8_kernel<<<tokens, hidden >= 2048 ? 256 : 128, 0, stream>>>((const __nv_bfloat16*)y, slot_of, weights, top, (const __nv_bfloat16*)x,
                                                                                             x_stride, (const __nv_bfloat16*)base, base_gate, (__nv_bfloat16*)out, hidden);
        return launch_status();
    }
    if (is_bf16)
        moe_combine_weighted_kernel<<<tokens, threads, 0, stream>>>((const __nv_bfloat16*)y, slot_of, weights, top, (const __nv_bfloat16*)x, x_stride,
                                                                    (const __nv_bfloat16*)base, base_gate, (__nv_bfloat16*)out, hidden);
    else
        moe_combine_weighted_kernel<<<tokens, threads, 0, stream>>>((const float*)y, slot_of, weights, top, (const float*)x, x_stride, (const float*)base,
                                                                    base_gate, (float*)out, hidden);
    return launch_status();
}

HB_EXPORT int hb_moe_route(const void* x, int is_bf16, int x_stride, const float* router, int tokens, int hidden, int experts, int top, int weighted,
                           int* chosen, float* weights, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (experts <= 0 || experts > 1024 || top <= 0 || top > experts || hidden <= 0) return HB_UNSUPPORTED_SIZE;
    const size_t shared = (size_t)(((hidden + 3) & ~3) + experts) * sizeof(float);
    if (shared > 200 * 1024) return HB_UNSUPPORTED_SIZE;
    if (is_bf16) {
        if (shared > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        moe_route_kernel<<<tokens, ROUTE_THREADS, shared, stream>>>((const __nv_bfloat16*)x, x_stride, router, hidden, experts, top, weighted, chosen, weights);
    } else {
        if (shared > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        moe_route_kernel<<<tokens, ROUTE_THREADS, shared, stream>>>((const float*)x, x_stride, router, hidden, experts, top, weighted, chosen, weights);
    }
    return launch_status();
}

// capacity: a multiple of pad, at least pairs + experts * (pad - 1) rounded up to it.  tile_expert and tile_rows (the real rows at the start
// of a tile) have capacity / pad entries.
HB_EXPORT int hb_moe_plan(const int* chosen, const float* weights, int pairs, int top, int experts, int pad, int capacity, int* slot_of,
                          int* slot_token, float* slot_weight, int* tile_expert, int* tile_rows, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (experts <= 0 || experts > 1024 || pad <= 0 || capacity % pad || top <= 0) return HB_UNSUPPORTED_SIZE;
    if ((long long)capacity < (long long)pairs + (long long)experts * (pad - 1)) return HB_BAD_ARGUMENT;
    moe_plan_kernel<<<1, PLAN_THREADS, 0, stream>>>(chosen, weights, pairs, top, experts, pad, capacity, slot_of, slot_token, slot_weight, tile_expert, tile_rows);
    return launch_status();
}

HB_EXPORT int hb_moe_gather(const void* x, int is_bf16, int x_stride, const int* slot_token, const float* slot_weight, void* out, int capacity,
                            int hidden, cudaStream_t stream) {
    if (capacity <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (is_bf16 && hidden % 8 == 0 && x_stride % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
        moe_gather_bf16x8_kernel<<<capacity, hidden >= 2048 ? 256 : 128, 0, stream>>>((const __nv_bfloat16*)x, x_stride, slot_token, slot_weight,
                                                                                     (__nv_bfloat16*)out, hidden);
        return launch_status();
    }
    if (is_bf16) moe_gather_kernel<<<capacity, threads, 0, stream>>>((const __nv_bfloat16*)x, x_stride, slot_token, slot_weight, (__nv_bfloat16*)out, hidden);
    else moe_gather_kernel<<<capacity, threads, 0, stream>>>((const float*)x, x_stride, slot_token, slot_weight, (float*)out, hidden);
    return launch_status();
}

// a [capacity, k] and c [capacity, n] dense, w [experts, n, k] dense; pad a multiple of 64.
HB_EXPORT int hb_moe_gemm(const void* a, const void* w, void* c, int is_bf16, const int* tile_expert, int pad, int capacity, int n, int k,
                          cudaStream_t stream) {
    if (capacity <= 0 || n <= 0) return 0;
    if (k <= 0 || pad % BM || capacity % pad) return HB_BAD_ARGUMENT;
    const dim3 grid((n + BN - 1) / BN, capacity / BM);
    if (grid.y > 65535) return HB_UNSUPPORTED_SIZE;
    if (is_bf16) moe_gemm_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)c, tile_expert, pad, n, k);
    else moe_gemm_kernel<<<grid, 256, 0, stream>>>((const float*)a, (const float*)w, (float*)c, tile_expert, pad, n, k);
    return launch_status();
}

// y [capacity, hidden] and base [tokens, hidden] (optional) in the activation type; out in the same type.
HB_EXPORT int hb_moe_combine(const void* y, const int* slot_of, int top, const void* base, void* out, int is_bf16, int tokens, int hidden,
                             cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (is_bf16 && hidden % 8 == 0 && (((uintptr_t)y | (uintptr_t)base | (uintptr_t)out) & 15) == 0) {
        moe_combine_bf16x8_kernel<<<tokens, hidden >= 2048 ? 256 : 128, 0, stream>>>((const __nv_bfloat16*)y, slot_of, top, (const __nv_bfloat16*)base,
                                                                                    (__nv_bfloat16*)out, hidden);
        return launch_status();
    }
    if (is_bf16)
        moe_combine_kernel<<<tokens, threads, 0, stream>>>((const __nv_bfloat16*)y, slot_of, top, (const __nv_bfloat16*)base, (__nv_bfloat16*)out, hidden);
    else
        moe_combine_kernel<<<tokens, threads, 0, stream>>>((const float*)y, slot_of, top, (const float*)base, (float*)out, hidden);
    return launch_status();
}
